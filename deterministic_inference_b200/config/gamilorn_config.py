"""Typed configuration of the Gamilorn design, read from the keys of its config.json.

A decoder with a learned position vector added to the token embedding, a residual stream in
float32, pre-norm layers (RMSNorm with weights stored around zero) whose mixer is two mixers
side by side on the same input -- grouped-query attention without a softmax (sigmoid weights,
a sliding window that keeps the first tokens, values of another size than keys, biases) and a
generalised delta rule with a matrix state per head -- an optional dense feed-forward with
the xIELU activation, and soft-capped logits.

config.json keys: ``architecture``, ``vocab``, ``width``, ``max_positions``, ``norm.eps``,
``logit_softcap`` and ``layers``: per layer ``type`` ("parallel"), ``mixer`` (``left``:
``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``mask.size``, ``mask.keep_first``;
``right``: ``heads``, ``dim``; ``left_scale``, ``right_scale``) and ``mlp`` (``kind`` "dense"
with ``ff``, or null).  The rank of the delta rule's decay map is the one size config.json
does not give; it is read from the shape of the checkpoint's tensor (``from_json``), or from
an optional ``right.decay_rank`` (configurations made in code).  Tensor names: ``embed``,
``pos``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.left.*``, ``l<i>.mix.right.*``,
``l<i>.mlp.*``, ``final.norm``, ``head``.
"""

from __future__ import annotations

import copy
import json
from dataclasses import dataclass
from pathlib import Path

from ..parts.spec import LayerSpec, ModelPlan, PartSpec, ScheduleEntry
from .model_config import ConfigError

def _positive(what: str, v) -> int:
    if not isinstance(v, int) or isinstance(v, bool) or v < 1:
        raise ConfigError(f"{what} must be a positive integer, got {v!r}")
    return v


@dataclass(frozen=True)
class GamilornConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    logit_softcap: float
    layers: tuple                 # the ``layers`` list of config.json, each with right.decay_rank filled in
    architecture: str = "Gamilorn"

    # ---- construction -----------------------------------------------------

    @classmethod
    def from_dict(cls, cfg: dict, decay_ranks=None) -> "GamilornConfig":
        """``decay_ranks``: per layer the rank found in the checkpoint (or None)."""
        missing = [k for k in ("vocab", "width", "max_positions", "norm", "logit_softcap", "layers")
                   if k not in cfg]
        if missing:
            raise ConfigError(f"config.json lacks required keys: {missing}")
        if not isinstance(cfg["norm"], dict) or "eps" not in cfg["norm"]:
            raise ConfigError("config.json: norm.eps is missing")
        layers = copy.deepcopy(list(cfg["layers"]))
        if not layers:
            raise ConfigError("config.json lists no layers")
        for i, layer in enumerate(layers):
            if layer.get("type") != "parallel":
                raise ConfigError(f"layer {i}: type {layer.get('type')!r} is not known (only 'parallel')")
            mixer = layer.get("mixer") or {}
            for k in ("left", "right", "left_scale", "right_scale"):
                if k not in mixer:
                    raise ConfigError(f"layer {i}: mixer.{k} is missing")
            left, right = mixer["left"], mixer["right"]
            for k in ("heads", "kv_heads", "dim", "vdim"):
                _positive(f"layer {i}: left.{k}", left.get(k))
            if left["heads"] % left["kv_heads"]:
                raise ConfigError(f"layer {i}: left.heads {left['heads']} is not a multiple of kv_heads "
                                  f"{left['kv_heads']}")
            if "scale" not in left:
                raise ConfigError(f"layer {i}: left.scale is missing")
            mask = left.get("mask") or {}
            _positive(f"layer {i}: left.mask.size", mask.get("size"))
            if not isinstance(mask.get("keep_first", 0), int) or mask.get("keep_first", 0) < 0:
                raise ConfigError(f"layer {i}: left.mask.keep_first must be a non-negative integer")
            for k in ("heads", "dim"):
                _positive(f"layer {i}: right.{k}", right.get(k))
            rank = None if decay_ranks is None else decay_ranks[i]
            if rank is None:
                rank = right.get("decay_rank")
            if rank is None:
                raise ConfigError(f"layer {i}: the rank of the decay map is not known: no checkpoint tensor "
                                  "to read it from and no right.decay_rank")
            right["decay_rank"] = _positive(f"layer {i}: right.decay_rank", int(rank))
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind") != "dense":
                    raise ConfigError(f"layer {i}: mlp.kind {mlp.get('kind')!r} is not known (only 'dense')")
                _positive(f"layer {i}: mlp.ff", mlp.get("ff"))
        out = cls(vocab=_positive("vocab", cfg["vocab"]), width=_positive("width", cfg["width"]),
                  max_positions=_positive("max_positions", cfg["max_positions"]),
                  norm_eps=float(cfg["norm"]["eps"]), logit_softcap=float(cfg["logit_softcap"]),
                  layers=tuple(layers), architecture=str(cfg.get("architecture", "Gamilorn")))
        if out.norm_eps <= 0 or out.logit_softcap <= 0:
            raise ConfigError("norm.eps and logit_softcap must be positive")
        return out

    @classmethod
    def from_json(cls, model_dir) -> "GamilornConfig":
        from ..weights.loader import read_header

        model_dir = Path(model_dir)
        cfg = json.loads((model_dir / "config.json").read_text())
        shapes = {}
        for f in sorted(model_dir.glob("*.safetensors")):
            for name, meta in read_header(f).items():
                shapes[name] = meta["shape"]
        ranks = []
        for i in range(len(cfg.get("layers", []))):
            shape = shapes.get(f"l{i}.mix.right.w1")
            ranks.append(int(shape[0]) if shape else None)
        return cls.from_dict(cfg, ranks)

    def to_dict(self) -> dict:
        """The config.json content that ``from_dict`` reads back unchanged."""
        return {"architecture": self.architecture, "layers": copy.deepcopy(list(self.layers)),
                "logit_softcap": self.logit_softcap, "max_positions": self.max_positions,
                "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}

    def validate(self) -> None:
        GamilornConfig.from_dict(self.to_dict())

    # ---- derived -----------------------------------------------------------

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    def num_parameters(self) -> int:
        w = self.width
        n = self.vocab * w * 2 + self.max_positions * w + w
        for layer in self.layers:
            left, right = layer["mixer"]["left"], layer["mixer"]["right"]
            q, k, v = left["heads"] * left["dim"], left["kv_heads"] * left["dim"], left["kv_heads"] * left["vdim"]
            n += (q + k + v) * (w + 1) + left["heads"] + left["heads"] * left["vdim"] * w
            hd = right["heads"] * right["dim"]
            n += 5 * hd * w + hd * w + right["decay_rank"] * (w + hd) + 3 * hd
            n += 2 * w
            if layer.get("mlp") is not None:
                n += 2 * layer["mlp"]["ff"] * w + 2
        return n

    # ---- the plan ------------------------------------------------------------

    def plan(self) -> ModelPlan:
        w = self.width
        norm = dict(size=w, eps=self.norm_eps, weight_offset=1.0)
        layers = []
        ignored = []
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            left, right = layer["mixer"]["left"], layer["mixer"]["right"]
            left_spec = PartSpec("sigmoid_attention", dict(
                prefix=p + "mix.left.", hidden_size=w, num_heads=left["heads"], num_kv_heads=left["kv_heads"],
                head_dim=left["dim"], v_head_dim=left["vdim"], scale=float(left["scale"]),
                window=left["mask"]["size"], keep_first=left["mask"].get("keep_first", 0)))
            right_spec = PartSpec("delta_rule", dict(
                prefix=p + "mix.right.", hidden_size=w, num_heads=right["heads"], head_dim=right["dim"],
                decay_rank=right["decay_rank"], norm_eps=self.norm_eps))
            mlp = layer.get("mlp")
            if mlp is None:
                ff, ff_norm = PartSpec("none", {}), PartSpec("none", {})
                ignored.append(p + "norm2")
            else:
                ff = PartSpec("dense_mlp", dict(prefix=p + "mlp.", hidden_size=w, intermediate_size=mlp["ff"],
                                                activation="xielu"))
                ff_norm = PartSpec("stream_rms_norm", dict(name=p + "norm2", **norm))
            layers.append(LayerSpec(
                block=PartSpec("pre_norm_f32_stream", {}),
                mixer=PartSpec("parallel", dict(
                    branches=[left_spec, right_spec],
                    scales=[float(layer["mixer"]["left_scale"]), float(layer["mixer"]["right_scale"])])),
                feed_forward=ff,
                mixer_norm=PartSpec("stream_rms_norm", dict(name=p + "norm1", **norm)),
                feed_forward_norm=ff_norm))
        return ModelPlan(
            hidden_size=w, vocab_size=self.vocab,
            embedding=PartSpec("token_position_embedding", dict(
                name="embed", position_name="pos", vocab_size=self.vocab, hidden_size=w,
                max_positions=self.max_positions)),
            head=PartSpec("linear_head", dict(name="head", vocab_size=self.vocab, hidden_size=w,
                                              softcap=self.logit_softcap)),
            final_norm=PartSpec("stream_rms_norm", dict(name="final.norm", **norm)),
            layers=tuple(layers),
            schedule=tuple(ScheduleEntry(layer=i, cache=i, writes_cache=True) for i in range(len(layers))),
            max_positions=self.max_positions,
            eos_token_ids=(),
            ignored_names=tuple(ignored),
        )
