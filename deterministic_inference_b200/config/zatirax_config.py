"""Typed configuration of the Zatirax design, read from the keys of its config.json.

A decoder with a scaled token embedding, a residual stream in float32, layers with an RMS norm in
front of and behind each sublayer, two kinds of mixer in any order -- grouped-query softmax attention
with q/k norm, partial rotation with stretched frequencies, a chunked mask, a sink in the softmax and a
sigmoid output gate ("attention"), and latent attention with a sliding window ("latent_attention") -- a
gated feed-forward with limited inputs, and a run of layers that is repeated with the same weights, a
learned vector added to the stream before each pass, each pass with caches of its own.

config.json keys: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``, ``loop``
(``start``, ``stop``, ``times``; optional) and ``layers``: per layer ``type``, ``mixer`` (attention:
``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``mask.size``, ``rot.base``, ``rot.dims``,
``rot.scaling``; latent_attention: ``heads``, ``dim``, ``rot_dim``, ``vdim``, ``kv_rank``, ``scale``,
``mask.size``, ``rot.base``, ``rot.dims``) and ``mlp`` (``kind`` "dense" with ``ff`` and ``limit``, or
null).  ``max_positions`` is optional (no part of the design needs a longest position; it bounds the
engine's block tables).  Tensor names: ``embed``, ``loop.step``, ``l<i>.norm1``, ``l<i>.norm1b``,
``l<i>.norm2``, ``l<i>.norm2b``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""

from __future__ import annotations

import copy
import json
from dataclasses import dataclass
from pathlib import Path
from typing import Optional

from ..parts.spec import LayerSpec, ModelPlan, PartSpec, ScheduleEntry
from .model_config import ConfigError

SWISH_ALPHA = 1.702          # the feed-forward's gate is g * sigmoid(1.702 g): fixed by the design
DEFAULT_MAX_POSITIONS = 1 << 20


def _positive(what: str, v) -> int:
    if not isinstance(v, int) or isinstance(v, bool) or v < 1:
        raise ConfigError(f"{what} must be a positive integer, got {v!r}")
    return v


def _rot(what: str, mixer: dict, size: int) -> dict:
    rot = mixer.get("rot")
    if not isinstance(rot, dict) or "base" not in rot or "dims" not in rot:
        raise ConfigError(f"{what}: rot.base and rot.dims are needed")
    dims = _positive(f"{what}: rot.dims", rot["dims"])
    if dims % 2 or dims > size:
        raise ConfigError(f"{what}: rot.dims {dims} must be even and at most {size}")
    if float(rot["base"]) <= 0:
        raise ConfigError(f"{what}: rot.base must be positive")
    sc = rot.get("scaling")
    if sc is not None:
        missing = [k for k in ("factor", "low", "high", "original") if k not in sc]
        if missing:
            raise ConfigError(f"{what}: rot.scaling lacks {missing}")
        if float(sc["high"]) <= float(sc["low"]) or float(sc["factor"]) <= 0 or float(sc["original"]) <= 0:
            raise ConfigError(f"{what}: rot.scaling needs high > low and positive factor and original")
    return rot


@dataclass(frozen=True)
class ZatiraxConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    layers: tuple                  # the ``layers`` list of config.json
    loop: Optional[tuple] = None   # (start, stop, times) or None
    max_positions: int = DEFAULT_MAX_POSITIONS
    architecture: str = "Zatirax"

    # ---- construction -----------------------------------------------------

    @classmethod
    def from_dict(cls, cfg: dict) -> "ZatiraxConfig":
        missing = [k for k in ("vocab", "width", "norm", "embedding", "layers") if k not in cfg]
        if missing:
            raise ConfigError(f"config.json lacks required keys: {missing}")
        if not isinstance(cfg["norm"], dict) or "eps" not in cfg["norm"]:
            raise ConfigError("config.json: norm.eps is missing")
        if not isinstance(cfg["embedding"], dict) or "scale" not in cfg["embedding"]:
            raise ConfigError("config.json: embedding.scale is missing")
        layers = copy.deepcopy(list(cfg["layers"]))
        if not layers:
            raise ConfigError("config.json lists no layers")
        for i, layer in enumerate(layers):
            kind, mixer = layer.get("type"), layer.get("mixer") or {}
            what = f"layer {i}"
            if kind == "attention":
                for k in ("heads", "kv_heads", "dim", "vdim"):
                    _positive(f"{what}: mixer.{k}", mixer.get(k))
                if mixer["heads"] % mixer["kv_heads"]:
                    raise ConfigError(f"{what}: heads {mixer['heads']} is not a multiple of kv_heads "
                                      f"{mixer['kv_heads']}")
                _rot(what, mixer, mixer["dim"])
            elif kind == "latent_attention":
                for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"):
                    _positive(f"{what}: mixer.{k}", mixer.get(k))
                rot = _rot(what, mixer, mixer["rot_dim"])
                if rot["dims"] != mixer["rot_dim"]:
                    raise ConfigError(f"{what}: rot.dims {rot['dims']} differs from rot_dim {mixer['rot_dim']}")
            else:
                raise ConfigError(f"{what}: type {kind!r} is not known ('attention', 'latent_attention')")
            if "scale" not in mixer:
                raise ConfigError(f"{what}: mixer.scale is missing")
            _positive(f"{what}: mixer.mask.size", (mixer.get("mask") or {}).get("size"))
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind") != "dense":
                    raise ConfigError(f"{what}: mlp.kind {mlp.get('kind')!r} is not known (only 'dense')")
                _positive(f"{what}: mlp.ff", mlp.get("ff"))
                if "limit" not in mlp or float(mlp["limit"]) <= 0:
                    raise ConfigError(f"{what}: mlp.limit must be a positive number")
        loop = cfg.get("loop")
        if loop is not None:
            for k in ("start", "stop", "times"):
                if not isinstance(loop.get(k), int) or isinstance(loop.get(k), bool):
                    raise ConfigError(f"loop.{k} must be an integer")
            if not (0 <= loop["start"] <= loop["stop"] <= len(layers)) or loop["times"] < 1:
                raise ConfigError(f"loop {loop!r} does not fit {len(layers)} layers")
            loop = (loop["start"], loop["stop"], loop["times"])
        out = cls(vocab=_positive("vocab", cfg["vocab"]), width=_positive("width", cfg["width"]),
                  norm_eps=float(cfg["norm"]["eps"]), embedding_scale=float(cfg["embedding"]["scale"]),
                  layers=tuple(layers), loop=loop,
                  max_positions=_positive("max_positions", cfg.get("max_positions", DEFAULT_MAX_POSITIONS)),
                  architecture=str(cfg.get("architecture", "Zatirax")))
        if out.norm_eps <= 0:
            raise ConfigError("norm.eps must be positive")
        return out

    @classmethod
    def from_json(cls, model_dir) -> "ZatiraxConfig":
        return cls.from_dict(json.loads((Path(model_dir) / "config.json").read_text()))

    def to_dict(self) -> dict:
        """The config.json content that ``from_dict`` reads back unchanged."""
        d = {"architecture": self.architecture, "embedding": {"scale": self.embedding_scale},
             "layers": copy.deepcopy(list(self.layers)), "norm": {"eps": self.norm_eps},
             "vocab": self.vocab, "width": self.width}
        if self.loop is not None:
            d["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        return d

    def validate(self) -> None:
        ZatiraxConfig.from_dict(self.to_dict())

    # ---- derived -----------------------------------------------------------

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    def layer_runs(self) -> list:
        """(layer, pass or None) in the order the layers run: the layers before the loop, the looped
        ones ``times`` times in a row, the rest."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        start, stop, times = self.loop
        runs = [(i, None) for i in range(start)]
        for t in range(times):
            runs += [(i, t) for i in range(start, stop)]
        return runs + [(i, None) for i in range(stop, n)]

    def num_parameters(self) -> int:
        w = self.width
        n = 2 * self.vocab * w + w + (self.loop[2] * w if self.loop is not None else 0)
        for layer in self.layers:
            m = layer["mixer"]
            if layer["type"] == "attention":
                q, kv = m["heads"] * m["dim"], m["kv_heads"] * m["dim"]
                n += (q + kv + m["kv_heads"] * m["vdim"] + 2 * m["heads"] * m["vdim"]) * w + 2 * m["dim"] + m["heads"]
            else:
                n += (m["heads"] * (m["dim"] + m["rot_dim"]) + m["kv_rank"] + m["rot_dim"]) * w + m["kv_rank"]
                n += m["heads"] * (m["dim"] + m["vdim"]) * m["kv_rank"] + m["heads"] * m["vdim"] * w
            n += 2 * w
            if layer.get("mlp") is not None:
                n += 3 * layer["mlp"]["ff"] * w + 2 * w
        return n

    # ---- the plan ------------------------------------------------------------

    def plan(self) -> ModelPlan:
        w = self.width
        norm = dict(size=w, eps=self.norm_eps)
        layers, ignored = [], []
        for i, layer in enumerate(self.layers):
            p, m = f"l{i}.", layer["mixer"]
            rot = m["rot"]
            if layer["type"] == "attention":
                mixer = PartSpec("masked_attention", dict(
                    prefix=p + "mix.", hidden_size=w, num_heads=m["heads"], num_kv_heads=m["kv_heads"],
                    head_dim=m["dim"], v_head_dim=m["vdim"], scale=float(m["scale"]),
                    position_encoding=PartSpec("rope", dict(head_dim=m["dim"], rotary_dim=rot["dims"],
                                                            theta=float(rot["base"]), scaling=rot.get("scaling"))),
                    qk_norm_eps=self.norm_eps, mask="chunk", mask_size=m["mask"]["size"], sink=True, gate=True))
            else:
                mixer = PartSpec("latent_attention", dict(
                    prefix=p + "mix.", hidden_size=w, num_heads=m["heads"], head_dim=m["dim"],
                    rot_dim=m["rot_dim"], v_head_dim=m["vdim"], kv_rank=m["kv_rank"], scale=float(m["scale"]),
                    position_encoding=PartSpec("rope", dict(head_dim=m["rot_dim"], rotary_dim=rot["dims"],
                                                            theta=float(rot["base"]), scaling=rot.get("scaling"))),
                    norm_eps=self.norm_eps, mask="window", mask_size=m["mask"]["size"]))
            mlp = layer.get("mlp")
            if mlp is None:
                ff, ff_norm = PartSpec("none", {}), PartSpec("none", {})
                ff_post = PartSpec("none", {})
                ignored += [p + "norm2", p + "norm2b"]
            else:
                ff = PartSpec("gated_mlp", dict(prefix=p + "mlp.", hidden_size=w, intermediate_size=mlp["ff"],
                                                activation="limited_swish", limit=float(mlp["limit"]),
                                                alpha=SWISH_ALPHA, names=("gate", "up", "down")))
                ff_norm = PartSpec("stream_rms_norm", dict(name=p + "norm2", **norm))
                ff_post = PartSpec("stream_post_norm", dict(name=p + "norm2b", **norm))
            layers.append(LayerSpec(
                block=PartSpec("sandwich_f32_stream", dict(
                    mixer_post_norm=PartSpec("stream_post_norm", dict(name=p + "norm1b", **norm)),
                    feed_forward_post_norm=ff_post)),
                mixer=mixer, feed_forward=ff,
                mixer_norm=PartSpec("stream_rms_norm", dict(name=p + "norm1", **norm)),
                feed_forward_norm=ff_norm))
        # every run of a layer has a cache of its own; a pass's first layer adds the pass's vector
        schedule = []
        for cache_id, (i, t) in enumerate(self.layer_runs()):
            enters = t if (t is not None and i == self.loop[0]) else None
            schedule.append(ScheduleEntry(layer=i, cache=cache_id, writes_cache=True, enter_vector=enters))
        looped = self.loop is not None and self.loop[1] > self.loop[0]
        if not looped:
            ignored.append("loop.step")       # (nothing is looped: the vectors, if stored, are not used)
        return ModelPlan(
            hidden_size=w, vocab_size=self.vocab,
            embedding=PartSpec("scaled_token_embedding", dict(name="embed", vocab_size=self.vocab, hidden_size=w,
                                                              scale=self.embedding_scale)),
            head=PartSpec("linear_head", dict(name="head", vocab_size=self.vocab, hidden_size=w)),
            final_norm=PartSpec("stream_rms_norm", dict(name="final.norm", **norm)),
            layers=tuple(layers), schedule=tuple(schedule),
            max_positions=self.max_positions, eos_token_ids=(),
            ignored_names=tuple(ignored),
            stream_addend=PartSpec("row_vectors", dict(name="loop.step", count=self.loop[2], hidden_size=w))
            if looped else None,
        )
