"""Tiny Gamilorn models for the tests: configurations that differ in every size and option
(also in values that may happen to be equal or 1 elsewhere: one key/value head, key and value
sizes equal or not, a window shorter than the kept first keys, no kept keys, a layer without
a feed-forward), written with random weights by the package's writer and then rescaled so that
every mechanism weighs in the logits: scores of unit size, selective sigmoid weights, decays
spread over (e^-0.61, 1), logits that reach the soft cap."""

from __future__ import annotations

import math
from pathlib import Path

import torch


def _layer(heads, kv_heads, dim, vdim, window, keep, scale, r_heads, r_dim, rank, ls, rs, ff):
    return {"type": "parallel",
            "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
                               "mask": {"size": window, "keep_first": keep}},
                      "left_scale": ls,
                      "right": {"heads": r_heads, "dim": r_dim, "decay_rank": rank},
                      "right_scale": rs},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


CONFIGS = {
    # three unlike layers; the last has more kept keys than its window is long
    "g1": dict(page_size=16, seed=21, config={
        "architecture": "Gamilorn", "vocab": 160, "width": 96, "max_positions": 512,
        "norm": {"eps": 2e-5}, "logit_softcap": 9.0,
        "layers": [_layer(4, 2, 16, 24, 12, 3, 0.25, 3, 16, 4, 0.9, 1.3, 128),
                   _layer(2, 2, 32, 32, 40, 0, 0.2, 2, 24, 8, 1.0, 0.5, None),
                   _layer(3, 1, 8, 40, 5, 9, 0.4, 1, 48, 3, 0.7, 1.1, 64)]}),
    # one layer, one head of everything, a window no prompt reaches, pages of 32
    "g2": dict(page_size=32, seed=22, config={
        "architecture": "Gamilorn", "vocab": 300, "width": 128, "max_positions": 1024,
        "norm": {"eps": 1e-6}, "logit_softcap": 30.0,
        "layers": [_layer(1, 1, 64, 64, 4096, 0, 0.125, 2, 64, 16, 1.0, 1.0, 200)]}),
    # heads of 128 in the recurrence, a window that ends inside a page, pages of 8
    "g3": dict(page_size=8, seed=23, config={
        "architecture": "Gamilorn", "vocab": 211, "width": 64, "max_positions": 700,
        "norm": {"eps": 1e-5}, "logit_softcap": 12.0,
        "layers": [_layer(8, 4, 24, 16, 21, 13, 0.2, 1, 128, 6, 1.1, 0.8, 96),
                   _layer(2, 1, 48, 56, 100, 1, 0.15, 4, 8, 2, 0.6, 1.4, None)]}),
    # sizes that are multiples of nothing: rows that start on no 16-byte border, key and value
    # sizes the tensor-core kernel does not take, state heads of 18 (copies of 4 bytes), rank 3
    "g4": dict(page_size=16, seed=24, config={
        "architecture": "Gamilorn", "vocab": 131, "width": 100, "max_positions": 300,
        "norm": {"eps": 1e-5}, "logit_softcap": 10.0,
        "layers": [_layer(3, 3, 24, 40, 9, 2, 0.2, 5, 18, 3, 1.0, 1.0, 50),
                   _layer(6, 2, 20, 12, 30, 7, 0.22, 2, 36, 5, 0.8, 0.9, None)]}),
}


def sharpen(model_dir) -> None:
    from safetensors.torch import load_file, save_file

    path = Path(model_dir) / "model.safetensors"
    tensors = load_file(str(path))
    g = torch.Generator().manual_seed(5)

    def unit(t, gain):      # a matrix drawn with std 0.02 -> std gain / sqrt(inputs)
        return t.float() * (gain / (0.02 * math.sqrt(t.shape[-1])))

    for name, t in list(tensors.items()):
        x = None
        end = name.split(".", 1)[-1] if name.startswith("l") else name
        if name in ("embed",):
            x = t.float() * 50.0
        elif name == "pos":
            x = t.float() * 25.0
        elif name == "head":
            x = unit(t, 3.0)
        elif end in ("mix.left.q", "mix.left.k"):
            x = unit(t, 1.6)
        elif end in ("mix.left.v", "mix.right.r", "mix.right.k", "mix.right.v", "mix.right.g", "mix.right.a",
                     "mix.right.w1", "mlp.up", "mlp.down", "mix.right.o"):
            x = unit(t, 1.0)
        elif end == "mix.left.o":
            x = unit(t, 0.7)
        elif end == "mix.right.w2":
            x = unit(t, 2.0)
        elif end in ("mix.left.q.b", "mix.left.k.b", "mix.left.v.b", "mix.right.a.b"):
            x = t.float() * 15.0
        elif end == "mix.right.w0":
            x = t.float() * 50.0
        elif end == "mix.left.pb":
            x = -1.5 + t.float() * 25.0
        elif end == "mlp.act":
            x = t.float() * 25.0
        elif "norm" in end and end != "mix.right.norm":
            x = t.float() * 5.0
        if x is not None:
            tensors[name] = x.to(t.dtype)
    save_file(tensors, str(path), metadata={"format": "pt"})


def write_tiny(name: str, out_dir) -> Path:
    from deterministic_inference_b200.config.gamilorn_config import GamilornConfig
    from deterministic_inference_b200.weights import write_random_model

    spec = CONFIGS[name]
    write_random_model(GamilornConfig.from_dict(spec["config"]), spec["seed"], out_dir)
    sharpen(out_dir)
    return Path(out_dir)


def requests(vocab: int, lens, seed: int):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lens]
