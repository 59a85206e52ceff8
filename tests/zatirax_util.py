"""Tiny Zatirax models for the tests: configurations that differ in every size and option (also
in values that may happen to be equal or 1 elsewhere: one key/value head or as many as query heads,
key and value sizes equal or not, a full or a partial rotation, stretched frequencies or not, a loop
in the middle, over everything, of one pass, or none, a layer without a feed-forward, masks shorter
than a page and longer than any prompt), written with random weights by the package's writer and
then rescaled so that every mechanism weighs in the logits: scores of unit size, sinks that take a
visible share, pass vectors and limits that bite."""

from __future__ import annotations

import math
from pathlib import Path

import torch


def attention(heads, kv_heads, dim, vdim, chunk, rot_dims, base, scaling=None, scale=None, ff=None, limit=1.0):
    rot = {"base": base, "dims": rot_dims}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": chunk},
                      "rot": rot, "scale": scale if scale is not None else 1.0 / math.sqrt(dim)},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff, "limit": limit}}


def latent(heads, dim, rot_dim, vdim, rank, window, base, scale=None, ff=None, limit=1.0):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank,
                      "mask": {"size": window}, "rot": {"base": base, "dims": rot_dim},
                      "scale": scale if scale is not None else 1.0 / math.sqrt(dim + rot_dim)},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff, "limit": limit}}


CONFIGS = {
    # a loop in the middle (three passes over two unlike layers), a layer without a feed-forward
    "z1": dict(page_size=16, seed=41, config={
        "architecture": "Zatirax", "vocab": 150, "width": 64, "norm": {"eps": 2e-5}, "embedding": {"scale": 3.0},
        "loop": {"start": 1, "stop": 3, "times": 3},
        "layers": [latent(2, 16, 8, 24, 32, 11, 5000.0, ff=96, limit=0.7),
                   attention(4, 2, 16, 24, 16, 8, 300.0, scaling=(4.0, 1.0, 3.0, 64), ff=None),
                   attention(3, 1, 32, 16, 13, 32, 10000.0, ff=80, limit=1.5),
                   latent(3, 8, 4, 8, 16, 40, 100.0, ff=72, limit=0.9)]}),
    # no loop; masks no prompt reaches; one head of everything; pages of 32
    "z2": dict(page_size=32, seed=42, config={
        "architecture": "Zatirax", "vocab": 300, "width": 96, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
        "layers": [attention(1, 1, 48, 48, 4096, 16, 20000.0, scaling=(8.0, 1.0, 4.0, 128), ff=128, limit=2.0),
                   latent(1, 32, 16, 40, 24, 4096, 10000.0, ff=None)]}),
    # the loop is the whole model; masks shorter than a page; sizes that are multiples of nothing; pages of 8
    "z3": dict(page_size=8, seed=43, config={
        "architecture": "Zatirax", "vocab": 131, "width": 100, "norm": {"eps": 1e-5}, "embedding": {"scale": 7.5},
        "loop": {"start": 0, "stop": 2, "times": 2},
        "layers": [attention(6, 3, 20, 12, 7, 10, 777.0, scaling=(2.0, 0.5, 2.0, 32), ff=50, limit=0.5),
                   latent(5, 12, 6, 18, 21, 5, 50.0, ff=30, limit=1.2)]}),
    # sizes the tensor-core kernels take; a loop of one pass; masks that end inside a page
    "z4": dict(page_size=16, seed=44, config={
        "architecture": "Zatirax", "vocab": 211, "width": 128, "norm": {"eps": 1e-5}, "embedding": {"scale": 5.0},
        "loop": {"start": 1, "stop": 2, "times": 1},
        "layers": [attention(4, 2, 64, 64, 72, 32, 10000.0, scaling=(8.0, 1.0, 4.0, 64), ff=192, limit=1.0),
                   latent(4, 32, 32, 32, 64, 41, 10000.0, ff=192, limit=1.0),
                   attention(2, 2, 128, 128, 100, 64, 500.0, ff=None)]}),
    # five layers in another order, a loop over the middle three, grouped heads on the tensor-core kernels,
    # windows and chunks of whole pages
    "z5": dict(page_size=16, seed=45, config={
        "architecture": "Zatirax", "vocab": 512, "width": 256, "norm": {"eps": 1e-6}, "embedding": {"scale": 10.0},
        "loop": {"start": 1, "stop": 4, "times": 2},
        "layers": [latent(8, 32, 16, 32, 128, 64, 30000.0, ff=384, limit=1.0),
                   attention(8, 2, 64, 64, 128, 32, 10000.0, scaling=(8.0, 1.0, 4.0, 256), ff=384, limit=2.0),
                   attention(8, 4, 64, 64, 64, 16, 40000.0, ff=None),
                   latent(4, 64, 32, 64, 64, 128, 10000.0, ff=256, limit=0.8),
                   attention(4, 4, 128, 128, 96, 32, 20000.0, scaling=(4.0, 1.0, 2.0, 128), ff=384, limit=1.0)]}),
}


def sharpen(model_dir) -> None:
    from safetensors.torch import load_file, save_file

    path = Path(model_dir) / "model.safetensors"
    tensors = load_file(str(path))

    def unit(t, gain):      # a matrix drawn with std 0.02 -> std gain / sqrt(inputs)
        return t.float() * (gain / (0.02 * math.sqrt(t.shape[-1])))

    for name, t in list(tensors.items()):
        end = name.split(".", 1)[-1] if name.startswith("l") and name[1].isdigit() else name
        x = None
        if name == "embed":
            x = t.float() * 50.0
        elif name == "head":
            x = unit(t, 3.0)
        elif name == "loop.step":
            x = t.float() * 40.0
        elif end in ("mix.q", "mix.uk"):
            x = unit(t, 1.8)
        elif end in ("mix.k", "mix.v", "mix.g", "mix.o", "mix.dkv", "mix.uv", "mlp.gate", "mlp.up", "mlp.down"):
            x = unit(t, 1.2)
        elif end == "mix.sink":
            x = 0.5 + t.float() * 40.0
        if x is not None:
            tensors[name] = x.to(t.dtype)
    save_file(tensors, str(path), metadata={"format": "pt"})


def write_tiny(name: str, out_dir) -> Path:
    from deterministic_inference_b200.config.zatirax_config import ZatiraxConfig
    from deterministic_inference_b200.weights import write_random_model

    spec = CONFIGS[name]
    write_random_model(ZatiraxConfig.from_dict(spec["config"]), spec["seed"], out_dir)
    sharpen(out_dir)
    return Path(out_dir)


def requests(vocab: int, lens, seed: int):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lens]
