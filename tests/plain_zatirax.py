"""A plain, slow implementation of the Zatirax design: whole sequences, no cache, no batches,
float64 by default, one function per mechanism, written from the design's equations.  It
shares no code with the package; the tests compare the package with it.

Notation: n tokens, width W.  Softmax attention: H query heads, G key/value heads, key size D,
value size E.  Latent attention: H heads with D unrotated and R rotated query/key dimensions,
value size E, latent size C.
"""

from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch

DT = torch.float64


def read_model_dir(model_dir, dtype=DT):
    """(config dict, {name: tensor}) of a folder with config.json and model.safetensors."""
    model_dir = Path(model_dir)
    cfg = json.loads((model_dir / "config.json").read_text())
    raw = (model_dir / "model.safetensors").read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    data = raw[8 + n:]
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32}
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        a, b = meta["data_offsets"]
        t = torch.frombuffer(bytearray(data[a:b]), dtype=kinds[meta["dtype"]]).reshape(meta["shape"])
        out[name] = t.to(dtype) if t.is_floating_point() else t
    return cfg, out


# ---- one function per mechanism ------------------------------------------------------------

def rms_norm(x, w, eps):
    """x over its root mean square (eps inside the root), times the weight as stored."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def rotary_frequencies(dims, base, scaling=None):
    """f_i = base^(-2i/dims), i < dims/2; with ``scaling`` long wavelengths are stretched:
    wavelength below original/high: kept; above original/low: divided by factor; between: a
    blend that is linear in original/wavelength."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=DT)
    if scaling:
        factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
        out = []
        for fi in f.tolist():
            wl = 2 * math.pi / fi
            if wl < orig / high:
                out.append(fi)
            elif wl > orig / low:
                out.append(fi / factor)
            else:
                s = (orig / wl - low) / (high - low)
                out.append((1 - s) * fi / factor + s * fi)
        f = torch.tensor(out, dtype=DT)
    return f


def rotate(x, positions, freqs):
    """x [n, ..., D]: the first 2 * len(freqs) dimensions of the last axis are rotated, dimension
    i paired with i + len(freqs); the rest pass."""
    half = freqs.shape[0]
    a = positions.to(x.dtype)[:, None] * freqs.to(x.dtype)[None, :]          # [n, half]
    while a.dim() < x.dim():
        a = a.unsqueeze(1)
    cos, sin = torch.cos(a), torch.sin(a)
    u, v, rest = x[..., :half], x[..., half:2 * half], x[..., 2 * half:]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, rest], dim=-1)


def window_mask(n, size, offset=0):
    """query offset + i sees key j with 0 <= i' - j < size."""
    i = torch.arange(offset, offset + n)[:, None]
    j = torch.arange(offset + n)[None, :]
    return (j <= i) & (i - j < size)


def chunk_mask(n, size, offset=0):
    """query i sees key j <= i of its own chunk of ``size`` positions, chunks counted from 0."""
    i = torch.arange(offset, offset + n)[:, None]
    j = torch.arange(offset + n)[None, :]
    return (j <= i) & (i // size == j // size)


def softmax_attention(q, k, v, scale, mask, sink=None):
    """q [n, H, D], k [m, G, D], v [m, G, E], mask [n, m] -> [n, H, E].  ``sink`` [H]: the
    denominator also holds exp(sink_h), which has no value."""
    n, heads, _ = q.shape
    group = heads // k.shape[1]
    out = []
    for h in range(heads):
        g = h // group
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~mask, -math.inf)
        m = s.max(-1, keepdim=True).values
        if sink is not None:
            m = torch.maximum(m, sink[h].expand_as(m))
        e = torch.exp(s - m)
        den = e.sum(-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[h] - m)
        out.append((e / den) @ v[:, g])
    return torch.stack(out, dim=1)


def limited_gate(g, u, limit, alpha=1.702):
    """min(g, limit) * sigmoid(alpha * min(g, limit)) * (clamp(u, -limit, limit) + 1)."""
    g = torch.clamp(g, max=limit)
    u = torch.clamp(u, -limit, limit)
    return g * torch.sigmoid(alpha * g) * (u + 1)


# ---- the model ---------------------------------------------------------------------------------

def _keep(x):
    return x


def as_stored_bf16(x):
    """What a tensor is after a trip through bfloat16 storage."""
    return x.to(torch.bfloat16).to(x.dtype)


def gated_sink_attention(h, positions, w, p, c, eps, rnd=_keep):
    """The 'attention' mixer: q/k norm per head, partial rotation with stretched frequencies,
    chunked mask, softmax with a sink, sigmoid output gate."""
    n = h.shape[0]
    heads, groups, d, e = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = rnd(h @ w[p + "q"].T).view(n, heads, d)
    k = rnd(h @ w[p + "k"].T).view(n, groups, d)
    v = rnd(h @ w[p + "v"].T).view(n, groups, e)
    q = rms_norm(q, w[p + "q.norm"], eps)
    k = rms_norm(k, w[p + "k.norm"], eps)
    f = rotary_frequencies(c["rot"]["dims"], c["rot"]["base"], c["rot"].get("scaling"))
    q, k = rnd(rotate(q, positions, f)), rnd(rotate(k, positions, f))
    o = softmax_attention(q, k, v, c["scale"], chunk_mask(n, c["mask"]["size"]), w[p + "sink"])
    gate = torch.sigmoid(rnd(h @ w[p + "g"].T))
    return rnd(rnd(rnd(o).reshape(n, -1) * gate) @ w[p + "o"].T)


def latent_attention(h, positions, w, p, c, eps, rnd=_keep):
    """The 'latent_attention' mixer, with keys and values rebuilt from the latent for every token."""
    n = h.shape[0]
    heads, d, r, e, rank = c["heads"], c["dim"], c["rot_dim"], c["vdim"], c["kv_rank"]
    q = rnd(h @ w[p + "q"].T).view(n, heads, d + r)
    down = rnd(h @ w[p + "dkv"].T)
    latent = rnd(rms_norm(down[:, :rank], w[p + "dkv.norm"], eps))
    f = rotary_frequencies(c["rot"]["dims"], c["rot"]["base"], c["rot"].get("scaling"))
    k_rot = rnd(rotate(down[:, rank:], positions, f))                         # [n, R], shared by the heads
    q_rot = rnd(rotate(q[..., d:], positions, f))
    k_plain = rnd(latent @ w[p + "uk"].T).view(n, heads, d)
    v = rnd(latent @ w[p + "uv"].T).view(n, heads, e)
    qq = torch.cat([q[..., :d], q_rot], dim=-1)
    kk = torch.cat([k_plain, k_rot[:, None, :].expand(n, heads, r)], dim=-1)
    o = softmax_attention(qq, kk, v, c["scale"], window_mask(n, c["mask"]["size"]))
    return rnd(rnd(o).reshape(n, -1) @ w[p + "o"].T)


def feed_forward(h, w, p, c, rnd=_keep):
    g, u = h @ w[p + "gate"].T, h @ w[p + "up"].T
    return rnd(rnd(limited_gate(g, u, c["limit"])) @ w[p + "down"].T)


def layer_order(cfg):
    """(layer, pass or None) in the order they run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    out = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        out += [(i, t) for i in range(loop["start"], loop["stop"])]
    out += [(i, None) for i in range(loop["stop"], n)]
    return out


def forward(cfg, w, tokens, bf16_storage=False, return_layers=False):
    """Logits [n, vocab] of one whole sequence."""
    rnd = as_stored_bf16 if bf16_storage else _keep
    eps = cfg["norm"]["eps"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    n = tokens.shape[0]
    positions = torch.arange(n)
    x = w["embed"][tokens] * cfg["embedding"]["scale"]
    loop = cfg.get("loop")
    layers_out = []
    for i, t in layer_order(cfg):
        if t is not None and i == loop["start"]:
            x = x + w["loop.step"][t]
        layer, p = cfg["layers"][i], f"l{i}."
        h = rnd(rms_norm(x, w[p + "norm1"], eps))
        if layer["type"] == "attention":
            m = gated_sink_attention(h, positions, w, p + "mix.", layer["mixer"], eps, rnd)
        elif layer["type"] == "latent_attention":
            m = latent_attention(h, positions, w, p + "mix.", layer["mixer"], eps, rnd)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(m, w[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            h = rnd(rms_norm(x, w[p + "norm2"], eps))
            x = x + rms_norm(feed_forward(h, w, p + "mlp.", layer["mlp"], rnd), w[p + "norm2b"], eps)
        layers_out.append(x)
    logits = rnd(rms_norm(x, w["final.norm"], eps)) @ w["head"].T
    if return_layers:
        return logits, torch.stack(layers_out)
    return logits
