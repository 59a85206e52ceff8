"""A plain, slow implementation of the Gamilorn design: whole sequences, no cache, no batches,
float64 by default, one function per mechanism, written from the design's equations.  It
shares no code with the package; the tests compare the package with it.

Notation: n tokens, width W; for the attention branch H query heads, G key/value heads, key
size D, value size E; for the recurrent branch heads of size D with a state S [D, D].
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

def unit_rms(x, eps):
    """x over its root mean square, eps inside the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def zero_centred_norm(x, w, eps):
    """RMS norm whose stored weight is the distance from one."""
    return unit_rms(x, eps) * (1.0 + w)


def visible(n, window, keep_first, offset=0):
    """[n, offset + n] mask: query at position offset + i against key j."""
    i = torch.arange(offset, offset + n)[:, None]
    j = torch.arange(offset + n)[None, :]
    return (j <= i) & ((i - j < window) | (j < keep_first))


def sigmoid_window_attention(q, k, v, scale, head_bias, window, keep_first):
    """q [n, H, D], k [n, G, D], v [n, G, E] -> [n, H, E]; weights sigmoid(score + bias), not normalised."""
    n, heads, _ = q.shape
    group = heads // k.shape[1]
    mask = visible(n, window, keep_first)
    out = []
    for h in range(heads):
        g = h // group
        score = (q[:, h] @ k[:, g].T) * scale + head_bias[h]
        out.append((torch.sigmoid(score) * mask) @ v[:, g])
    return torch.stack(out, dim=1)


def decay_of(x, w1, w2, w0):
    """exp(-e^(-1/2) sigmoid(w2 tanh(w1 x) + w0)) per channel."""
    return torch.exp(-math.exp(-0.5) * torch.sigmoid(torch.tanh(x @ w1.T) @ w2.T + w0))


def delta_rule(r, k, v, w, a, state=None):
    """All [n, H, D]; state [H, D, D] or None (zeros).  Returns (o [n, H, D], last state)."""
    n, heads, d = r.shape
    s = torch.zeros(heads, d, d, dtype=r.dtype) if state is None else state.clone()
    u = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    out = []
    for t in range(n):
        read = torch.einsum("hi,hij->hj", u[t], s)                    # u^T S_(t-1)
        s = (w[t][:, :, None] * s - (a[t] * u[t])[:, :, None] * read[:, None, :]
             + k[t][:, :, None] * v[t][:, None, :])
        out.append(torch.einsum("hij,hi->hj", s, r[t]))
    return torch.stack(out), s


def xielu(z, p, q):
    sp = torch.nn.functional.softplus
    neg = torch.clamp(z, max=0.0)
    return torch.where(z > 0, sp(p) * z * z + z / 2, (0.5 + sp(q)) * (torch.expm1(neg) - neg) + z / 2)


def softcap(x, c):
    return c * torch.tanh(x / c)


# ---- the model ---------------------------------------------------------------------------------

def _keep(x):
    return x


def as_stored_bf16(x):
    """What a tensor is after a trip through bfloat16 storage."""
    return x.to(torch.bfloat16).to(x.dtype)


def left_branch(h, w, p, c, rnd=_keep):
    n = h.shape[0]
    q = rnd(h @ w[p + "q"].T + w[p + "q.b"]).view(n, c["heads"], c["dim"])
    k = rnd(h @ w[p + "k"].T + w[p + "k.b"]).view(n, c["kv_heads"], c["dim"])
    v = rnd(h @ w[p + "v"].T + w[p + "v.b"]).view(n, c["kv_heads"], c["vdim"])
    o = sigmoid_window_attention(q, k, v, c["scale"], w[p + "pb"], c["mask"]["size"],
                                 c["mask"].get("keep_first", 0))
    return rnd(rnd(o).reshape(n, -1) @ w[p + "o"].T)


def right_branch(h, w, p, c, eps, rnd=_keep):
    n = h.shape[0]
    shape = (n, c["heads"], c["dim"])
    r, k, v = ((h @ w[p + x].T).view(shape) for x in ("r", "k", "v"))
    decay = decay_of(h, w[p + "w1"], w[p + "w2"], w[p + "w0"]).view(shape)
    rate = torch.sigmoid(h @ w[p + "a"].T + w[p + "a.b"]).view(shape)
    o, _ = delta_rule(r, k, v, decay, rate)
    o = unit_rms(o, eps).reshape(n, -1) * w[p + "norm"] * torch.sigmoid(h @ w[p + "g"].T)
    return rnd(rnd(o) @ w[p + "o"].T)


def forward(cfg, w, tokens, streams=None, store_bf16=False):
    """Logits [n, vocab] of one whole sequence; ``streams``: a list that receives the residual
    stream after every layer.  ``store_bf16``: what an engine that keeps its activations in
    bfloat16 between kernels would round is rounded (norm outputs, q/k/v, the mixers' and the
    feed-forward's inner results and outputs), everything else stays as it is: a yardstick
    for what storage rounding alone does to the logits."""
    rnd = as_stored_bf16 if store_bf16 else _keep
    tokens = torch.as_tensor(tokens)
    n = tokens.shape[0]
    eps = cfg["norm"]["eps"]
    x = w["embed"][tokens] + w["pos"][:n]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        h = rnd(zero_centred_norm(x, w[p + "norm1"], eps))
        x = x + m["left_scale"] * left_branch(h, w, p + "mix.left.", m["left"], rnd) \
            + m["right_scale"] * right_branch(h, w, p + "mix.right.", m["right"], eps, rnd)
        if layer.get("mlp") is not None:
            h = rnd(zero_centred_norm(x, w[p + "norm2"], eps))
            act = w[p + "mlp.act"]
            x = x + rnd(rnd(xielu(h @ w[p + "mlp.up"].T, act[0], act[1])) @ w[p + "mlp.down"].T)
        if streams is not None:
            streams.append(x.clone())
    return softcap(rnd(zero_centred_norm(x, w["final.norm"], eps)) @ w["head"].T, cfg["logit_softcap"])


def generate(cfg, w, prompt, num_new):
    """Greedy continuation, recomputing the whole sequence for every token."""
    ids = list(prompt)
    for _ in range(num_new):
        ids.append(int(torch.argmax(forward(cfg, w, ids)[-1])))
    return ids[len(prompt):]
