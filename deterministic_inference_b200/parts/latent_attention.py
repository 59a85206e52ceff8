"""Attention whose keys and values are rebuilt from a small latent vector per token, which is all
the cache keeps.

q = W_q x, per head [``head_dim`` plain | ``rot_dim`` rotated] elements.  W_dkv x has ``kv_rank`` +
``rot_dim`` rows: the first kv_rank, RMS-normed with a weight, are the latent c; the last rot_dim,
rotated by the token's position, are a key part k_r that all heads share.  Head h's key is
[W_uk,h c | k_r] and its value W_uv,h c, so

    score_h(i, j) = (q_plain,h(i) . W_uk,h c(j) + q_rot,h(i) . k_r(j)) * scale
                  = ([W_uk,h^T q_plain,h(i) | q_rot,h(i)] . [c(j) | k_r(j)]) * scale,
    out_h(i)      = W_uv,h sum_j p_h(i, j) c(j).

The second forms are what runs: the query is taken through the key map once, attention runs over
the cached rows [c | k_r] as ONE key head of kv_rank + rot_dim elements whose first kv_rank
elements double as the value, and the weighted latent goes through the value map.  A token costs
kv_rank + rot_dim cache elements whatever the number of heads.  Softmax over the keys the mask
shows ("causal", "window", "chunk" as in ``masked_attention``); norms, angles, scores and the softmax
are float32.
"""

from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import Mixer
from .registry import POSITION_ENCODINGS, register_mixer
from .spec import PagedKVSpec, PartSpec, TensorSpec


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    def __init__(self, ctx, prefix: str, hidden_size: int, num_heads: int, head_dim: int, rot_dim: int,
                 v_head_dim: int, kv_rank: int, scale: float, position_encoding: PartSpec, norm_eps: float,
                 mask: str = "causal", mask_size: Optional[int] = None, names: Optional[dict] = None):
        if mask not in ("causal", "window", "chunk"):
            raise ValueError(f"mask {mask!r} is not known ('causal', 'window', 'chunk')")
        if mask != "causal" and (mask_size is None or int(mask_size) < 1):
            raise ValueError(f"a {mask} mask needs a positive mask_size")
        self.prefix = prefix
        self.hidden_size, self.num_heads = int(hidden_size), int(num_heads)
        self.head_dim, self.rot_dim, self.v_head_dim = int(head_dim), int(rot_dim), int(v_head_dim)
        self.kv_rank, self.scale, self.norm_eps = int(kv_rank), float(scale), float(norm_eps)
        self.mask, self.mask_size = mask, None if mask == "causal" else int(mask_size)
        self.names = dict(q="q", down="dkv", latent_norm="dkv.norm", key_map="uk", value_map="uv", o="o")
        self.names.update(names or {})
        self.position_encoding = POSITION_ENCODINGS.build(position_encoding, ctx)
        if self.position_encoding.rotary_dim != self.rot_dim:
            raise ValueError(f"latent_attention: the rotation covers {self.position_encoding.rotary_dim} "
                             f"elements, the rotated part has {self.rot_dim}")
        self.out_dtype = ctx.dtype
        self.w_in = self.w_key = self.w_value = self.w_o = self.latent_norm = self.freq = None

    def tensor_specs(self):
        p, n, w = self.prefix, self.names, self.hidden_size
        h, d, r, e, c = self.num_heads, self.head_dim, self.rot_dim, self.v_head_dim, self.kv_rank
        return [TensorSpec(p + n["q"], (h * (d + r), w)), TensorSpec(p + n["down"], (c + r, w)),
                TensorSpec(p + n["latent_norm"], (c,), role="vector", init="one_plus_normal"),
                TensorSpec(p + n["key_map"], (h * d, c)), TensorSpec(p + n["value_map"], (h * e, c)),
                TensorSpec(p + n["o"], (w, h * e))]

    def load(self, tensors):
        p, n = self.prefix, self.names
        h, d, e, c = self.num_heads, self.head_dim, self.v_head_dim, self.kv_rank
        self.w_in = torch.cat([tensors[p + n["q"]], tensors[p + n["down"]]], dim=0).contiguous()
        self.latent_norm = tensors[p + n["latent_norm"]]
        # per head [K, N]: the key map takes a query's plain part [d] to the latent's size [c]; the
        # value map takes a weighted latent [c] to the head's value [e]
        self.w_key = tensors[p + n["key_map"]].view(h, d, c).contiguous()
        self.w_value = tensors[p + n["value_map"]].view(h, e, c).transpose(1, 2).contiguous()
        self.w_o = tensors[p + n["o"]]
        self.freq = self.position_encoding.frequencies()

    def cache_spec(self):
        return PagedKVSpec(1, self.kv_rank + self.rot_dim, self.mask_size, v_head_dim=0,
                           mask="chunk" if self.mask == "chunk" else "window")

    def forward(self, x, step, cache):
        h, d, r, e, c = self.num_heads, self.head_dim, self.rot_dim, self.v_head_dim, self.kv_rank
        proj = ops.as_tensor(ops.linear(x, self.w_in))
        t, width = proj.shape
        q = ops.latent_prepare(proj, h, d, r, c, self.latent_norm, self.norm_eps, self.freq, step.positions,
                               cache.kv if cache.writes else None, cache.slot_mapping, cache.page_size,
                               self.out_dtype)
        ops.heads_linear(proj.as_strided((t, h, d), (width, d + r, 1)), self.w_key, q[:, :, :c])
        latent = ops.masked_attention(q, cache.kv, cache.attention_meta, self.scale, 1, c, cache.page_size,
                                      self.mask, self.mask_size, values_in_keys=True)
        o = torch.empty(t, h, e, dtype=proj.dtype, device=proj.device)
        ops.heads_linear(latent, self.w_value, o)
        return ops.linear(o.view(t, h * e), self.w_o)
