"""Grouped-query attention without a softmax over a paged cache.

q = W_q x (+ b_q), k = W_k x (+ b_k), v = W_v x (+ b_v) as one product of the concatenated
weights; query head h reads key/value head h // (heads / kv_heads); key heads have
``head_dim`` elements, value heads ``v_head_dim``.  No position encoding enters the scores.
A query at position i sees key j <= i if i - j < ``window`` or j < ``keep_first`` (no window:
every j <= i); the weight of a visible key is sigmoid(q . k * scale + head_bias[h]) and the
weights are not normalised: out_i = sum_j weight_ij v_j.  Then the output projection on the
concatenated heads.  Scores, weights and the sum over keys are float32.
"""

from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import Mixer
from .registry import register_mixer
from .spec import PagedKVSpec, TensorSpec


@register_mixer("sigmoid_attention")
class SigmoidAttention(Mixer):
    def __init__(self, ctx, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int,
                 head_dim: int, v_head_dim: int, scale: float, window: Optional[int] = None,
                 keep_first: int = 0, bias: bool = True, head_bias: bool = True,
                 names: Optional[dict] = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads {num_heads} is not a multiple of num_kv_heads {num_kv_heads}")
        self.prefix = prefix
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.head_dim, self.v_head_dim = int(head_dim), int(v_head_dim)
        self.scale = float(scale)
        self.window = None if window is None else int(window)
        self.keep_first = int(keep_first) if self.window is not None else 0
        self.bias, self.head_bias = bool(bias), bool(head_bias)
        # checkpoint names of the parts' tensors, after the prefix
        self.names = dict(q="q", k="k", v="v", o="o", bias_suffix=".b", head_bias="pb")
        self.names.update(names or {})
        self.out_dtype = ctx.dtype
        self.w_qkv = self.b_qkv = self.w_o = self.pb = None

    def tensor_specs(self):
        p, n, w = self.prefix, self.names, self.hidden_size
        sizes = dict(q=self.num_heads * self.head_dim, k=self.num_kv_heads * self.head_dim,
                     v=self.num_kv_heads * self.v_head_dim)
        specs = []
        for which in ("q", "k", "v"):
            specs.append(TensorSpec(p + n[which], (sizes[which], w)))
            if self.bias:
                specs.append(TensorSpec(p + n[which] + n["bias_suffix"], (sizes[which],), role="vector",
                                        init="normal"))
        if self.head_bias:
            specs.append(TensorSpec(p + n["head_bias"], (self.num_heads,), role="vector", init="normal"))
        specs.append(TensorSpec(p + n["o"], (w, self.num_heads * self.v_head_dim)))
        return specs

    def load(self, tensors):
        p, n = self.prefix, self.names
        self.w_qkv = torch.cat([tensors[p + n[x]] for x in ("q", "k", "v")], dim=0).contiguous()
        if self.bias:
            self.b_qkv = torch.cat([tensors[p + n[x] + n["bias_suffix"]] for x in ("q", "k", "v")]).contiguous()
        if self.head_bias:
            self.pb = tensors[p + n["head_bias"]]
        self.w_o = tensors[p + n["o"]]

    def cache_spec(self):
        return PagedKVSpec(self.num_kv_heads, self.head_dim, self.window, v_head_dim=self.v_head_dim,
                           keep_first=self.keep_first)

    def forward(self, x, step, cache):
        # the projection's float32 accumulator takes the bias before anything is rounded
        qkv = ops.linear(x, self.w_qkv, out_dtype=torch.float32 if x.dtype != torch.float32 else None)
        q = ops.qkv_bias_cache(qkv, self.b_qkv, self.num_heads, self.num_kv_heads, self.head_dim,
                               self.v_head_dim, cache.kv if cache.writes else None, cache.slot_mapping,
                               cache.page_size, self.out_dtype)
        o = ops.sigmoid_attention(q, cache.kv, cache.attention_meta, self.scale, self.pb, self.v_head_dim,
                                  cache.page_size, self.window, self.keep_first)
        return ops.linear(o.view(o.shape[0], self.num_heads * self.v_head_dim), self.w_o)
