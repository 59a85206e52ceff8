"""Generalised delta rule: a linear recurrence with a matrix state per head.

r = W_r x, k = W_k x, v = W_v x (heads x ``head_dim`` each).  Per head and key channel a
decay w = exp(-decay_scale * sigmoid(W_w2 tanh(W_w1 x) + w0)) (a low-rank map of rank
``decay_rank``) and a removal rate a = sigmoid(W_a x + b_a).  With the unit key
u = k / sqrt(sum(k^2) + key_eps) of each head the state S [head_dim keys, head_dim values]
moves as
    S_t = diag(w_t) S_(t-1) - (a_t * u_t) (u_t^T S_(t-1)) + k_t v_t^T     (both terms read S_(t-1))
and o_t = S_t^T r_t.  Each head's o is divided by its root mean square (``norm_eps``), the
concatenated heads are multiplied by a weight and by sigmoid(W_g x), then projected by W_o.
The state starts at zero, is float32 and lives in the request's state slot; decays, rates,
unit keys and the recurrence are float32 whatever the engine's storage type.
"""

from __future__ import annotations

import math
from typing import Optional

import torch

from ..kernels import ops
from .base import Mixer
from .registry import register_mixer
from .spec import StateSpec, TensorSpec


@register_mixer("delta_rule")
class DeltaRule(Mixer):
    # the kernels take the sequences' state slots from the step's device metadata, and a
    # sequence on state slot 0 (padding) starts from zero and stores nothing
    state_on_device = True

    def __init__(self, ctx, prefix: str, hidden_size: int, num_heads: int, head_dim: int, decay_rank: int,
                 norm_eps: float, decay_scale: float = math.exp(-0.5), key_eps: float = 1e-6,
                 names: Optional[dict] = None):
        self.prefix = prefix
        self.hidden_size, self.num_heads, self.head_dim = int(hidden_size), int(num_heads), int(head_dim)
        self.decay_rank = int(decay_rank)
        self.norm_eps, self.decay_scale, self.key_eps = float(norm_eps), float(decay_scale), float(key_eps)
        self.names = dict(r="r", k="k", v="v", g="g", a="a", a_bias="a.b", w1="w1", w2="w2", w0="w0",
                          norm="norm", o="o")
        self.names.update(names or {})
        self.out_dtype = ctx.dtype
        self.w_in = self.w2_t = self.w0 = self.a_bias = self.norm_weight = self.w_o = None

    def tensor_specs(self):
        p, n, w = self.prefix, self.names, self.hidden_size
        hd = self.num_heads * self.head_dim
        return [TensorSpec(p + n[x], (hd, w)) for x in ("r", "k", "v", "g", "a")] + [
            TensorSpec(p + n["a_bias"], (hd,), role="vector", init="normal"),
            TensorSpec(p + n["w1"], (self.decay_rank, w)),
            TensorSpec(p + n["w2"], (hd, self.decay_rank)),
            TensorSpec(p + n["w0"], (hd,), role="vector", init="normal"),
            TensorSpec(p + n["norm"], (hd,), role="vector", init="one_plus_normal"),
            TensorSpec(p + n["o"], (w, hd)),
        ]

    def load(self, tensors):
        p, n = self.prefix, self.names
        # one product for everything that is read from x: [r | k | v | g | a | w1]
        self.w_in = torch.cat([tensors[p + n[x]] for x in ("r", "k", "v", "g", "a", "w1")], dim=0).contiguous()
        self.w2_t, self.w0 = tensors[p + n["w2"]].t().contiguous(), tensors[p + n["w0"]]
        self.a_bias, self.norm_weight = tensors[p + n["a_bias"]], tensors[p + n["norm"]]
        self.w_o = tensors[p + n["o"]]

    def cache_spec(self):
        return StateSpec((self.num_heads, self.head_dim, self.head_dim), "float32")

    def forward(self, x, step, cache):
        proj = ops.linear(x, self.w_in, out_dtype=torch.float32 if x.dtype != torch.float32 else None)
        y = ops.delta_rule(proj, self.w2_t, self.w0, self.a_bias, self.norm_weight, cache.state, step,
                           self.num_heads, self.head_dim, self.decay_rank, self.decay_scale, self.key_eps,
                           self.norm_eps, self.out_dtype)
        return ops.linear(y, self.w_o)
