"""Dense gated feed-forward: down( act(gate(x)) * up(x) ), no biases; gate and up
are one product of the concatenated weights, gate first
(sid/model/qwen3.py:82-86, sid/model/loader.py:97-101)."""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import FeedForward
from .registry import register_feed_forward
from .spec import TensorSpec


@register_feed_forward("gated_mlp")
class GatedMLP(FeedForward):
    """``activation`` "silu": silu(gate) * up.  "limited_swish": with g = min(gate, limit) and
    u = clamp(up, -limit, limit), g * sigmoid(alpha * g) * (u + 1), in float32 from the product's
    accumulator where it is at hand.  ``names``: the checkpoint names of gate, up and down after the
    prefix."""

    def __init__(self, ctx, prefix: str, hidden_size: int, intermediate_size: int,
                 activation: str = "silu", limit: float = None, alpha: float = 1.702, names=None):
        if activation not in ("silu", "limited_swish"):
            raise ValueError(f"gated_mlp: activation {activation!r} has no kernel ('silu', 'limited_swish')")
        if activation == "limited_swish" and (limit is None or float(limit) <= 0):
            raise ValueError("gated_mlp: 'limited_swish' needs a positive limit")
        self.prefix, self.activation = prefix, activation
        self.limit, self.alpha = None if limit is None else float(limit), float(alpha)
        self.names = tuple(names) if names else ("gate_proj.weight", "up_proj.weight", "down_proj.weight")
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.out_dtype = ctx.dtype
        self.w_gate_up = self.w_down = None

    def tensor_specs(self):
        p, h, i = self.prefix, self.hidden_size, self.intermediate_size
        gate, up, down = self.names
        return [TensorSpec(p + gate, (i, h)), TensorSpec(p + up, (i, h)), TensorSpec(p + down, (h, i))]

    def load(self, tensors):
        p = self.prefix
        gate, up, down = self.names
        self.w_gate_up = torch.cat([tensors[p + gate], tensors[p + up]], dim=0).contiguous()
        self.w_down = tensors[p + down]

    def forward(self, x):
        if self.activation == "silu":
            return ops.linear(ops.gated_linear(x, self.w_gate_up), self.w_down)
        gate_up = ops.linear(x, self.w_gate_up)       # (few rows: split-k partial sums, added in float32 by the gate)
        return ops.linear(ops.limited_gate(gate_up, self.limit, self.alpha, self.out_dtype), self.w_down)


@register_feed_forward("dense_mlp")
class DenseMLP(FeedForward):
    """down( act(up(x)) ), no gate and no biases.  ``activation`` "xielu": with the two stored
    numbers p, q of ``act_name`` and softplus(y) = log(1 + exp(y)),
    act(z) = softplus(p) z^2 + z / 2 for z > 0 and (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2
    otherwise, computed in float32 from the product's accumulator where it is at hand."""

    def __init__(self, ctx, prefix: str, hidden_size: int, intermediate_size: int,
                 activation: str = "xielu", up_name: str = "up", down_name: str = "down",
                 act_name: str = "act"):
        if activation != "xielu":
            raise ValueError(f"dense_mlp: activation {activation!r} has no kernel (only 'xielu')")
        self.prefix, self.names = prefix, (up_name, down_name, act_name)
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.out_dtype = ctx.dtype
        self.w_up = self.w_down = None
        self.alpha_p = self.alpha_n = None

    def tensor_specs(self):
        p, h, i = self.prefix, self.hidden_size, self.intermediate_size
        up, down, act = self.names
        return [TensorSpec(p + up, (i, h)), TensorSpec(p + down, (h, i)),
                TensorSpec(p + act, (2,), role="vector")]

    def load(self, tensors):
        up, down, act = self.names
        self.w_up, self.w_down = tensors[self.prefix + up], tensors[self.prefix + down]
        pq = torch.nn.functional.softplus(tensors[self.prefix + act].to("cpu", torch.float32))
        self.alpha_p, self.alpha_n = float(pq[0]), float(torch.tensor(0.5, dtype=torch.float32) + pq[1])

    def forward(self, x):
        z = ops.linear(x, self.w_up, out_dtype=torch.float32 if x.dtype != torch.float32 else None)
        return ops.linear(ops.xielu(z, self.alpha_p, self.alpha_n, self.out_dtype), self.w_down)


@register_feed_forward("none")
class NoFeedForward(FeedForward):
    """A layer without a feed-forward; the block leaves the step out."""

    def __init__(self, ctx, **_):
        pass
