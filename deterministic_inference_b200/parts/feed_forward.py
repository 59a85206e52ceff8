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
    def __init__(self, ctx, prefix: str, hidden_size: int, intermediate_size: int,
                 activation: str = "silu"):
        if activation != "silu":
            raise ValueError(f"gated_mlp: activation {activation!r} has no kernel (only 'silu')")
        self.prefix = prefix
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.w_gate_up = self.w_down = None

    def tensor_specs(self):
        p, h, i = self.prefix, self.hidden_size, self.intermediate_size
        return [TensorSpec(p + "gate_proj.weight", (i, h)), TensorSpec(p + "up_proj.weight", (i, h)),
                TensorSpec(p + "down_proj.weight", (h, i))]

    def load(self, tensors):
        p = self.prefix
        self.w_gate_up = torch.cat([tensors[p + "gate_proj.weight"], tensors[p + "up_proj.weight"]],
                                   dim=0).contiguous()
        self.w_down = tensors[p + "down_proj.weight"]

    def forward(self, x):
        return ops.linear(ops.gated_linear(x, self.w_gate_up), self.w_down)


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
