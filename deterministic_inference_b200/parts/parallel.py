"""Several mixers side by side: every branch reads the same input, and the result is
sum_i scale_i * branch_i(x).  The sum is left to the reader (the float32 residual stream adds
the branches' outputs in float32, in branch order).  Each branch keeps the cache of its own
kind; the schedule entry's cache is a composite with one member per branch."""

from __future__ import annotations

from ..kernels import ops
from .base import Mixer
from .registry import MIXERS, register_mixer
from .spec import CompositeSpec, StateSpec


@register_mixer("parallel")
class ParallelMixers(Mixer):
    def __init__(self, ctx, branches: list, scales: list):
        if len(branches) != len(scales) or not branches:
            raise ValueError(f"parallel mixers: {len(branches)} branches and {len(scales)} scales")
        self.branches = [MIXERS.build(spec, ctx) for spec in branches]
        self.scales = [float(s) for s in scales]

    @property
    def state_on_device(self) -> bool:
        return all(getattr(b, "state_on_device", False) or not isinstance(b.cache_spec(), StateSpec)
                   for b in self.branches)

    def tensor_specs(self):
        return [s for b in self.branches for s in b.tensor_specs()]

    def load(self, tensors):
        for b in self.branches:
            b.load(tensors)

    def cache_spec(self):
        return CompositeSpec(tuple(b.cache_spec() for b in self.branches))

    def forward(self, x, step, cache):
        outs = [b.forward(x, step, cache.members[i]) for i, b in enumerate(self.branches)]
        return ops.WeightedSum(list(zip(self.scales, outs)))
