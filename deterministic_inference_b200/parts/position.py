"""Rotary position encoding (rotate-half over the first ``rotary_dim`` dims of a
head): inv_freq_i = theta^(-i/(r/2)), angle = pos * inv_freq_i, all in float32;
the table [max_positions, rotary_dim] = [cos | sin] is built once
(sid/kernels/rope.py:41-48).  The rotation itself runs inside the attention
mixer's fused q/k kernel, which takes this table, or, for mixers that compute the
angles themselves, the frequencies (``frequencies()``; no table and no longest position).

``scaling`` (``factor``, ``low``, ``high``, ``original``) stretches long wavelengths: with
l_i = 2 pi / f_i, a frequency with l_i < original / high stays; one with l_i > original / low
becomes f_i / factor; between the two, with s = (original / l_i - low) / (high - low), it
becomes (1 - s) f_i / factor + s f_i."""

from __future__ import annotations

import math
from typing import Optional

import torch

from .base import PositionEncoding
from .registry import register_position_encoding


@register_position_encoding("rope")
class RotaryEmbedding(PositionEncoding):
    def __init__(self, ctx, head_dim: int, rotary_dim: int, theta: float, max_positions: Optional[int] = None,
                 scaling: Optional[dict] = None):
        if rotary_dim % 2 or rotary_dim > head_dim:
            raise ValueError(f"rotary_dim {rotary_dim} must be even and at most head_dim {head_dim}")
        self.head_dim, self.rotary_dim = int(head_dim), int(rotary_dim)
        self.theta = float(theta)
        self.max_positions = None if max_positions is None else int(max_positions)
        self.scaling = None
        if scaling:
            self.scaling = tuple(float(scaling[k]) for k in ("factor", "low", "high", "original"))
            if self.scaling[2] <= self.scaling[1] or self.scaling[0] <= 0 or self.scaling[3] <= 0:
                raise ValueError(f"rope scaling {scaling!r}: needs high > low and positive factor, original")
        self.ctx = ctx
        self._table = self._freq = None

    def frequency_list(self) -> list:
        """The rotary_dim / 2 frequencies as Python floats (computed in double precision)."""
        out = []
        for i in range(self.rotary_dim // 2):
            f = self.theta ** (-2.0 * i / self.rotary_dim)
            if self.scaling is not None:
                factor, low, high, original = self.scaling
                wavelength = 2.0 * math.pi / f
                if wavelength > original / low:
                    f = f / factor
                elif wavelength >= original / high:
                    s = (original / wavelength - low) / (high - low)
                    f = (1.0 - s) * f / factor + s * f
            out.append(f)
        return out

    def frequencies(self) -> torch.Tensor:
        """float32 [rotary_dim / 2] on the device: a kernel's angle is position * frequency."""
        if self._freq is None:
            key = ("rope_freq", self.rotary_dim, self.theta, self.scaling)
            f = self.ctx.shared.get(key)
            if f is None:
                f = torch.tensor(self.frequency_list(), dtype=torch.float64).to(torch.float32).to(self.ctx.device)
                self.ctx.shared[key] = f
            self._freq = f
        return self._freq

    def prepare(self):
        if self.max_positions is None:       # no table: the mixer's kernel computes the angles
            self.frequencies()
            return
        if self.scaling is not None:
            key = ("rope", self.rotary_dim, self.theta, self.max_positions, self.scaling)
            table = self.ctx.shared.get(key)
            if table is None:
                pos = torch.arange(self.max_positions, dtype=torch.float32, device=self.ctx.device)
                freqs = torch.outer(pos, self.frequencies())
                table = torch.cat([freqs.cos(), freqs.sin()], dim=-1).contiguous()
                self.ctx.shared[key] = table
            self._table = table
            return
        key = ("rope", self.rotary_dim, self.theta, self.max_positions)
        table = self.ctx.shared.get(key)
        if table is None:
            half = self.rotary_dim // 2
            dev = self.ctx.device
            inv_freq = 1.0 / (self.theta ** (torch.arange(0, half, dtype=torch.float32, device=dev) / half))
            pos = torch.arange(self.max_positions, dtype=torch.float32, device=dev)
            freqs = torch.outer(pos, inv_freq)
            table = torch.cat([freqs.cos(), freqs.sin()], dim=-1).contiguous()
            self.ctx.shared[key] = table
        self._table = table

    def rotary_table(self):
        if self.max_positions is None:
            raise ValueError("this rotary encoding was built without a longest position: it has no table")
        if self._table is None:
            self.prepare()
        return self._table


@register_position_encoding("none")
class NoPositionEncoding(PositionEncoding):
    """No position encoding: q and k go to attention as projected."""

    def __init__(self, ctx, **_):
        pass
