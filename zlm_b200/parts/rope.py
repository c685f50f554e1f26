"""Rotary position encoding with half-split pairs (i, i + head_dim/2).

inv[i] = theta^(-2 i / head_dim) for i < n_rot/2; the pair is turned by the angle
pos * inv[i] (src/image/zcom.zig:95-109, src/kernels/transformer/rope.zig:161-206).
The table of inverse frequencies is computed once, in 64-bit, and rounded to
fp32; the angle and its sine and cosine are computed in fp32 in the kernel that
also norms the heads and writes the cache, so this part only carries its table.
"""
from __future__ import annotations

import math
from typing import Any, Mapping, Optional

import torch

from ..registry import register_position_encoding
from .base import PositionEncoding, StepContext


@register_position_encoding("rope_half_split")
class RotaryHalfSplit(PositionEncoding):
    fused = True      # applied inside the attention mixer's norm/rotate/write kernel

    def __init__(self, theta: float, head_dim: int, n_rot: Optional[int] = None,
                 scaling: Optional[Mapping[str, Any]] = None):
        """``scaling`` ({"factor", "original", "fast", "slow"}): frequencies blended for contexts longer than the
        ``original`` one.  With where(t) = head_dim * ln(original / (2 pi t)) / (2 ln theta), lo = max(floor(where(fast)),
        0), hi = min(ceil(where(slow)), head_dim - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), frequency i
        becomes f_i / factor * ramp_i + f_i * (1 - ramp_i), and cosines and sines are multiplied by ``mscale`` =
        0.1 ln(factor) + 1 (the kernel that rotates takes it as a parameter)."""
        self.theta = float(theta)
        self.scaling = None if scaling is None else {k: float(scaling[k]) for k in ("factor", "original", "fast", "slow")}
        self.mscale = 1.0 if self.scaling is None else 0.1 * math.log(self.scaling["factor"]) + 1.0
        self.head_dim = int(head_dim)
        self.n_rot = int(head_dim if n_rot is None else n_rot)
        if self.n_rot % 2 or self.n_rot > self.head_dim or self.n_rot <= 0:
            raise ValueError(f"rope: n_rot={self.n_rot} must be even and at most head_dim={self.head_dim}")
        self.inv_freq: Optional[torch.Tensor] = None

    def attach(self, rt) -> None:
        super().attach(rt)
        i = torch.arange(self.n_rot // 2, dtype=torch.float64)
        inv = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / self.head_dim)
        if self.scaling is not None:
            sc = self.scaling

            def where(turns: float) -> float:
                return self.head_dim * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))
            lo = max(math.floor(where(sc["fast"])), 0)
            hi = min(math.ceil(where(sc["slow"])), self.head_dim - 1)
            ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            inv = inv / sc["factor"] * ramp + inv * (1.0 - ramp)
        self.inv_freq = inv.to(torch.float32).to(rt.device)

    def table(self, ctx: StepContext) -> torch.Tensor:
        """cos and sin of every token of the step at this part's frequencies, [2, n_rot/2, T]
        fp32: computed by the first layer that asks in a step and shared by all layers with
        the same frequencies (the positions of a step are the same in every layer)."""
        if self.scaling is not None:
            raise NotImplementedError("rope: the step's table is not built for scaled frequencies (their kernels take "
                                      "inv_freq and mscale)")
        key = ("rope_table", self.theta, self.head_dim, self.n_rot)
        t = ctx.extras.get(key)
        if t is None:
            t = ctx.scratch(f"rope.table.{self.theta}.{self.head_dim}.{self.n_rot}", (2, self.n_rot // 2, ctx.T),
                            torch.float32)
            self.rt.k.rope_table(t, self.inv_freq, self.n_rot, ctx.token_pos)
            ctx.extras[key] = t
        return t


@register_position_encoding("rope_interleaved")
class RotaryInterleaved(PositionEncoding):
    """Rotary encoding on neighbouring pairs (2i, 2i + 1), i < dims / 2: the pair is turned by
    pos * base^(-2i / dims); what lies beyond ``dims`` in the rotated vector passes unchanged.  The
    part carries the table of frequencies (computed in 64-bit, rounded to fp32); the mixer's own
    kernel forms the angle, its sine and cosine in fp32."""
    fused = True
    interleaved = True

    def __init__(self, base: float, dims: int):
        self.base = float(base)
        self.n_rot = int(dims)
        if self.n_rot % 2 or self.n_rot < 0:
            raise ValueError(f"rope: dims={self.n_rot} must be even")
        self.inv_freq: Optional[torch.Tensor] = None

    def attach(self, rt) -> None:
        super().attach(rt)
        i = torch.arange(self.n_rot // 2, dtype=torch.float64)
        inv = torch.pow(torch.tensor(self.base, dtype=torch.float64), -2.0 * i / max(self.n_rot, 1))
        self.inv_freq = inv.to(torch.float32).to(rt.device)


@register_position_encoding("none")
class NoPosition(PositionEncoding):
    fused = True
    inv_freq = None
    n_rot = 0

    def __init__(self, **_):
        pass
