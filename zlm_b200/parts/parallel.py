"""Two mixers side by side on one input: out = left_scale * left(x) + right_scale * right(x).

Each side is any registered mixer ({"kind": ..., its parameters}); its tensors carry the prefix ``left.`` or
``right.``.  What the sides ask of the cache is passed on: at most one of them may keep keys and values per token (the
layer has one place in the paged cache), and their per-sequence states become a pair (``LayerIO.state`` is then a
tuple, None where a side asked for nothing).  Each side adds its result into a zeroed fp32 row per token of its own;
one kernel forms the scaled sum in fp32 and adds it where the block wants the mixer's result.
"""
from __future__ import annotations

from typing import Any, Dict, Mapping, Optional

import torch

from ..registry import MIXERS, lookup, register_mixer
from .base import CacheRequest, LayerIO, Mixer, ParamSpec, StepContext


@register_mixer("parallel")
class ParallelMixers(Mixer):
    def __init__(self, hidden_size: int, left: Mapping[str, Any], right: Mapping[str, Any], left_scale: float = 1.0,
                 right_scale: float = 1.0):
        self.hidden = int(hidden_size)
        self.sides = {}
        for name, spec in (("left", left), ("right", right)):
            spec = dict(spec)
            kind = spec.pop("kind")
            if kind == "parallel":
                raise ValueError("parallel: a side cannot itself be a pair of mixers")
            self.sides[name] = lookup(MIXERS, "mixer", kind)(hidden_size=self.hidden, **spec)
        self.scales = {"left": float(left_scale), "right": float(right_scale)}

    @property
    def left(self) -> Mixer:
        return self.sides["left"]

    @property
    def right(self) -> Mixer:
        return self.sides["right"]

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {f"{side}.{n}": p for side, m in self.sides.items() for n, p in m.param_specs().items()}

    def attach(self, rt) -> None:
        super().attach(rt)
        for m in self.sides.values():
            m.attach(rt)

    def bind(self, params: Dict[str, torch.Tensor]) -> None:
        for side, m in self.sides.items():
            m.bind({n[len(side) + 1:]: t for n, t in params.items() if n.startswith(side + ".")})

    def tensors(self) -> Dict[str, torch.Tensor]:
        return {f"{side}.{n}": t for side, m in self.sides.items() for n, t in m.tensors().items()}

    def cache_request(self) -> Optional[CacheRequest]:
        asks = [r for r in (m.cache_request() for m in self.sides.values()) if r is not None]
        if len(asks) > 1:
            raise ValueError("parallel: both sides keep keys and values per token; a layer has one place in the paged cache")
        return asks[0] if asks else None

    def state_request(self):
        asks = tuple(m.state_request() for m in self.sides.values())
        return asks if any(a is not None for a in asks) else None

    @property
    def graph_safe(self) -> bool:      # type: ignore[override]
        return all(m.graph_safe for m in self.sides.values())

    def prefers_plain_launches(self, rows: int) -> bool:
        return any(m.prefers_plain_launches(rows) for m in self.sides.values())

    def step_key(self, ctx: StepContext):
        keys = tuple(k for k in (m.step_key(ctx) for m in self.sides.values()) if k is not None)
        return keys or None

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: StepContext, io: LayerIO) -> None:
        rt, k = self.rt, self.rt.k
        states = io.state if isinstance(io.state, tuple) else (None, None)
        outs = []
        for j, (side, m) in enumerate(self.sides.items()):
            y = rt.ws.get(f"parallel.{side}", residual.shape, torch.float32)
            # (the block's word that ``residual`` counts as zeros, if it gave one, is put back after the side has run:
            # the kernel object's ``scaled_sum`` below then stores instead of adding)
            swap = getattr(k, "swap_blank", None)
            if swap is not None:
                was = swap(y)
            else:
                y.zero_()
            m.forward(x, y, ctx, LayerIO(cache=io.cache if m.cache_request() is not None else None, state=states[j]))
            if swap is not None:
                swap(was)
            outs.append(y)
        k.scaled_sum(residual, outs[0], self.scales["left"], outs[1], self.scales["right"], accumulate=True)
