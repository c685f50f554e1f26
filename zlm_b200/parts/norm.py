"""RMSNorm over rows of the fp32 residual stream.

y = (x * 1/sqrt(mean(x^2) + eps)) * w, weight used as it is
(src/kernels/transformer/norm.zig:4-37).  ``scalar``: the checkpoint holds one gain for the whole
row (a tensor without dimensions) instead of a weight per coordinate.  ``layer_scale``: a second vector ``scale``
multiplies the normed row coordinate by coordinate (a layer's learned scale on its sublayer's output).
``one_plus``: the checkpoint stores the weight around zero and the row is multiplied by 1 + w (the sum is made once,
in fp32, when the weights are bound).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..registry import register_norm
from .base import Norm, ParamSpec


@register_norm("rms_norm")
class RMSNorm(Norm):
    reads_stream_by_kernel = True

    def __init__(self, size: int, eps: float, scalar: bool = False, layer_scale: bool = False, one_plus: bool = False):
        self.size = int(size)
        self.one_plus = bool(one_plus)
        self.stored: Optional[torch.Tensor] = None
        self.eps = float(eps)
        self.scalar = bool(scalar)
        self.layer_scale = bool(layer_scale)
        self.weight: Optional[torch.Tensor] = None
        self.gain: Optional[torch.Tensor] = None
        self.scale: Optional[torch.Tensor] = None
        self.reads_stream_by_kernel = not self.layer_scale      # (with a scale the plain norm kernel is not the whole norm)

    def param_specs(self) -> Dict[str, ParamSpec]:
        s = {"weight": ParamSpec(() if self.scalar else (self.size,), kind="vector",
                                 init="normal" if self.one_plus else "one_plus_normal")}
        if self.layer_scale:
            s["scale"] = ParamSpec((self.size,), kind="vector", init="one_plus_normal")
        return s

    def bind(self, params: Dict[str, torch.Tensor]) -> None:
        self.weight = params["weight"]
        if self.one_plus:
            self.stored = self.weight
            self.weight = (1.0 + self.stored.float()).contiguous()
        self.scale = params.get("scale")
        if self.scalar:
            # the kernels (and the products that fold a norm in) read a weight per coordinate: the one
            # gain, widened to 32 bits (exact), repeated along the row
            self.gain = self.stored if self.one_plus else self.weight
            self.weight = self.weight.float().reshape(1).expand(self.size).contiguous()

    def tensors(self) -> Dict[str, torch.Tensor]:
        out = {"weight": self.gain if self.scalar else (self.stored if self.one_plus else self.weight)}
        if self.layer_scale:
            out["scale"] = self.scale
        return out

    def forward(self, out: torch.Tensor, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
        w = self.weight
        if self.layer_scale:
            # norm weight and scale as one vector (their fp32 product, made once)
            if getattr(self, "_w_scaled", None) is None:
                self._w_scaled = (self.weight.float() * self.scale.float()).contiguous()
            w = self._w_scaled
        self.rt.k.rmsnorm(out, x, w, self.eps, rows)

    def add_into(self, stream: torch.Tensor, y: torch.Tensor, cast_out: Optional[torch.Tensor] = None) -> bool:
        fused = getattr(self.rt.k, "norm_scale_add", None)
        if fused is None:
            return super().add_into(stream, y)
        if cast_out is None:
            fused(stream, y, self.weight, self.eps, self.scale if self.layer_scale else None)
            return False
        fused(stream, y, self.weight, self.eps, self.scale if self.layer_scale else None, cast_out=cast_out)
        return True


    def add_into_then_norm(self, stream: torch.Tensor, y: torch.Tensor, nxt: Norm, out: torch.Tensor) -> bool:
        """stream += norm(y) and out = nxt(stream) in one kernel, if both norms are of this kind without a scale of
        their own and the kernel object has the kernel; the answer says whether it was done (else nothing was)."""
        fused = getattr(self.rt.k, "norm_add_norm", None)
        if (fused is None or not isinstance(nxt, RMSNorm) or self.layer_scale or nxt.layer_scale or y.dtype != torch.float32
                or self.size > getattr(self.rt.k, "NORM_ADD_NORM_MAX", 0)):
            return False
        fused(stream, y, self.weight, self.eps, out, nxt.weight, nxt.eps)
        return True


@register_norm("none")
class NoNorm(Norm):
    """Stands where a layer has nothing to norm (a layer without a feed-forward): no tensors, never run."""

    def __init__(self, size: int):
        self.size = int(size)

    def forward(self, out: torch.Tensor, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
        raise RuntimeError("a 'none' norm stands for a part that does not exist and is never run")
