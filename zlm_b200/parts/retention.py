"""Retention: linear attention with one fixed decay per head, no softmax and no denominator.

    q = rot(W_q x), k = rot(W_k x) * head_dim^-1/2, v = W_v x     (heads x head_dim, heads x v_dim)
    S_t = decay_h * S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t         per head; S starts at zero
    y = W_o (unit_norm(o) * act(W_g x))                            unit_norm per head over v_dim, no weight

Options that other designs use: ``qkv_act="silu"`` (q, k and v pass through silu right after their projections),
``k_scale`` (1.0: none), ``out_norm="row"`` (the heads of o are normed together, over heads x v_dim, with a weight per
column, tensor ``norm.weight``, instead of each head by itself without one).

The state S [heads, head_dim, v_dim] is fp32 and is what the mixer keeps per sequence (``StateRequest``); it keeps
no keys or values.  Everything between the projections and the gate (angles, rotated q and k, decay, state, o,
the heads' norm) is fp32 in both compute dtypes.  The rotation is a registered position encoding whose table of
frequencies the kernel reads (``rope_half_split``: the first n_rot coordinates of a head, halves against each other).
"""
from __future__ import annotations

from typing import Any, Dict, Mapping, Optional, Sequence

import torch

from ..registry import POSITION_ENCODINGS, lookup, register_mixer
from .base import LayerIO, Mixer, ParamSpec, StateRequest, StepContext


@register_mixer("retention")
class Retention(Mixer):
    reads_input_by_products = True       # x goes into the fused projection and nowhere else

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, v_dim: int, decay: Sequence[float],
                 norm_eps: float, position: Optional[Mapping[str, Any]] = None, gate: str = "silu",
                 k_scale: Optional[float] = None, qkv_act: str = "none", out_norm: str = "head"):
        self.hidden = int(hidden_size)
        self.H, self.D, self.V = int(num_heads), int(head_dim), int(v_dim)
        self.decay_values = [float(d) for d in decay]
        if len(self.decay_values) != self.H:
            raise ValueError(f"retention: {len(self.decay_values)} decays for {self.H} heads")
        if gate not in ("silu", "sigmoid"):
            raise ValueError(f"retention: gate={gate!r}")
        if qkv_act not in ("none", "silu") or out_norm not in ("head", "row"):
            raise ValueError(f"retention: qkv_act={qkv_act!r}, out_norm={out_norm!r}")
        self.eps, self.gate, self.qkv_act, self.out_norm = float(norm_eps), gate, qkv_act, out_norm
        self.k_scale = float(self.D ** -0.5 if k_scale is None else k_scale)
        position = dict(position or {"kind": "none"})
        self.position = lookup(POSITION_ENCODINGS, "position encoding", position.pop("kind"))(**position)
        if getattr(self.position, "interleaved", False) or not getattr(self.position, "fused", False):
            raise ValueError("retention: the rotation must be one whose table the kernel reads (rope_half_split or none)")
        self.QK, self.VV = self.H * self.D, self.H * self.V
        if getattr(self.position, "mscale", 1.0) != 1.0:
            raise ValueError("this mixer's kernels do not take a rotation with scaled frequencies")

    def param_specs(self) -> Dict[str, ParamSpec]:
        s = {"q_proj.weight": ParamSpec((self.QK, self.hidden)), "k_proj.weight": ParamSpec((self.QK, self.hidden)),
             "v_proj.weight": ParamSpec((self.VV, self.hidden)), "g_proj.weight": ParamSpec((self.VV, self.hidden)),
             "o_proj.weight": ParamSpec((self.hidden, self.VV))}
        if self.out_norm == "row":
            s["norm.weight"] = ParamSpec((self.VV,), kind="vector", init="one_plus_normal")
        return s

    def state_request(self) -> Optional[StateRequest]:
        return StateRequest((self.H, self.D, self.V), torch.float32)

    def attach(self, rt) -> None:
        super().attach(rt)
        self.position.attach(rt)
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=rt.device)

    def bind(self, params: Dict[str, torch.Tensor]) -> None:
        # one fused projection: rows [q | k | v | g]
        self.w_in = torch.cat([params.pop("q_proj.weight"), params.pop("k_proj.weight"), params.pop("v_proj.weight"),
                               params.pop("g_proj.weight")], dim=0).contiguous()
        self.w_o = params.pop("o_proj.weight")
        self.w_norm = params.pop("norm.weight", None)
        self.check_products(in_proj=self.w_in, o_proj=self.w_o)

    def tensors(self) -> Dict[str, torch.Tensor]:
        a, b = self.QK, 2 * self.QK
        out = {"q_proj.weight": self.w_in[:a], "k_proj.weight": self.w_in[a:b], "v_proj.weight": self.w_in[b:b + self.VV],
               "g_proj.weight": self.w_in[b + self.VV:], "o_proj.weight": self.w_o}
        if self.w_norm is not None:
            out["norm.weight"] = self.w_norm
        return out

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: StepContext, io: LayerIO) -> None:
        rt, k = self.rt, self.rt.k
        T = x.shape[0]
        proj = rt.ws.get("retention.proj", (T, 2 * self.QK + 2 * self.VV), rt.dtype)
        k.linear(proj, x, self.w_in)
        if self.qkv_act == "silu":
            k.silu_rows(proj, 2 * self.QK + self.VV)
        o = rt.ws.get("retention.o", (T, self.VV), torch.float32)
        # many tokens: the step's cosines and sines come from the table that the position encoding computes once a
        # step for all layers with its frequencies; few tokens: the kernel forms its own
        table = self.position.table(ctx) if (T > 16 and self.position.n_rot and hasattr(self.position, "table")) else None
        k.retention(o, proj, 0, self.QK, 2 * self.QK, self.position.inv_freq, self.position.n_rot, self.decay, io.state,
                    ctx, self.H, self.D, self.V, self.k_scale, cos_sin=table)
        y = rt.ws.get("retention.gated", (T, self.VV), rt.dtype)
        if self.out_norm == "row":
            k.norm_gate(y, o, proj[:, 2 * self.QK + self.VV:], self.H, self.V, "row", self.w_norm, self.eps, self.gate)
        else:
            k.head_gate(y, o.view(T, self.H, self.V), proj[:, 2 * self.QK + self.VV:], self.H, self.V, True, self.eps, self.gate)
        k.linear(residual, y, self.w_o, accumulate=True, defer=True)       # a norm reads the stream next
