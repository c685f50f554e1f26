"""Two recurrent mixers whose whole memory of a sequence is a fixed-size fp32 state.

``rglru``: a recurrent block with a real-gated linear recurrent unit.  Two branches of ``width`` channels read the
mixer's input:

    y = gelu_tanh(W_y x + b_y)
    u = conv(W_x x + b_x) + b_c                  a causal convolution per channel over ``conv_taps`` tokens
    r = sigmoid(A_r[b] u_b + c_r[b]),  i = sigmoid(A_i[b] u_b + c_i[b])      u in ``blocks`` equal parts, a square
                                                                              matrix per part
    log a = -decay_scale * r * softplus(lam),   S_t = a S_(t-1) + sqrt(1 - a^2) * i * u,   out = W_o (S * y)

The state per sequence is S and the convolution's last ``conv_taps - 1`` inputs, one fp32 tensor [conv_taps, width].

``gated_linear_attention``: linear attention whose state decays per key channel by a gate computed from the input:

    q = W_q x * head_dim^-1/2, k = W_k x, v = W_v x                          heads x head_dim, heads x v_dim
    alpha = sigmoid(W_a2 (W_a1 x) + b_a)^(1/tau)                             heads x head_dim, through a low rank
    S_t = diag(alpha_t) S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t               per head
    out = W_o (rms_norm_per_head(o) * w_norm * silu(W_g x))                  w_norm [v_dim] shared by the heads

The state per sequence is S [heads, head_dim, v_dim] fp32.  In both mixers everything between the projections and the
output projection's input is fp32 whatever the compute dtype.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..registry import register_mixer
from .base import LayerIO, Mixer, ParamSpec, StateRequest, StepContext


@register_mixer("rglru")
class RecurrentGatedUnit(Mixer):
    def __init__(self, hidden_size: int, width: int, blocks: int, conv_taps: int, decay_scale: float = 8.0,
                 out_scale: float = 1.0):
        self.hidden, self.W, self.B, self.taps = int(hidden_size), int(width), int(blocks), int(conv_taps)
        self.c_decay, self.out_scale = float(decay_scale), float(out_scale)
        if self.W <= 0 or self.B <= 0 or self.W % self.B:
            raise ValueError(f"rglru: {self.W} channels in {self.B} blocks")
        if not 1 <= self.taps <= 8:
            raise ValueError(f"rglru: a convolution of {self.taps} taps (1 to 8 are built)")

    def param_specs(self) -> Dict[str, ParamSpec]:
        W, K, bs = self.W, self.hidden, self.W // self.B
        return {"y_proj.weight": ParamSpec((W, K)), "y_proj.bias": ParamSpec((W,), init="zeros"),
                "x_proj.weight": ParamSpec((W, K)), "x_proj.bias": ParamSpec((W,), init="zeros"),
                "conv.weight": ParamSpec((W, self.taps)), "conv.bias": ParamSpec((W,), init="zeros"),
                "a_gate.weight": ParamSpec((self.B, bs, bs)), "a_gate.bias": ParamSpec((self.B, bs), init="zeros"),
                "i_gate.weight": ParamSpec((self.B, bs, bs)), "i_gate.bias": ParamSpec((self.B, bs), init="zeros"),
                "lam": ParamSpec((W,)), "o_proj.weight": ParamSpec((K, W))}

    def state_request(self) -> Optional[StateRequest]:
        return StateRequest((self.taps, self.W), torch.float32)

    def bind(self, params: Dict[str, torch.Tensor]) -> None:
        # one fused projection: rows [y | x]
        self.w_in = torch.cat([params.pop("y_proj.weight"), params.pop("x_proj.weight")], dim=0).contiguous()
        dt = self.w_in.dtype
        self.small = {n: params.pop(n).to(dt).contiguous() for n in
                      ("y_proj.bias", "x_proj.bias", "conv.weight", "conv.bias", "a_gate.weight", "a_gate.bias",
                       "i_gate.weight", "i_gate.bias", "lam")}
        self.w_o = params.pop("o_proj.weight")
        # the two gates' matrices block by block, [A_r[b] ; A_i[b]]: what a many-token bfloat16 step multiplies on the
        # tensor cores
        self.w_gates = (torch.cat([self.small["a_gate.weight"], self.small["i_gate.weight"]], dim=1).contiguous()
                        if dt == torch.bfloat16 else None)
        self.check_products(in_proj=self.w_in, o_proj=self.w_o)

    def tensors(self) -> Dict[str, torch.Tensor]:
        return {"y_proj.weight": self.w_in[:self.W], "x_proj.weight": self.w_in[self.W:], "o_proj.weight": self.w_o,
                **self.small}

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: StepContext, io: LayerIO) -> None:
        rt, k, p = self.rt, self.rt.k, self.small
        T = x.shape[0]
        proj = rt.ws.get("rglru.proj", (T, 2 * self.W), rt.dtype)
        k.linear(proj, x, self.w_in)
        gated = rt.ws.get("rglru.gated", (T, self.W), rt.dtype)
        k.rglru(gated, proj, self.W, 0, p["x_proj.bias"], p["y_proj.bias"], p["conv.weight"], p["conv.bias"],
                p["a_gate.weight"], p["i_gate.weight"], p["a_gate.bias"], p["i_gate.bias"], p["lam"], self.c_decay, io.state,
                ctx, self.W, self.B, self.taps, self.out_scale, gates=self.w_gates)
        k.linear(residual, gated, self.w_o, accumulate=True, defer=True)       # a norm reads the stream next


@register_mixer("gated_linear_attention")
class GatedLinearAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, v_dim: int, tau: float, norm_eps: float,
                 rank: Optional[int] = None, gate: str = "silu"):
        """``rank``: the width of the decay's low-rank projection; None: whatever the checkpoint's tensors have."""
        self.hidden = int(hidden_size)
        self.H, self.D, self.V, self.rank = int(num_heads), int(head_dim), int(v_dim), int(-1 if rank is None else rank)
        self.tau, self.eps, self.gate = float(tau), float(norm_eps), gate
        if min(self.H, self.D, self.V) <= 0 or self.rank == 0 or self.rank < -1 or not self.tau > 0:
            raise ValueError(f"gated linear attention: {self.H} heads of {self.D} / {self.V}, rank {self.rank}, tau {self.tau}")
        if self.D > 128:
            raise ValueError(f"gated linear attention: keys of {self.D} columns (up to 128 are built)")
        if gate not in ("silu", "sigmoid"):
            raise ValueError(f"gated linear attention: gate={gate!r}")
        self.QK, self.VV = self.H * self.D, self.H * self.V

    def param_specs(self) -> Dict[str, ParamSpec]:
        K = self.hidden
        return {"q_proj.weight": ParamSpec((self.QK, K)), "k_proj.weight": ParamSpec((self.QK, K)),
                "v_proj.weight": ParamSpec((self.VV, K)), "g_proj.weight": ParamSpec((self.VV, K)),
                "a_down.weight": ParamSpec((self.rank, K)), "a_up.weight": ParamSpec((self.QK, self.rank)),
                "a_up.bias": ParamSpec((self.QK,), init="zeros"),
                "norm.weight": ParamSpec((self.V,), kind="vector", init="one_plus_normal"),
                "o_proj.weight": ParamSpec((K, self.VV))}

    def state_request(self) -> Optional[StateRequest]:
        return StateRequest((self.H, self.D, self.V), torch.float32)

    def bind(self, params: Dict[str, torch.Tensor]) -> None:
        # one fused projection: rows [q | k | v | g | the decay's low rank]
        self.w_in = torch.cat([params.pop("q_proj.weight"), params.pop("k_proj.weight"), params.pop("v_proj.weight"),
                               params.pop("g_proj.weight"), params.pop("a_down.weight")], dim=0).contiguous()
        self.rank = self.w_in.shape[0] - 2 * self.QK - 2 * self.VV
        if params["a_up.weight"].shape[1] != self.rank:
            raise ValueError(f"gated linear attention: the decay's two matrices disagree on their rank "
                             f"({self.rank} and {params['a_up.weight'].shape[1]})")
        dt = self.w_in.dtype
        self.a_up, self.a_bias = params.pop("a_up.weight").to(dt).contiguous(), params.pop("a_up.bias").to(dt).contiguous()
        self.w_norm = params.pop("norm.weight")
        self.w_o = params.pop("o_proj.weight")
        self.check_products(in_proj=self.w_in, o_proj=self.w_o)

    def tensors(self) -> Dict[str, torch.Tensor]:
        a, b, c, d = self.QK, 2 * self.QK, 2 * self.QK + self.VV, 2 * self.QK + 2 * self.VV
        return {"q_proj.weight": self.w_in[:a], "k_proj.weight": self.w_in[a:b], "v_proj.weight": self.w_in[b:c],
                "g_proj.weight": self.w_in[c:d], "a_down.weight": self.w_in[d:], "a_up.weight": self.a_up,
                "a_up.bias": self.a_bias, "norm.weight": self.w_norm, "o_proj.weight": self.w_o}

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: StepContext, io: LayerIO) -> None:
        rt, k = self.rt, self.rt.k
        T = x.shape[0]
        QK, VV = self.QK, self.VV
        proj = rt.ws.get("gla.proj", (T, 2 * QK + 2 * VV + self.rank), rt.dtype)
        k.linear(proj, x, self.w_in)
        alpha = rt.ws.get("gla.alpha", (T, QK), torch.float32)
        k.lowrank_decay(alpha, proj, 2 * QK + 2 * VV, self.a_up, self.a_bias, self.tau)
        o = rt.ws.get("gla.o", (T, VV), torch.float32)
        k.linear_attention(o, proj, 0, QK, 2 * QK, alpha, None, io.state, ctx, self.H, self.D, self.V, self.D ** -0.5)
        y = rt.ws.get("gla.gated", (T, VV), rt.dtype)
        k.norm_gate(y, o, proj[:, 2 * QK + VV: 2 * QK + 2 * VV], self.H, self.V, "head", self.w_norm, self.eps, self.gate)
        k.linear(residual, y, self.w_o, accumulate=True, defer=True)       # a norm reads the stream next
