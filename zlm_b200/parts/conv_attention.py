"""Grouped-query attention whose q, k and v pass through a short causal convolution over time, with a sink in the
softmax and a gate on the output.

    q, k, v = conv(W_q x), conv(W_k x), conv(W_v x)     per channel: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros
                                                        before the sequence's start
    q, k <- unit_norm per head over head_dim (``qk_norm``; no weight, no rotation: positions do not enter the scores)
    s_ij = q_i . k_j * scale   for 0 <= i - j < window (window 0: all earlier tokens)
    p_ij = exp(s_ij) / (1 + sum_j exp(s_ij))            (``sink``: one more term of score 0 that has no value)
    y = W_o (concat_h(p v) * sigmoid(W_g x))

Options that other designs use: ``conv=False`` (no convolution and no ``*_conv`` tensors); ``qk_norm`` "head" (RMS norm
per head with one weight of head_dim shared by the heads, tensors ``q_norm.weight`` / ``k_norm.weight``) or "row" (RMS
norm over the whole projection, all heads of q, or of k, at once, with a weight per channel); ``position`` (a registered
rotation whose frequencies the kernel reads, after the norm); ``gate="none"`` (no gate and no ``g_proj``).

Query head h reads kv head h // (heads / kv_heads).  Keys are ``head_dim`` wide and values ``v_dim``; in the cache
both are padded with zeros to one width, so that the pages have the layout the library's attention kernels read.  The
last taps - 1 projected values of a sequence are its state (``StateRequest``).
"""
from __future__ import annotations

from typing import Any, Dict, Mapping, Optional, Union

import torch

from ..registry import POSITION_ENCODINGS, lookup, register_mixer
from .base import CacheRequest, LayerIO, Mixer, ParamSpec, StateRequest, StepContext


@register_mixer("conv_attention")
class ConvAttention(Mixer):
    reads_input_by_products = True       # x goes into the fused projection and nowhere else

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, v_dim: int, conv_taps: int,
                 scale: float, norm_eps: float, window: int = 0, qk_norm: Union[bool, str] = True, sink: bool = True,
                 gate: str = "sigmoid", conv: bool = True, position: Optional[Mapping[str, Any]] = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"attention: {num_heads} heads over {num_kv_heads} kv heads")
        if gate not in ("silu", "sigmoid", "none"):
            raise ValueError(f"attention: gate={gate!r}")
        qk_norm = {True: "unit", False: "none"}.get(qk_norm, qk_norm)
        if qk_norm not in ("none", "unit", "head", "row"):
            raise ValueError(f"attention: qk_norm={qk_norm!r}")
        self.hidden = int(hidden_size)
        self.H, self.G, self.D, self.V = int(num_heads), int(num_kv_heads), int(head_dim), int(v_dim)
        self.taps, self.scale, self.eps = int(conv_taps), float(scale), float(norm_eps)
        self.window, self.qk_norm, self.sink, self.gate = int(window), qk_norm, bool(sink), gate
        self.conv = bool(conv)
        if not self.conv:
            self.taps = 1
        if self.taps < 1:
            raise ValueError(f"attention: a convolution of {self.taps} taps")
        position = dict(position or {"kind": "none"})
        self.position = lookup(POSITION_ENCODINGS, "position encoding", position.pop("kind"))(**position)
        if getattr(self.position, "interleaved", False) or not getattr(self.position, "fused", False):
            raise ValueError("attention: the rotation must be one whose frequencies the kernel reads (rope_half_split or none)")
        # what the first kernel of this kind took (convolution, per-head unit norm, a gate) stays on it
        self.general = (not self.conv) or self.qk_norm in ("head", "row") or bool(getattr(self.position, "n_rot", 0))
        # keys and values share one padded width in the cache (a multiple of 16: what the tensor-core kernels take)
        self.hdp = (max(self.D, self.V) + 15) // 16 * 16
        self.C = (self.H + self.G) * self.D + self.G * self.V          # convolved channels: q, k, v
        self.HV = self.H * self.V
        self.GW = self.HV if self.gate != "none" else 0        # the gate's columns in the fused projection

    def attach(self, rt) -> None:
        super().attach(rt)
        self.position.attach(rt)

    def param_specs(self) -> Dict[str, ParamSpec]:
        H, G, D, V, K, t = self.H, self.G, self.D, self.V, self.hidden, self.taps
        s = {"q_proj.weight": ParamSpec((H * D, K)), "k_proj.weight": ParamSpec((G * D, K)),
             "v_proj.weight": ParamSpec((G * V, K)), "o_proj.weight": ParamSpec((K, self.HV))}
        if self.gate != "none":
            s["g_proj.weight"] = ParamSpec((self.HV, K))
        if self.conv:
            s.update({"q_conv.weight": ParamSpec((H * D, t)), "k_conv.weight": ParamSpec((G * D, t)),
                      "v_conv.weight": ParamSpec((G * V, t))})
        if self.qk_norm in ("head", "row"):
            nq, nk = ((D,), (D,)) if self.qk_norm == "head" else ((H * D,), (G * D,))
            s["q_norm.weight"] = ParamSpec(nq, kind="vector", init="one_plus_normal")
            s["k_norm.weight"] = ParamSpec(nk, kind="vector", init="one_plus_normal")
        return s

    def cache_request(self) -> Optional[CacheRequest]:
        return CacheRequest(self.G, self.hdp, self.window)

    def state_request(self) -> Optional[StateRequest]:
        return StateRequest((self.taps - 1, self.C), self.rt.dtype) if (self.conv and self.taps > 1) else None

    def step_key(self, ctx: StepContext):
        # the decode kernel cuts the longest sequence's pages into parts (as for the rotary attention mixer)
        if not ctx.is_decode:
            return None
        from ..kernels import attention_len_bucket
        return ("gqa_attention", attention_len_bucket(ctx.max_len))

    def bind(self, params: Dict[str, torch.Tensor]) -> None:
        # one fused projection: rows [q | k | v | g]; the convolutions' taps in the same channel order
        rows = [params.pop("q_proj.weight"), params.pop("k_proj.weight"), params.pop("v_proj.weight")]
        if self.gate != "none":
            rows.append(params.pop("g_proj.weight"))
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.w_conv = (torch.cat([params.pop("q_conv.weight"), params.pop("k_conv.weight"), params.pop("v_conv.weight")],
                                 dim=0).contiguous() if self.conv else None)
        self.q_norm, self.k_norm = params.pop("q_norm.weight", None), params.pop("k_norm.weight", None)
        if self.q_norm is not None and self.q_norm.dtype != self.k_norm.dtype:
            self.q_norm, self.k_norm = self.q_norm.float(), self.k_norm.float()
        self.w_o = params.pop("o_proj.weight")
        self.w_o_stored = self.w_o
        if self.gate == "none" and self.V < self.hdp:
            # no gate kernel drops the heads' padding: the projection gets zero columns there instead
            wide = torch.zeros((self.hidden, self.H, self.hdp), dtype=self.w_o.dtype, device=self.w_o.device)
            wide[:, :, :self.V] = self.w_o.view(self.hidden, self.H, self.V)
            self.w_o = wide.view(self.hidden, self.H * self.hdp).contiguous()
        self.check_products(in_proj=self.w_in, o_proj=self.w_o)

    def tensors(self) -> Dict[str, torch.Tensor]:
        a, b, c = self.H * self.D, (self.H + self.G) * self.D, self.C
        out = {"q_proj.weight": self.w_in[:a], "k_proj.weight": self.w_in[a:b], "v_proj.weight": self.w_in[b:c],
               "o_proj.weight": self.w_o_stored}
        if self.gate != "none":
            out["g_proj.weight"] = self.w_in[c:]
        if self.conv:
            out.update({"q_conv.weight": self.w_conv[:a], "k_conv.weight": self.w_conv[a:b], "v_conv.weight": self.w_conv[b:]})
        if self.q_norm is not None:
            out.update({"q_norm.weight": self.q_norm, "k_norm.weight": self.k_norm})
        return out

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: StepContext, io: LayerIO) -> None:
        rt, k = self.rt, self.rt.k
        T = x.shape[0]
        cache = io.cache
        proj = rt.ws.get("conv_attn.proj", (T, self.C + self.GW), rt.dtype)
        k.linear(proj, x, self.w_in)
        q = rt.ws.get("conv_attn.q", (T, self.H * self.hdp), rt.dtype)
        if self.general:
            k.attn_prep(q, proj, self.w_conv, io.state, ctx, cache.block_table, cache.pool, self.H, self.G, self.D, self.V,
                        self.taps, self.qk_norm, self.q_norm, self.k_norm, self.eps, self.position.inv_freq,
                        int(getattr(self.position, "n_rot", 0) or 0), float(getattr(self.position, "mscale", 1.0)))
        else:
            k.conv_norm_write(q, proj, self.w_conv, io.state, ctx, cache.block_table, cache.pool, self.H, self.G, self.D,
                              self.V, self.taps, self.qk_norm == "unit", self.eps)
        out = rt.ws.get("conv_attn.out", (T, self.H * self.hdp), rt.dtype)
        key = self.step_key(ctx)
        k.attention(out, q, cache.pool, cache.block_table, ctx.token_pos, ctx.token_slot, self.H, self.G, self.hdp,
                    self.scale, self.window, ctx, len_bucket=key[1] if key else None,
                    v_dim=self.V if self.V < self.hdp else None, sink=self.sink)
        if self.gate == "none":
            y = out             # (the output projection has zero columns where the heads are padded)
        else:
            y = rt.ws.get("conv_attn.gated", (T, self.HV), rt.dtype)
            k.head_gate(y, out.view(T, self.H, self.hdp), proj[:, self.C:], self.H, self.V, False, self.eps, self.gate)
        k.linear(residual, y, self.w_o, accumulate=True, defer=True)       # a norm reads the stream next
