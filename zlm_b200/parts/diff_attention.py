"""Differential attention: every head has two attention maps over the same values, and the second, times a learned
number, is taken from the first.

With h the mixer's input, per token (H query heads over G key/value heads, query head i reads key/value head
i // (H / G)):

    q = W_q h   [H, 2, dim]        k = W_k h   [G, 2, dim]        v = W_v h   [G, vdim]
    q, k <- RMSNorm over dim of every head and map (one weight for q, one for k), then rotation of neighbouring pairs
            (2i, 2i+1) of the first ``position.dims`` coordinates by pos * base^(-2i / dims)
    s_m(i, j) = (q_m(i) . k_m(j)) * scale,  then  s <- softcap * tanh(s / softcap)  (if softcap > 0)
    a_m = softmax_j(s_m) v   over the keys j <= i of i's own chunk of ``chunk`` positions (chunk 0: all j <= i)
    lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff            (one number for the layer; lq1 ... [dim])
    o = (a_1 - lambda a_2) / sqrt(mean((a_1 - lambda a_2)^2) + eps) * (1 - diff)    per head over vdim
    y = W_o [heads' o]

The two maps run through the library's attention kernels as two query heads and two key heads that share one value
head (``v_share`` = 2): the cache holds, per token, 2G key heads and G value heads, keys and values padded with zeros
to one width (a multiple of 16, what the tensor-core kernels take).  Norms, angles, scores, softmax, lambda and the
head's unit norm are 32-bit whatever the compute dtype.
"""
from __future__ import annotations

from typing import Any, Dict, Mapping, Optional

import torch

from ..registry import POSITION_ENCODINGS, lookup, register_mixer
from .base import CacheRequest, LayerIO, Mixer, ParamSpec, StepContext


@register_mixer("diff_attention")
class DiffAttention(Mixer):
    reads_input_by_products = True       # x goes into the fused q/k/v projection and nowhere else

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, v_dim: int, scale: float,
                 diff: float, norm_eps: float, softcap: float = 0.0, chunk: int = 0, window: int = 0,
                 position: Optional[Mapping[str, Any]] = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"attention: {num_heads} heads over {num_kv_heads} kv heads")
        self.hidden = int(hidden_size)
        self.H, self.G, self.D, self.V = int(num_heads), int(num_kv_heads), int(head_dim), int(v_dim)
        if min(self.H, self.G, self.D, self.V) <= 0:
            raise ValueError("attention: heads, kv heads, dim and vdim must be positive")
        self.scale, self.diff, self.eps, self.softcap = float(scale), float(diff), float(norm_eps), float(softcap)
        self.chunk, self.window = int(chunk), int(window)
        if self.softcap < 0 or self.chunk < 0 or self.window < 0:
            raise ValueError("attention: softcap, chunk and window cannot be negative")
        position = dict(position or {"kind": "none"})
        self.position = lookup(POSITION_ENCODINGS, "position encoding", position.pop("kind"))(**position)
        if not getattr(self.position, "fused", False) or not (getattr(self.position, "interleaved", False)
                                                               or self.position.n_rot == 0):
            raise ValueError("differential attention rotates neighbouring pairs in its own kernel: "
                             "position must be 'rope_interleaved' or 'none'")
        if self.position.n_rot > self.D:
            raise ValueError(f"attention: {self.position.n_rot} rotated dimensions in a head of {self.D}")
        # keys and values share one padded width in the cache
        self.hdp = (max(self.D, self.V) + 15) // 16 * 16
        self.NQ, self.NK, self.NV = 2 * self.H * self.D, 2 * self.G * self.D, self.G * self.V
        self.lam = 0.0

    def param_specs(self) -> Dict[str, ParamSpec]:
        K, D = self.hidden, self.D
        s = {"q": ParamSpec((self.NQ, K)), "k": ParamSpec((self.NK, K)), "v": ParamSpec((self.NV, K)),
             "o": ParamSpec((K, self.H * self.V)),
             "q.norm": ParamSpec((D,), kind="vector", init="one_plus_normal"),
             "k.norm": ParamSpec((D,), kind="vector", init="one_plus_normal")}
        for n in ("lq1", "lk1", "lq2", "lk2"):
            s[n] = ParamSpec((D,), kind="vector", init="normal")
        return s

    def cache_request(self) -> Optional[CacheRequest]:
        return CacheRequest(2 * self.G, self.hdp, self.window, chunk=self.chunk, value_heads=self.G)

    def attach(self, rt) -> None:
        super().attach(rt)
        self.position.attach(rt)

    def step_key(self, ctx: StepContext):
        # the decode kernel cuts the longest sequence's pages into parts (as for the other attention mixers)
        if not ctx.is_decode:
            return None
        from ..kernels import PAGE_TOKENS, attention_len_bucket
        # (with chunks a query's keys span a chunk's pages at most, however long the sequence)
        reach = min(ctx.max_len, self.chunk + PAGE_TOKENS) if self.chunk else ctx.max_len
        return ("gqa_attention", attention_len_bucket(reach))

    def bind(self, params: Dict[str, torch.Tensor]) -> None:
        # one fused projection: rows [q | k | v], with rows of zeros up to a multiple of 8
        rows = [params.pop("q"), params.pop("k"), params.pop("v")]
        n = self.NQ + self.NK + self.NV
        if n % 8:
            rows.append(torch.zeros((8 - n % 8, self.hidden), dtype=rows[0].dtype, device=rows[0].device))
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.w_o = params.pop("o")
        self.q_norm, self.k_norm = params.pop("q.norm"), params.pop("k.norm")
        if self.q_norm.dtype != self.k_norm.dtype:
            self.q_norm, self.k_norm = self.q_norm.float(), self.k_norm.float()
        self.lvec = {n: params.pop(n) for n in ("lq1", "lk1", "lq2", "lk2")}
        f = {n: t.float() for n, t in self.lvec.items()}
        # one number for the layer, in 32-bit
        lam = torch.exp((f["lq1"] * f["lk1"]).sum()) - torch.exp((f["lq2"] * f["lk2"]).sum()) + torch.tensor(
            self.diff, dtype=torch.float32, device=f["lq1"].device)
        self.lam = float(lam)
        self.check_products(in_proj=self.w_in, o_proj=self.w_o)

    def tensors(self) -> Dict[str, torch.Tensor]:
        a, b = self.NQ, self.NQ + self.NK
        return {"q": self.w_in[:a], "k": self.w_in[a:b], "v": self.w_in[b: b + self.NV], "o": self.w_o,
                "q.norm": self.q_norm, "k.norm": self.k_norm, **self.lvec}

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: StepContext, io: LayerIO) -> None:
        rt, k = self.rt, self.rt.k
        T = x.shape[0]
        H, G, hdp = self.H, self.G, self.hdp
        cache = io.cache
        proj = rt.ws.get("diff_attn.proj", (T, self.w_in.shape[0]), rt.dtype)
        k.linear(proj, x, self.w_in)
        q = rt.ws.get("diff_attn.q", (T, 2 * H * hdp), rt.dtype)
        k.diff_prep(q, proj, self.q_norm, self.k_norm, self.eps, self.position.inv_freq, self.position.n_rot,
                    ctx.token_pos, ctx.token_slot, cache.block_table, cache.pool, H, G, self.D, self.V)
        a = rt.ws.get("diff_attn.maps", (T, 2 * H * hdp), rt.dtype)
        key = self.step_key(ctx)
        k.attention(a, q, cache.pool, cache.block_table, ctx.token_pos, ctx.token_slot, 2 * H, 2 * G, hdp, self.scale,
                    self.window, ctx, len_bucket=key[1] if key else None, v_dim=self.V if self.V < hdp else None,
                    chunk=self.chunk, softcap=self.softcap, v_share=2)
        o = rt.ws.get("diff_attn.out", (T, H * self.V), rt.dtype)
        k.diff_combine(o, a, H, G, self.V, hdp, self.lam, 1.0 - self.diff, self.eps)
        k.linear(residual, o, self.w_o, accumulate=True, defer=True)       # a norm reads the stream next
