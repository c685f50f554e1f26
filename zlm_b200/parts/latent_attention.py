"""Latent attention: keys and values of every head are projections of one small latent per
token, and only that latent is cached.

With h the mixer's input, per token:

    q = W_q h                        per head [dim | rot_dim]: a plain part and a rotated part
    [c_raw | kr_raw] = W_dkv h       kv_rank + rot_dim rows
    c  = RMSNorm(c_raw) * w_c        the latent (weight per coordinate)
    kr = rot(kr_raw, pos)            a rotated key slice, the same for every head
    k_h = [W_uk_h c | kr],  v_h = W_uv_h c
    score_h(i, j) = (q_h(i) . k_h(j)) * scale,  j in the window ending at i;  softmax;  y = W_o [heads' outputs]

Options: ``sink`` (a learned number per head, tensor ``sink`` [heads], whose exponential joins the softmax's denominator:
it has no key and no value and is not scaled), ``gate`` (head h's output is multiplied by sigmoid(W_g h)_h, tensor ``g``
[heads, hidden], one number per head from the mixer's own input) and ``chunk`` (a query sees only the keys of its own
chunk of that many positions, counted from position 0).

The cache record of a token is [c | kr] (``CacheRequest.token_shape``); a layer built with
``kv_proj=False`` has no W_dkv and reads the records of the schedule entry its own entry names
(``ScheduleEntry.cache_of``), with its own W_uk, W_uv, queries and everything else.

The step folds the up-projections away from the cached side: q'_h = W_uk_h^T q_h[:dim] makes the
score q'_h . c + rot(q_h[dim:]) . kr, and sum_j p_j v_h(j) = W_uv_h (sum_j p_j c_j), so attention
runs over the records as they are: one key/value record per token that all heads read.

Whole prompts in bfloat16 (every sequence of the step starts at 0) may run *unfolded* instead: the step's records are
gathered, [W_uk | W_uv] is applied to their latents as one product, per-head keys [W_uk_h c | kr] and values
[W_uv_h c | 0] go to a scratch pool of the library's attention layout, and the library's flash attention serves the
step: (dim + rot_dim + v_dim) instead of (2 kv_rank + rot_dim) multiply-adds for every query, key and head.  The cache
receives the same records either way.
"""
from __future__ import annotations

from typing import Any, Dict, Mapping, Optional

import torch

from ..registry import POSITION_ENCODINGS, lookup, register_mixer
from .base import CacheRequest, LayerIO, Mixer, ParamSpec, StepContext


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    reads_input_by_products = True       # x goes into the fused q / latent projection and nowhere else

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, rot_dim: int, v_dim: int, kv_rank: int,
                 scale: float, norm_eps: float = 1e-6, window: int = 0,
                 position: Optional[Mapping[str, Any]] = None, kv_proj: bool = True, sink: bool = False,
                 gate: bool = False, chunk: int = 0):
        self.hidden = int(hidden_size)
        self.H, self.dn, self.dr, self.dv, self.r = int(num_heads), int(head_dim), int(rot_dim), int(v_dim), int(kv_rank)
        if min(self.H, self.dv, self.r) <= 0 or self.dn < 0 or self.dr < 0 or self.dn + self.dr <= 0:
            raise ValueError("latent attention: heads, v_dim, kv_rank and dim + rot_dim must be positive")
        self.scale, self.eps, self.window = float(scale), float(norm_eps), int(window)
        self.kv_proj = bool(kv_proj)
        self.sink, self.gate, self.chunk = bool(sink), bool(gate), int(chunk)
        self.sinks: Optional[torch.Tensor] = None
        position = dict(position or {"kind": "none"})
        self.position = lookup(POSITION_ENCODINGS, "position encoding", position.pop("kind"))(**position)
        if not getattr(self.position, "fused", False) or not (getattr(self.position, "interleaved", False)
                                                               or self.position.n_rot == 0):
            raise ValueError("latent attention rotates neighbouring pairs in its own kernel: "
                             "position must be 'rope_interleaved' or 'none'")
        if self.position.n_rot > self.dr:
            raise ValueError(f"latent attention: {self.position.n_rot} rotated dimensions in a part of {self.dr}")
        self.Dq, self.R = self.dn + self.dr, self.r + self.dr
        self.Q = self.H * self.Dq

    # ---- declarations -----------------------------------------------------
    def param_specs(self) -> Dict[str, ParamSpec]:
        s = {"q": ParamSpec((self.Q, self.hidden)),
             "uk": ParamSpec((self.H * self.dn, self.r)),
             "uv": ParamSpec((self.H * self.dv, self.r)),
             "o": ParamSpec((self.hidden, self.H * self.dv))}
        if self.kv_proj:
            s["dkv"] = ParamSpec((self.R, self.hidden))
            s["dkv.norm"] = ParamSpec((self.r,), kind="vector", init="one_plus_normal")
        if self.sink:
            s["sink"] = ParamSpec((self.H,), kind="vector", init="normal")
        if self.gate:
            s["g"] = ParamSpec((self.H, self.hidden))
        return s

    def cache_request(self) -> Optional[CacheRequest]:
        return CacheRequest(1, self.R, self.window, token_shape=(self.R,), chunk=self.chunk)

    def attach(self, rt) -> None:
        super().attach(rt)
        self.position.attach(rt)

    def step_key(self, ctx: StepContext):
        # the decode kernel cuts the longest sequence's pages into splits: its grid, and with it a
        # captured step, holds for one rounded length
        if not ctx.is_decode:
            return None
        from ..kernels import PAGE_TOKENS, attention_len_bucket
        # (with chunks a query's keys span a chunk's pages at most, however long the sequence)
        reach = min(ctx.max_len, self.chunk + PAGE_TOKENS) if self.chunk else ctx.max_len
        return ("latent_attention", attention_len_bucket(reach))

    def bind(self, params: Dict[str, torch.Tensor]) -> None:
        H, dn, dv, r = self.H, self.dn, self.dv, self.r
        w_q = params.pop("q")
        # one fused projection: rows [q | c_raw | kr_raw | gate], with rows of zeros up to a multiple of 8
        rows = [w_q]
        if self.kv_proj:
            rows.append(params.pop("dkv"))
            self.c_norm = params.pop("dkv.norm")
        else:
            self.c_norm = None
        self.g_off = sum(w.shape[0] for w in rows)
        if self.gate:
            rows.append(params.pop("g"))
            n = self.g_off + H
            if n % 8:
                rows.append(torch.zeros((8 - n % 8, self.hidden), dtype=w_q.dtype, device=w_q.device))
        self.w_in = torch.cat(rows, dim=0).contiguous() if len(rows) > 1 else w_q
        self.N_in = self.w_in.shape[0]
        if self.sink:
            self.sinks = params.pop("sink").float().contiguous()
        # per head: W_uk_h^T [r, dn] (folds into the query), W_uv_h [dv, r] (unfolds the output)
        self.w_uk_t = params.pop("uk").view(H, dn, r).transpose(1, 2).contiguous()
        self.w_uv = params.pop("uv").view(H, dv, r).contiguous()
        self.w_o = params.pop("o")
        self.check_products(q=self.w_in, o=self.w_o)
        # Whole prompts in bfloat16 may run unfolded (see ``_forward_unfolded``): the up-projections as one matrix
        # [W_uk | W_uv] applied to the step's latents, and W_o with a zero column for every column that pads a
        # head's values to the keys' width
        hd = dn + self.dr
        self.unfoldable = bool(
            self.w_o.dtype == torch.bfloat16 and hd % 16 == 0 and 16 <= hd <= 192 and dv <= hd and r % 8 == 0
            and self.R % 8 == 0 and self.Q % 8 == 0 and self.N_in % 8 == 0
            and hasattr(self.rt.k, "latent_unfold"))
        if self.unfoldable:
            self.w_ukv = torch.cat([self.w_uk_t.transpose(1, 2).reshape(H * dn, r), self.w_uv.reshape(H * dv, r)]).contiguous()
            pad = torch.zeros(self.hidden, H, hd, dtype=self.w_o.dtype, device=self.w_o.device)
            pad[:, :, :dv] = self.w_o.view(self.hidden, H, dv)
            self.w_o_pad = pad.view(self.hidden, H * hd).contiguous()

    def tensors(self) -> Dict[str, torch.Tensor]:
        out = {"q": self.w_in[: self.Q], "o": self.w_o,
               "uk": self.w_uk_t.transpose(1, 2).reshape(self.H * self.dn, self.r),
               "uv": self.w_uv.reshape(self.H * self.dv, self.r)}
        if self.kv_proj:
            out["dkv"] = self.w_in[self.Q: self.Q + self.R]
            out["dkv.norm"] = self.c_norm
        if self.sink:
            out["sink"] = self.sinks
        if self.gate:
            out["g"] = self.w_in[self.g_off: self.g_off + self.H]
        return out

    # ---- the step -----------------------------------------------------------
    UNFOLD_FROM = 128        # tokens of a step from which whole prompts run unfolded

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: StepContext, io: LayerIO) -> None:
        rt, k = self.rt, self.rt.k
        T = x.shape[0]
        H, dn, dr, dv, r, R = self.H, self.dn, self.dr, self.dv, self.r, self.R
        cache = io.cache
        writes = cache.writes and self.kv_proj
        if cache.writes != self.kv_proj:
            raise ValueError("latent attention: a layer without W_dkv must read another entry's cache, "
                             "and one with W_dkv keeps its own")
        if (self.unfoldable and T >= self.UNFOLD_FROM and not ctx.is_decode and ctx.h_seq_start
                and not any(ctx.h_seq_start)):
            self._forward_unfolded(x, residual, ctx, cache, writes)
            return
        qd = rt.ws.get("lat.qd", (T, self.N_in), rt.dtype)
        k.linear(qd, x, self.w_in)
        q = qd[:, : self.Q]
        q3 = qd.as_strided((T, H, self.Dq), (qd.stride(0), self.Dq, 1))
        # the folded query [q' | rotated part] of every head
        ql = rt.ws.get("lat.ql", (T, H, R), rt.dtype)
        k.latent_prep(q, ql[:, :, r:], qd[:, self.Q: self.Q + R] if writes else None, self.c_norm, self.eps,
                      self.position.inv_freq, self.position.n_rot, ctx.token_pos, ctx.token_slot,
                      cache.block_table, cache.pool, H, dn, dr, r)
        if dn:
            k.head_linear(ql[:, :, :r], q3[:, :, :dn], self.w_uk_t)
        else:
            ql[:, :, :r].zero_()
        ol = rt.ws.get("lat.ol", (T, H * r), rt.dtype)
        key = self.step_key(ctx)
        k.latent_attention(ol, ql.view(T, H * R), cache.pool, cache.block_table, ctx.token_pos, ctx.token_slot,
                           H, r, dr, self.scale, self.window, ctx, len_bucket=key[1] if key else None,
                           **self._options())
        ov = rt.ws.get("lat.ov", (T, H * dv), rt.dtype)
        k.head_linear(ov.view(T, H, dv), ol.view(T, H, r), self.w_uv)
        if self.gate:
            k.head_scalar_gate(ov.view(T, H, dv), qd[:, self.g_off: self.g_off + H])
        k.linear(residual, ov, self.w_o, accumulate=True, defer=True)       # a norm reads the stream next

    def _options(self) -> Dict[str, Any]:
        """The attention kernels' words for the sink and the chunks (none of them for a mixer without)."""
        o: Dict[str, Any] = {}
        if self.sink:
            o["sinks"] = self.sinks
        if self.chunk:
            o["chunk"] = self.chunk
        return o

    def _step_pages(self, ctx: StepContext):
        """Pages for the step's own tokens, sequence after sequence (whole prompts: positions start at 0), as a table
        [sequences, pages] on the device and their number; made once per step and shared by the layers."""
        made = ctx.extras.get("latent.step_pages")
        if made is None:
            from ..kernels import PAGE_TOKENS
            need = [(n + PAGE_TOKENS - 1) // PAGE_TOKENS for n in ctx.h_seq_new]
            table = torch.zeros((ctx.R, max(need)), dtype=torch.int32)
            at = 0
            for i, n in enumerate(need):
                table[i, :n] = torch.arange(at, at + n, dtype=torch.int32)
                at += n
            rows = torch.arange(ctx.R, dtype=torch.int32)
            made = (table.to(self.rt.device), rows.to(self.rt.device), at)
            ctx.extras["latent.step_pages"] = made
        return made

    def _forward_unfolded(self, x: torch.Tensor, residual: torch.Tensor, ctx: StepContext, cache, writes: bool) -> None:
        """Whole prompts: the records go to the cache as always, but the step's attention runs over per-head keys
        [W_uk_h c | kr] and values W_uv_h c of its own tokens, written out once into a scratch pool of the library's
        attention layout: (dim + rot_dim + v_dim) instead of (2 kv_rank + rot_dim) multiply-adds for every query, key
        and head, on the library's flash attention kernels (tcgen05 at a key width of 128)."""
        import types
        from ..kernels import PAGE_TOKENS
        rt, k = self.rt, self.rt.k
        T = x.shape[0]
        H, dn, dr, dv, r, R = self.H, self.dn, self.dr, self.dv, self.r, self.R
        hd = dn + dr
        qd = rt.ws.get("lat.qd", (T, self.N_in), rt.dtype)
        k.linear(qd, x, self.w_in)
        q = qd[:, : self.Q]
        q3 = qd.as_strided((T, H, self.Dq), (qd.stride(0), self.Dq, 1))
        # rotated query parts in place; the records into their pages and, for this step's products, into plain rows
        # (a layer that reads another layer's records gathers them from the pages instead)
        rec = rt.ws.get("lat.rec", (T, R), rt.dtype)
        if writes:
            k.latent_prep(q, q3[:, :, dn:], qd[:, self.Q: self.Q + R], self.c_norm, self.eps,
                          self.position.inv_freq, self.position.n_rot, ctx.token_pos, ctx.token_slot,
                          cache.block_table, cache.pool, H, dn, dr, r, rec_out=rec)
        else:
            k.latent_prep(q, q3[:, :, dn:], None, self.c_norm, self.eps,
                          self.position.inv_freq, self.position.n_rot, ctx.token_pos, ctx.token_slot,
                          cache.block_table, cache.pool, H, dn, dr, r)
            k.latent_gather(rec, cache.pool, cache.block_table, ctx.token_pos, ctx.token_slot)
        kv = rt.ws.get("lat.kv", (T, H * (dn + dv)), rt.dtype)
        k.linear(kv, rec[:, :r], self.w_ukv)
        table, rows, pages = self._step_pages(ctx)
        spool = rt.ws.get("lat.unfolded", (pages, 2, H, PAGE_TOKENS, hd), rt.dtype)
        # places beyond a sequence's last token are never written and are multiplied by weights of zero: fresh memory
        # there must hold numbers, so a buffer that has grown is cleared once
        seen = getattr(rt, "_unfolded_cleared", (0, 0))
        if seen[0] != spool.data_ptr() or seen[1] < spool.numel():
            spool.zero_()
            rt._unfolded_cleared = (spool.data_ptr(), spool.numel())
        k.latent_unfold(spool, table, kv, rec, ctx.token_pos, ctx.token_seq, H, dn, dr, dv, r)
        plan = types.SimpleNamespace(is_decode=False, cu_seqlens=ctx.cu_seqlens, seq_slot=rows, seq_start=ctx.seq_start,
                                     R=ctx.R, max_new=ctx.max_new, max_len=ctx.max_len, scratch=ctx.scratch,
                                     h_seq_start=ctx.h_seq_start, h_seq_new=ctx.h_seq_new)
        ao = rt.ws.get("lat.ao", (T, H * hd), rt.dtype)
        k.attention(ao, q, spool, table, ctx.token_pos, ctx.token_seq, H, H, hd, self.scale, self.window, plan,
                    v_dim=dv, **self._options())
        if self.gate:
            k.head_scalar_gate(ao.view(T, H, hd), qd[:, self.g_off: self.g_off + H])
        k.linear(residual, ao, self.w_o_pad, accumulate=True, defer=True)      # a norm reads the stream next
