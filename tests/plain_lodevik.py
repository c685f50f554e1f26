"""A plain, slow implementation of the Lodevik design: one function per mechanism, float64 torch on the CPU, whole
sequences at once, no cache.  It shares no code with the package; the tests compare the engine with it.

Notation: a sequence of n tokens; x [n, width] is the residual stream; a tensor dictionary maps the checkpoint's
names to [out, in] matrices applied as W x.
"""
from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional, Sequence

import torch

F = torch.float64


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate_pairs(x: torch.Tensor, pos: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """x [n, ..., d]: coordinates (2i, 2i+1), i < dims/2, of the last axis are turned by pos * base^(-2i/dims);
    the coordinates from ``dims`` on stay."""
    if dims == 0:
        return x.clone()
    i = torch.arange(dims // 2, dtype=F)
    ang = pos.to(F)[:, None] * torch.pow(torch.tensor(base, dtype=F), -2.0 * i / dims)[None, :]     # [n, dims/2]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    c, s = torch.cos(ang).view(shape), torch.sin(ang).view(shape)
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def embed(tokens: Sequence[int], table: torch.Tensor, scale: float, bigram: Optional[torch.Tensor] = None,
          buckets: int = 0, mul_prev: int = 0, mul_cur: int = 0) -> torch.Tensor:
    """Row of the table times ``scale``, plus (with a bigram table of buckets + 1 rows) the row
    (prev * mul_prev + cur * mul_cur) mod buckets, or the last row for the sequence's first token."""
    out = []
    for j, t in enumerate(tokens):
        r = table[t].to(F) * scale
        if bigram is not None:
            row = buckets if j == 0 else (tokens[j - 1] * mul_prev + t * mul_cur) % buckets
            r = r + bigram[row].to(F)
        out.append(r)
    return torch.stack(out)


def visible(n: int, chunk: int = 0) -> torch.Tensor:
    """[n, n] bool: query i sees key j when j <= i and, with chunks, both lie in the same chunk of ``chunk``
    positions counted from 0."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    ok = j <= i
    if chunk:
        ok = ok & (i // chunk == j // chunk)
    return ok


def softmax_with_sink(s: torch.Tensor, ok: torch.Tensor, sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """s [heads, n, n]; masked softmax over the last axis; with ``sink`` [heads] the denominator also holds
    exp(sink_h), which has no key and no value."""
    s = s.masked_fill(~ok[None], -math.inf)
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink.to(F).view(-1, 1, 1))
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink.to(F).view(-1, 1, 1) - m)
    return e / den


def attend(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, ok: torch.Tensor, softcap: float = 0.0,
           sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q, k [n, heads, d], v [n, heads, dv], ok [n, n] -> [n, heads, dv]: p = softmax_j(cap(q_i . k_j * scale)) over
    the visible j, cap(s) = softcap * tanh(s / softcap) (softcap 0: none), the sink in the denominator only."""
    s = torch.einsum("ihd,jhd->hij", q.to(F), k.to(F)) * scale
    if softcap:
        s = softcap * torch.tanh(s / softcap)
    return torch.einsum("hij,jhd->ihd", softmax_with_sink(s, ok, sink), v.to(F))


def latent_attention(h: torch.Tensor, w: Mapping[str, torch.Tensor], heads: int, dim: int, rot_dim: int, vdim: int,
                     kv_rank: int, scale: float, rot_base: float, rot_dims: int, eps: float,
                     chunk: int = 0) -> torch.Tensor:
    """h [n, width] -> [n, width].  Tensors: q, dkv, dkv.norm, uk, uv, o and optionally sink [heads], g [heads, width]."""
    n = h.shape[0]
    pos = torch.arange(n)
    q = (h @ w["q"].to(F).T).view(n, heads, dim + rot_dim)
    d = h @ w["dkv"].to(F).T
    c = rms_norm(d[:, :kv_rank], w["dkv.norm"].to(F), eps)
    kr = rotate_pairs(d[:, kv_rank:], pos, rot_base, rot_dims)                       # [n, rot_dim], one for all heads
    qr = rotate_pairs(q[:, :, dim:], pos, rot_base, rot_dims)
    k = (c @ w["uk"].to(F).T).view(n, heads, dim)
    v = (c @ w["uv"].to(F).T).view(n, heads, vdim)
    # a head's key is [its own unrotated part | the rotated part that all heads share]
    qq = torch.cat([q[:, :, :dim], qr], dim=-1)
    kk = torch.cat([k, kr[:, None, :].expand(n, heads, rot_dim)], dim=-1)
    o = attend(qq, kk, v, scale, visible(n, chunk), 0.0, w.get("sink"))
    if "g" in w:
        o = o * torch.sigmoid(h @ w["g"].to(F).T)[:, :, None]
    return o.reshape(n, heads * vdim) @ w["o"].to(F).T


def diff_lambda(w: Mapping[str, torch.Tensor], diff: float) -> float:
    a = torch.exp((w["lq1"].to(F) * w["lk1"].to(F)).sum())
    b = torch.exp((w["lq2"].to(F) * w["lk2"].to(F)).sum())
    return float(a - b + diff)


def diff_attention(h: torch.Tensor, w: Mapping[str, torch.Tensor], heads: int, kv_heads: int, dim: int, vdim: int,
                   scale: float, softcap: float, diff: float, rot_base: float, rot_dims: int, eps: float,
                   chunk: int = 0) -> torch.Tensor:
    """Two attention maps per head over the same values, subtracted.  Tensors: q [heads*2*dim, width],
    k [kv_heads*2*dim, width], v [kv_heads*vdim, width], q.norm, k.norm [dim], lq1, lk1, lq2, lk2 [dim], o."""
    n = h.shape[0]
    pos = torch.arange(n)
    q = (h @ w["q"].to(F).T).view(n, heads, 2, dim)
    k = (h @ w["k"].to(F).T).view(n, kv_heads, 2, dim)
    v = (h @ w["v"].to(F).T).view(n, kv_heads, vdim)
    q = rotate_pairs(rms_norm(q, w["q.norm"].to(F), eps), pos, rot_base, rot_dims)
    k = rotate_pairs(rms_norm(k, w["k.norm"].to(F), eps), pos, rot_base, rot_dims)
    rep = heads // kv_heads
    kk = k.repeat_interleave(rep, dim=1)                 # query head h reads kv head h // rep
    vv = v.repeat_interleave(rep, dim=1)
    ok = visible(n, chunk)
    lam = diff_lambda(w, diff)
    maps = [attend(q[:, :, m], kk[:, :, m], vv, scale, ok, softcap) for m in range(2)]
    o = unit_rms(maps[0] - lam * maps[1], eps) * (1.0 - diff)
    return o.reshape(n, heads * vdim) @ w["o"].to(F).T


def gated_ff(h: torch.Tensor, w: Mapping[str, torch.Tensor]) -> torch.Tensor:
    return (gelu_tanh(h @ w["gate"].to(F).T) * (h @ w["up"].to(F).T)) @ w["down"].to(F).T


def _sub(tensors: Mapping[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def mixer(h: torch.Tensor, layer: Mapping, w: Mapping[str, torch.Tensor], eps: float) -> torch.Tensor:
    m = layer["mixer"]
    rot = m.get("rot") or {"base": 10000.0, "dims": 0}
    chunk = (m.get("mask") or {}).get("size", 0)
    if layer["type"] == "latent_attention":
        return latent_attention(h, w, m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["scale"],
                                rot["base"], rot["dims"], eps, chunk)
    if layer["type"] == "attention":
        return diff_attention(h, w, m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"], m["scale"],
                              m.get("softcap", 0.0), m["diff"], rot["base"], rot["dims"], eps, chunk)
    raise ValueError(layer["type"])


def forward(config: Mapping, tensors: Mapping[str, torch.Tensor], tokens: Sequence[int], streams: Optional[List] = None
            ) -> torch.Tensor:
    """Logits [n, vocab] of one sequence; ``streams`` receives the residual stream after every layer."""
    eps = config["norm"]["eps"]
    e = config["embedding"]
    bg = e.get("bigram")
    x = embed(tokens, tensors["embed"], e.get("scale", 1.0), tensors.get("bigram") if bg else None,
              *((bg["buckets"], bg["mul_prev"], bg["mul_cur"]) if bg else ()))
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        y = mixer(x, layer, _sub(tensors, p + "mix."), eps)
        x = x + rms_norm(y, tensors[p + "norm1"].to(F), eps) * tensors[p + "ls1"].to(F)
        if layer.get("mlp") is not None:
            y = gated_ff(x, _sub(tensors, p + "mlp."))
            x = x + rms_norm(y, tensors[p + "norm2"].to(F), eps) * tensors[p + "ls2"].to(F)
        if streams is not None:
            streams.append(x.clone())
    x = rms_norm(x, tensors["final.norm"].to(F), eps)
    return (x @ tensors["embed"].to(F).T) * config.get("logit_scale", 1.0)
