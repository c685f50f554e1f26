"""A plain, slow implementation of the Sudupel design: one function per mechanism, float64 on the CPU, whole
sequences only (positions count from 0, every state starts at zero).  It shares no code with the package: the
tests compare the package's kernels, cache and scheduler with it.

A model is (config, tensors): ``config`` is the design's config.json as a dict, ``tensors`` maps checkpoint names to
torch tensors.  ``forward(config, tensors, tokens)`` returns (logits [T, vocab], stream after every layer
[layers, T, width], every token's closest routing call).
"""
from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional, Tuple

import torch

F64 = torch.float64


def _w(tensors: Mapping[str, torch.Tensor], name: str) -> torch.Tensor:
    return tensors[name].to(F64)


# ---------------------------------------------------------------------------------------------- small pieces
def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float, one_plus: bool = False) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis, times the weight (or 1 + weight)."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    if weight is None:
        return y
    return y * (1.0 + weight if one_plus else weight)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def causal_conv(u: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y_t[c] = sum_j w[c, j] u_(t - taps + 1 + j)[c] (+ bias[c]); u [T, C], w [C, taps]; zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u], 0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + pad[j:j + T] * w[:, j]
    return y if bias is None else y + bias


def rotary_frequencies(rot: Mapping) -> Tuple[torch.Tensor, float]:
    """Frequencies f_i, i < dims / 2, with the YaRN blend if ``scaling`` is there, and the factor on cos and sin."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
    sc = rot.get("scaling")
    if sc is None:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def where(turns: float) -> float:
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(where(float(sc["fast"]))), 0)
    hi = min(math.ceil(where(float(sc["slow"]))), dims - 1)
    ramp = torch.tensor([min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(dims // 2)], dtype=F64)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: Optional[Mapping]) -> torch.Tensor:
    """x [T, heads, dim]: the first rot.dims coordinates of each head, i paired with i + dims/2."""
    if rot is None or int(rot["dims"]) == 0:
        return x
    dims = int(rot["dims"])
    f, m = rotary_frequencies(rot)
    a = positions.to(F64)[:, None] * f[None, :]
    cos, sin = (torch.cos(a) * m)[:, None, :], (torch.sin(a) * m)[:, None, :]
    u, v = x[..., :dims // 2], x[..., dims // 2:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], -1)


def softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: int, sink: bool) -> torch.Tensor:
    """q [T, H, D], k [T, G, D], v [T, G, V] -> [T, H * V].  Query i sees j with 0 <= i - j (< window, if any);
    ``sink``: one more term of score 0 without a value in the denominator."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    i = torch.arange(T)
    seen = (i[:, None] >= i[None, :])
    if window:
        seen &= (i[:, None] - i[None, :]) < window
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~seen, -math.inf)
        m = s.max(-1, keepdim=True).values
        if sink:
            m = m.clamp_min(0.0)
        e = torch.exp(s - m)
        den = e.sum(-1, keepdim=True) + (torch.exp(-m) if sink else 0.0)
        out[:, h] = (e / den) @ v[:, g]
    return out.reshape(T, -1)


def linear_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor) -> torch.Tensor:
    """Per head S_t = diag(decay_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t.  q, k [T, H, D], v [T, H, V],
    decay [T, H, D] (a fixed decay per head is the same number in every row and channel) -> [T, H, V]."""
    T, H, D = q.shape
    S = torch.zeros(H, D, v.shape[2], dtype=F64)
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for t in range(T):
        S = decay[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return out


# ---------------------------------------------------------------------------------------------- mixers
def attention_full_norm(h, positions, p: str, c: Mapping, tensors, eps: float) -> torch.Tensor:
    """The left half of 'parallel': q and k normed over the whole projection, rotation, every earlier key, a sink."""
    T = h.shape[0]
    H, G, D, V = int(c["heads"]), int(c.get("kv_heads", c["heads"])), int(c["dim"]), int(c["vdim"])
    q = rms_norm(h @ _w(tensors, p + "q").T, _w(tensors, p + "q.norm"), eps)
    k = rms_norm(h @ _w(tensors, p + "k").T, _w(tensors, p + "k.norm"), eps)
    v = h @ _w(tensors, p + "v").T
    q, k = rotate(q.view(T, H, D), positions, c.get("rot")), rotate(k.view(T, G, D), positions, c.get("rot"))
    o = softmax_attention(q, k, v.view(T, G, V), float(c["scale"]), 0, True)
    return o @ _w(tensors, p + "o").T


def attention_conv_window(h, positions, p: str, c: Mapping, tensors, eps: float) -> torch.Tensor:
    """The left half of 'parallel_2': short convolutions on q, k, v, per-head norm with a shared weight, rotation,
    a sliding window, ordinary softmax."""
    T = h.shape[0]
    H, G, D, V = int(c["heads"]), int(c.get("kv_heads", c["heads"])), int(c["dim"]), int(c["vdim"])
    q, k, v = (h @ _w(tensors, p + n).T for n in "qkv")
    if c.get("conv"):
        q, k, v = (causal_conv(x, _w(tensors, p + n + ".conv")) for x, n in ((q, "q"), (k, "k"), (v, "v")))
    q = rms_norm(q.view(T, H, D), _w(tensors, p + "q.norm"), eps)
    k = rms_norm(k.view(T, G, D), _w(tensors, p + "k.norm"), eps)
    q, k = rotate(q, positions, c.get("rot")), rotate(k, positions, c.get("rot"))
    window = int(c["mask"]["size"]) if c.get("mask") else 0
    o = softmax_attention(q, k, v.view(T, G, V), float(c["scale"]), window, False)
    return o @ _w(tensors, p + "o").T


def recurrent_block(h, p: str, c: Mapping, tensors) -> torch.Tensor:
    """The right half of 'parallel': two branches, a convolution, block-diagonal gates, a real-gated linear recurrence."""
    W, B = int(c["width"]), int(c["blocks"])
    y = gelu_tanh(h @ _w(tensors, p + "y").T + _w(tensors, p + "y.b"))
    u = causal_conv(h @ _w(tensors, p + "x").T + _w(tensors, p + "x.b"), _w(tensors, p + "conv"), _w(tensors, p + "conv.b"))
    T = h.shape[0]
    ub = u.view(T, B, W // B)
    r = torch.sigmoid(torch.einsum("boi,tbi->tbo", _w(tensors, p + "ra"), ub) + _w(tensors, p + "ra.b")).reshape(T, W)
    i = torch.sigmoid(torch.einsum("boi,tbi->tbo", _w(tensors, p + "ri"), ub) + _w(tensors, p + "ri.b")).reshape(T, W)
    log_a = -8.0 * r * torch.nn.functional.softplus(_w(tensors, p + "lam"))
    a = torch.exp(log_a)
    S = torch.zeros(W, dtype=F64)
    out = torch.zeros(T, W, dtype=F64)
    for t in range(T):
        S = a[t] * S + torch.sqrt(1.0 - a[t] ** 2) * i[t] * u[t]
        out[t] = S
    return (out * y) @ _w(tensors, p + "o").T


def gated_linear_attention(h, p: str, c: Mapping, tensors, eps: float) -> torch.Tensor:
    """The right half of 'parallel_2': a decay per key channel from a low-rank projection."""
    T = h.shape[0]
    H, D, V, tau = int(c["heads"]), int(c["dim"]), int(c["vdim"]), float(c["tau"])
    q = (h @ _w(tensors, p + "q").T * D ** -0.5).view(T, H, D)
    k = (h @ _w(tensors, p + "k").T).view(T, H, D)
    v = (h @ _w(tensors, p + "v").T).view(T, H, V)
    z = (h @ _w(tensors, p + "a1").T) @ _w(tensors, p + "a2").T + _w(tensors, p + "a2.b")
    alpha = torch.sigmoid(z) ** (1.0 / tau)
    o = linear_recurrence(q, k, v, alpha.view(T, H, D))
    o = rms_norm(o, _w(tensors, p + "norm"), eps).reshape(T, H * V)
    return (o * silu(h @ _w(tensors, p + "g").T)) @ _w(tensors, p + "o").T


def lightning_attention(h, p: str, c: Mapping, tensors, eps: float) -> torch.Tensor:
    """Mixer 'lightning': silu on q, k, v, a fixed decay per head, the heads normed together, a sigmoid gate."""
    T = h.shape[0]
    H, D, V = int(c["heads"]), int(c["dim"]), int(c["vdim"])
    q = silu(h @ _w(tensors, p + "q").T).view(T, H, D)
    k = silu(h @ _w(tensors, p + "k").T).view(T, H, D)
    v = silu(h @ _w(tensors, p + "v").T).view(T, H, V)
    decay = torch.tensor(c["decay"], dtype=F64)[None, :, None].expand(T, H, D)
    o = linear_recurrence(q, k, v, decay).reshape(T, H * V)
    o = rms_norm(o, _w(tensors, p + "norm"), eps)
    return (o * torch.sigmoid(h @ _w(tensors, p + "g").T)) @ _w(tensors, p + "o").T


def mixer(kind: str, h, positions, p: str, c: Mapping, tensors, eps: float) -> torch.Tensor:
    if kind == "parallel":
        return (float(c["left_scale"]) * attention_full_norm(h, positions, p + "left.", c["left"], tensors, eps)
                + float(c["right_scale"]) * recurrent_block(h, p + "right.", c["right"], tensors))
    if kind == "parallel_2":
        return (float(c["left_scale"]) * attention_conv_window(h, positions, p + "left.", c["left"], tensors, eps)
                + float(c["right_scale"]) * gated_linear_attention(h, p + "right.", c["right"], tensors, eps))
    if kind == "lightning":
        return lightning_attention(h, p, c, tensors, eps)
    raise ValueError(kind)


# ---------------------------------------------------------------------------------------------- feed-forwards
def dense_ff(h, p: str, c: Mapping, tensors) -> torch.Tensor:
    limit = float(c["limit"])
    g = (h @ _w(tensors, p + "gate").T).clamp(max=limit)
    u = (h @ _w(tensors, p + "up").T).clamp(-limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ _w(tensors, p + "down").T


def route(z: torch.Tensor, correction: torch.Tensor, top: int, groups: int, keep: int, tilt: float = 0.0):
    """z [T, E] router logits -> (chosen experts [T, top], their weights, how close each token's choice was).  Scores
    sigmoid(z); the choice adds the correction; a group's mark is the sum of its two largest choice scores (its one
    score if it has one expert); experts outside the best ``keep`` groups cannot be chosen (their choice scores count as
    minus infinity); the weights are the scores without the correction.  ``tilt`` pushes the choice scores of even
    experts up and of odd ones down by that much (to find the tokens whose choice hangs on a rounding); the third result
    is the smallest gap between something chosen and something not (groups' marks, then choice scores)."""
    T, E = z.shape
    s = torch.sigmoid(z)
    c = s + correction + tilt * (1.0 - 2.0 * (torch.arange(E) % 2)).to(F64)
    per = E // groups
    margin = torch.full((T,), math.inf, dtype=F64)
    if groups > 1 and keep < groups:
        mark = c.view(T, groups, per).topk(min(2, per), -1).values.sum(-1)
        best = mark.topk(keep + 1, -1)
        margin = best.values[:, keep - 1] - best.values[:, keep]
        kept = torch.zeros(T, groups, dtype=torch.bool)
        kept.scatter_(1, best.indices[:, :keep], True)
        c = c.masked_fill(~kept[:, :, None].expand(T, groups, per).reshape(T, E), -math.inf)
    order = c.topk(min(top + 1, E), -1)
    if top < E:
        margin = torch.minimum(margin, order.values[:, top - 1] - order.values[:, top])
    idx = order.indices[:, :top]
    return idx, s.gather(1, idx), margin


def moe_ff(h, p: str, c: Mapping, tensors, tilt: float = 0.0):
    r = c["router"]
    E, top = int(r["experts"]), int(r["top"])
    g = r.get("groups") or {"count": 1, "keep": 1}
    idx, wgt, margin = route(h @ _w(tensors, p + "router").T, _w(tensors, p + "correction"), top, int(g["count"]),
                             int(g["keep"]), tilt)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            a = silu(_w(tensors, f"{p}e{e}.gate") @ h[t]) * (_w(tensors, f"{p}e{e}.up") @ h[t])
            out[t] += wgt[t, j] * (_w(tensors, f"{p}e{e}.down") @ a)
    return out, margin


# ---------------------------------------------------------------------------------------------- the model
def forward(config: Mapping, tensors: Mapping[str, torch.Tensor], tokens: List[int], tilt: float = 0.0):
    """-> (logits [T, vocab], the stream after every layer [layers, T, width], every token's closest routing call)."""
    eps = float(config["norm"]["eps"])
    T = len(tokens)
    positions = torch.arange(T)
    x = _w(tensors, "embed")[torch.tensor(tokens)] * float((config.get("embedding") or {}).get("scale", 1.0))
    streams = []
    margin = torch.full((T,), math.inf, dtype=F64)
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = rms_norm(x, _w(tensors, p + "norm1"), eps, True)
        x = x + rms_norm(mixer(layer["type"], h, positions, p + "mix.", layer["mixer"], tensors, eps),
                         _w(tensors, p + "norm1b"), eps, True)
        ff = layer.get("mlp")
        if ff is not None:
            h = rms_norm(x, _w(tensors, p + "norm2"), eps, True)
            if ff["kind"] == "dense":
                y = dense_ff(h, p + "mlp.", ff, tensors)
            else:
                y, m = moe_ff(h, p + "mlp.", ff, tensors, tilt)
                margin = torch.minimum(margin, m)
            x = x + rms_norm(y, _w(tensors, p + "norm2b"), eps, True)
        streams.append(x.clone())
    h = rms_norm(x, _w(tensors, "final.norm"), eps, True)
    logits = h @ _w(tensors, "head").T
    cap = config.get("logit_softcap")
    if cap:
        logits = float(cap) * torch.tanh(logits / float(cap))
    return logits, torch.stack(streams), margin
