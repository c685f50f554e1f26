"""Small Lodevik configurations and weights for the tests.

The configurations differ from each other, and from layer to layer, in every size and option: head counts (also 1,
also kv heads = heads and one kv head for all), key and value sizes that differ both ways and are no multiples of 16,
rotation over a part of a head and over all of it and none, latents narrower and wider than a head, chunks below a
page, of exactly a page, a little above it, of two pages and none, a cap on the scores that bites and none, a layer
without a feed-forward, pair tables of few and many buckets, scales other than 1.

Weights are drawn so that activations are of order one (matrices N(0, 1/in)): attention then depends visibly on
single keys, which N(0, 0.02) would hide."""
from __future__ import annotations

import json
import os
from typing import Dict, List, Sequence

import torch

import plain_lodevik as P


def _lat(heads, dim, rot_dim, vdim, kv_rank, scale, base=None, dims=0, chunk=0):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale}
    if dims:
        m["rot"] = {"base": base, "dims": dims}
    if chunk:
        m["mask"] = {"size": chunk}
    return m


def _att(heads, kv_heads, dim, vdim, scale, diff, softcap=0.0, base=None, dims=0, chunk=0):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if softcap:
        m["softcap"] = softcap
    if dims:
        m["rot"] = {"base": base, "dims": dims}
    if chunk:
        m["mask"] = {"size": chunk}
    return m


def _layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


LODE_A = {
    "architecture": "Lodevik", "vocab": 160, "width": 64, "norm": {"eps": 1e-5}, "logit_scale": 0.7,
    "embedding": {"scale": 1.5, "bigram": {"buckets": 37, "mul_prev": 11, "mul_cur": 5}},
    "layers": [
        _layer("attention", _att(4, 2, 24, 40, 0.3, 0.2, 3.0, 500.0, 8, 70), 48),
        _layer("latent_attention", _lat(3, 16, 8, 24, 40, 0.25, 10000.0, 8), 40),
        _layer("attention", _att(3, 3, 40, 8, 0.2, 0.45, 0.0, 100.0, 40, 48), 0),
        _layer("latent_attention", _lat(1, 24, 16, 8, 16, 0.2, 300.0, 4, 130), 24),
        _layer("attention", _att(2, 1, 16, 16, 0.4, 0.1, 20.0), 32),
    ],
}
# wider; a chunk of exactly a page and one of two pages; six query heads on one kv head; no pair table, no scales
LODE_B = {
    "architecture": "Lodevik", "vocab": 200, "width": 128, "norm": {"eps": 1e-6},
    "embedding": {"scale": 1.0},
    "layers": [
        _layer("latent_attention", _lat(5, 32, 32, 48, 64, 0.15, 100000.0, 32), 96),
        _layer("attention", _att(6, 1, 32, 64, 0.18, 0.35, 40.0, 20000.0, 16, 64), 64),
        _layer("latent_attention", _lat(2, 48, 16, 32, 24, 0.12, 1000.0, 16, 128), 0),
        _layer("attention", _att(2, 2, 56, 24, 0.13, 0.6, 1.5, 10.0, 56), 72),
    ],
}
LODE = {"A": LODE_A, "B": LODE_B}


def make_tensors(cfg_dict, seed: int) -> Dict[str, torch.Tensor]:
    """fp32 tensors by checkpoint name, every one rounded to bfloat16 values (so that both engine dtypes and the oracle
    compute on the same numbers)."""
    from zlm_b200.parts.model import DecoderModel
    from zlm_b200.registry import config_from_dict
    specs = DecoderModel(config_from_dict(cfg_dict).to_model_spec()).param_specs()
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name in sorted(specs):
        if specs[name].ignorable:
            continue
        shape = tuple(specs[name].shape)
        last = name.rsplit(".", 1)[-1]
        if last in ("lq1", "lk1", "lq2", "lk2"):
            t = 0.25 * torch.randn(shape, generator=g)
        elif last == "sink":
            t = torch.randn(shape, generator=g)
        elif last.startswith("ls"):
            t = 0.5 + 0.2 * torch.randn(shape, generator=g)
        elif len(shape) == 1:
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif name in ("embed", "bigram"):
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / shape[1] ** 0.5
        out[name] = t.to(torch.bfloat16).float()
    return out


def write_model(tmp_path, cfg, tensors, tag: str):
    from zlm_b200.weights import write_safetensors
    folder = os.path.join(str(tmp_path), f"lode_{tag}")
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), {n: t.to(torch.bfloat16) for n, t in tensors.items()})
    return folder


def make_model(tmp_path, name: str, seed: int = 0):
    """Writes the model to a folder; returns (folder, config mapping, float64 tensors for the oracle)."""
    cfg = LODE[name] if isinstance(name, str) else name
    tag = name if isinstance(name, str) else "custom"
    tensors = make_tensors(cfg, seed)
    return write_model(tmp_path, cfg, tensors, f"{tag}_{seed}"), cfg, {n: t.double() for n, t in tensors.items()}


def oracle_logits(tensors, cfg, ids: Sequence[int]) -> torch.Tensor:
    return P.forward(cfg, tensors, list(ids)).float()


# rows are compared as vectors: |got - want|_2 <= tol * |want|_2.  bfloat16: activations are rounded to 8 bits of
# mantissa between kernels while the oracle keeps 64-bit ones; every row has a loose bound and the median of many
# rows a tight one.  A wrong key, chunk edge, sink, state or position shows as tens of per cent (and to four digits in
# the 32-bit runs of the same kernels).
ROW_TOL = {"float32": 2e-4, "bfloat16": 8e-2}
MEDIAN_TOL = {"float32": 1e-4, "bfloat16": 2.5e-2}


def assert_rows_close(got: torch.Tensor, want: torch.Tensor, dtype: str, what: str = "", tol=None):
    got, want = got.float().cpu(), want.float().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    if got.dim() == 1:
        got, want = got[None], want[None]
    rel = (got - want).norm(dim=-1) / want.norm(dim=-1).clamp_min(1e-9)
    t = tol or ROW_TOL[dtype]
    assert float(rel.max()) <= t, (f"{what}: row {int(rel.argmax())} differs by {rel.max():.3e} of its norm; "
                                   f"rows over {t}: {(rel > t).nonzero().flatten().tolist()[:12]}")
    if len(rel) >= 8 and tol is None:
        assert float(rel.median()) <= MEDIAN_TOL[dtype], f"{what}: the median row differs by {rel.median():.3e} of its norm"


def prompts(vocab: int, lengths: Sequence[int], seed: int) -> List[List[int]]:
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]


def greedy_generate(tensors, cfg, prompt: Sequence[int], n: int) -> List[int]:
    """The oracle's greedy continuation (the whole sequence again for every token: it has no cache)."""
    ids, out = list(prompt), []
    for _ in range(n):
        tok = int(torch.argmax(P.forward(cfg, tensors, ids)[-1]))
        out.append(tok)
        ids.append(tok)
    return out
