"""Small Sudupel configurations and weights for the tests, and the oracle's inputs.

The configurations differ from each other, and from layer to layer, in every size and option: head counts (also 1,
also 18 query heads on one kv head, also kv heads = heads), key and value sizes that differ both ways and are no
multiples of 16 (keys wider than 128 too), convolutions of 1 to 8 taps and none, windows below a page, of exactly a
page, a little above two pages, and none, rotation over a part of a head, over all of it and none, with and without
the long-context blend of the frequencies, recurrent blocks of 1 to 6 diagonal blocks, decay ranks of 3 to 10,
temperatures of 1 to 12, routers with and without groups, one to four experts a token, dense layers with limits that
bite and that do not, a layer without a feed-forward, with and without embedding scale and logit cap.

Weights are drawn so that activations are of order one (matrices N(0, 1/in)): attention and routing then depend
visibly on single keys and experts, which N(0, 0.02) would hide."""
from __future__ import annotations

import copy
import json
import os
from typing import Dict, List, Sequence

import torch

import plain_sudupel as P


def att(heads, kv_heads, dim, vdim, scale, rot=None, conv=0, window=0):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot:
        m["rot"] = rot
    if conv:
        m["conv"] = conv
    if window:
        m["mask"] = {"size": window}
    return m


def rot(base, dims, scaling=None):
    r = {"base": base, "dims": dims}
    if scaling:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def rec(width, blocks, conv):
    return {"width": width, "blocks": blocks, "conv": conv}


def gla(heads, dim, vdim, tau, rank):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank}


def pair(left, right, ls, rs):
    return {"left": left, "right": right, "left_scale": ls, "right_scale": rs}


def light(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(ff, experts, top, count=None, keep=None):
    r = {"experts": experts, "top": top}
    if count:
        r["groups"] = {"count": count, "keep": keep}
    return {"kind": "moe", "expert": {"ff": ff}, "router": r}


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


SUDU_A = {
    "architecture": "Sudupel", "vocab": 160, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 4.0},
    "logit_softcap": 20.0,
    "layers": [
        layer("parallel", pair(att(4, 2, 24, 16, 0.3, rot(10000.0, 16, (4.0, 64, 8.0, 1.0))), rec(48, 3, 3), 0.7, 1.1), dense(40, 1.0)),
        layer("parallel_2", pair(att(3, 3, 16, 40, 0.5, rot(500.0, 16), conv=2, window=9), gla(2, 24, 20, 8.0, 6), 0.8, 0.5),
              moe(24, 8, 3, 4, 2)),
        layer("lightning", light(2, 40, 12, [0.9, 0.995]), None),
        layer("parallel_2", pair(att(2, 1, 32, 32, 0.35, conv=4, window=70), gla(1, 8, 64, 2.0, 3), 1.0, 1.3), moe(16, 6, 1)),
        layer("parallel", pair(att(2, 2, 8, 8, 1.0), rec(64, 1, 1), 1.2, 0.4), dense(32, 5.0)),
    ],
}
# wider; 18 query heads on one kv head; keys wider than 128; a window of exactly a page; eight taps; no embedding
# scale and no cap
SUDU_B = {
    "architecture": "Sudupel", "vocab": 200, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        layer("parallel_2", pair(att(18, 1, 16, 16, 0.5, rot(100.0, 8), conv=3, window=130), gla(4, 40, 8, 12.0, 10), 0.6, 0.9),
              dense(96, 2.0)),
        layer("lightning", light(3, 16, 24, [0.5, 0.97, 0.9999]), None),
        layer("parallel", pair(att(4, 2, 152, 8, 0.08, rot(40000.0, 152, (16.0, 32, 4.0, 0.5))), rec(96, 6, 4), 0.9, 0.8),
              moe(8, 4, 2, 2, 1)),
        layer("parallel_2", pair(att(2, 2, 64, 128, 0.2, rot(2e5, 64), conv=8, window=64), gla(2, 128, 16, 1.0, 8), 1.0, 1.0),
              moe(48, 12, 4, 3, 2)),
    ],
}
SUDU = {"A": SUDU_A, "B": SUDU_B}


def make_tensors(cfg_dict, seed: int) -> Dict[str, torch.Tensor]:
    """fp32 tensors by checkpoint name, every one rounded to bfloat16 values (so that both engine dtypes and the
    oracle compute on the same numbers)."""
    from zlm_b200.parts.model import DecoderModel
    from zlm_b200.registry import config_from_dict
    specs = DecoderModel(config_from_dict(cfg_dict).to_model_spec()).param_specs()
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name in sorted(specs):
        shape = specs[name].concrete_shape()
        last = name.rsplit(".", 1)[-1]
        if last in ("norm1", "norm2", "norm1b", "norm2b") or name == "final.norm":
            t = 0.2 * torch.randn(shape, generator=g)                  # stored around zero: the norm multiplies by 1 + w
        elif last == "correction":
            t = 0.1 * torch.randn(shape, generator=g)
        elif last == "lam":
            t = -2.5 + torch.randn(shape, generator=g)                  # decays between 0.3 and 0.98
        elif name.endswith(".a2.b"):
            t = 2.0 + torch.randn(shape, generator=g)
        elif last == "b":
            t = 0.3 * torch.randn(shape, generator=g)                   # biases
        elif last == "norm":
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)             # plain norm weights
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        elif last == "conv":
            t = torch.randn(shape, generator=g) * 0.7
        elif last in ("ra", "ri"):
            t = torch.randn(shape, generator=g) / shape[-1] ** 0.5
        else:
            t = torch.randn(shape, generator=g) / shape[-1] ** 0.5
            if last == "router":
                t = t * float(ROUTER_GAIN)          # scores spread over (0, 1): few choices hang on a close call
            if last == "a2":
                t = t * 2.0          # decays that differ from channel to channel and token to token
        out[name] = t.to(torch.bfloat16).float()
    return out


def write_model(tmp_path, cfg, tensors, tag: str):
    from zlm_b200.weights import write_safetensors
    folder = os.path.join(str(tmp_path), f"sudu_{tag}")
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), {n: t.to(torch.bfloat16) for n, t in tensors.items()})
    return folder


def make_model(tmp_path, name: str, seed: int = 0):
    """Writes the model to a folder; returns (folder, config mapping, float64 tensors for the oracle)."""
    cfg = SUDU[name]
    tensors = make_tensors(cfg, seed)
    return write_model(tmp_path, cfg, tensors, f"{name}_{seed}"), cfg, {n: t.double() for n, t in tensors.items()}


def one_layer(kind, mixer, mlp=None, width=64, vocab=96, **top):
    """A model of one layer around the mechanism under test."""
    cfg = {"architecture": "Sudupel", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
           "layers": [layer(kind, mixer, mlp)]}
    cfg.update(top)
    return cfg


def engine_for(tmp_path, cfg, tensors, dtype, tag, **kw):
    from zlm_b200 import Engine
    kw.setdefault("max_tokens", 2048)
    return Engine.from_pretrained(write_model(tmp_path, cfg, tensors, tag), dtype=dtype, **kw)


# how far a bfloat16 run's choice scores may be from the oracle's: activations rounded to 8 bits of mantissa move a
# router's sigmoid scores by a few thousandths
CLOSE_CALL = 0.02
ROUTER_GAIN = 2.0


class Oracle:
    """The oracle's logits of one sequence, and which positions do not hang on a router's close call (all of them in
    32-bit).  A bfloat16 run may choose another expert or group where two choice scores nearly tie; it then computes
    another function at that position and, through windows and states, at later ones.  So the oracle runs twice more
    with the choice scores pushed by CLOSE_CALL one way and the other; positions whose logits move, and positions with
    a close call of their own, are not compared; nor are positions that a rounding of the embeddings alone moves by
    4 % and more."""

    def __init__(self, tensors, cfg, ids: Sequence[int], dtype: str):
        logits, _, margin = P.forward(cfg, tensors, ids)
        self.logits = logits.float()
        self.safe = torch.ones(len(ids), dtype=torch.bool)
        if dtype != "float32" and any((l.get("mlp") or {}).get("kind") == "moe" for l in cfg["layers"]):
            self.safe &= margin >= CLOSE_CALL
            for tilt in (CLOSE_CALL, -CLOSE_CALL):
                other = P.forward(cfg, tensors, ids, tilt=tilt)[0]
                self.safe &= (other - logits).norm(dim=-1) <= 0.02 * logits.norm(dim=-1)
        if dtype != "float32":
            # positions where the design itself multiplies a rounding tenfold (a recurrence's output at a sequence's
            # first positions is one or two terms, (q.k) v, whose sign decides everything once the heads are divided
            # by their root mean square): three more runs on embeddings moved by a bfloat16 rounding or two (a relative 2^-7);
            # where that moves the logits by 4 % and more, no bfloat16 run can be held to the oracle
            for seed in (77, 78, 79):
                g = torch.Generator().manual_seed(seed)
                moved = dict(tensors)
                moved["embed"] = tensors["embed"] * (1.0 + 2.0 ** -7 * (2.0 * torch.rand(tensors["embed"].shape, generator=g,
                                                                                          dtype=torch.float64) - 1.0))
                other = P.forward(cfg, moved, ids)[0]
                self.safe &= (other - logits).norm(dim=-1) <= 0.04 * logits.norm(dim=-1)
            # (a sign that turns among a sequence's first tokens stays in the young states for a while: the 16 positions
            # after such a position are left out with it)
            for t in [t for t in range(min(16, len(ids))) if not bool(self.safe[t])]:
                self.safe[t:t + 16] = False

    def check(self, got: torch.Tensor, places, dtype: str, what: str = "") -> None:
        places = list(places)
        keep = [i for i, p in enumerate(places) if bool(self.safe[p])]
        assert len(keep) * 10 >= len(places) or len(places) < 32, f"{what}: too many close calls to test anything"
        if keep:
            assert_rows_close(got.float().cpu().reshape(len(places), -1)[keep], self.logits[[places[i] for i in keep]],
                              dtype, what)


def oracle(tensors, cfg, ids, dtype) -> Oracle:
    return Oracle(tensors, cfg, ids, dtype)


# rows are compared as vectors after their means are taken off (a capped head moves all logits of a row alike):
# |got - want|_2 <= row * |want|_2.  bfloat16: activations are rounded to 8 bits of mantissa between kernels while the
# oracle keeps 64-bit ones; every row has a loose bound and the median of many rows a tight one.  A wrong key, expert,
# state or position shows as tens of per cent (and to four digits in the 32-bit runs of the same kernels).  In bfloat16
# one row in twenty-five may pass the loose bound, up to OUTLIER_TOL: single positions where a clamp, a peaked softmax
# or a small sum that is divided by its root mean square multiplies a rounding (the same rows however the prompt is
# cut).
ROW_TOL = {"float32": 2e-4, "bfloat16": 8e-2}
MEDIAN_TOL = {"float32": 1e-4, "bfloat16": 2.5e-2}
OUTLIER_TOL = 0.3


def assert_rows_close(got: torch.Tensor, want: torch.Tensor, dtype: str, what: str = "", tol=None):
    got, want = got.float().cpu(), want.float().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    if got.dim() == 1:
        got, want = got[None], want[None]
    rel = (got - want).norm(dim=-1) / want.norm(dim=-1).clamp_min(1e-9)
    outliers = 0 if (dtype == "float32" or tol is not None) else max(1, len(rel) // 25)
    tol = tol or ROW_TOL[dtype]
    over = (rel > tol).nonzero().flatten().tolist()
    assert len(over) <= outliers and (not over or float(rel.max()) <= OUTLIER_TOL), (
        f"{what}: row {int(rel.argmax())} differs by {rel.max():.3e} of its norm; rows over {tol}: {over[:12]}")
    if len(rel) >= 8:
        assert float(rel.median()) <= MEDIAN_TOL[dtype], f"{what}: the median row differs by {rel.median():.3e} of its norm"


def prompts(vocab: int, lengths: Sequence[int], seed: int) -> List[List[int]]:
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]


def greedy_generate(tensors, cfg, prompt: Sequence[int], n: int) -> List[int]:
    """The oracle's greedy continuation (the whole sequence is run anew for every token: the oracle keeps no state)."""
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(torch.argmax(P.forward(cfg, tensors, ids)[0][-1])))
    return ids[len(prompt):]


def changed(cfg, path: Sequence, value):
    """A copy of the configuration with one value replaced (path: keys and indices from the top)."""
    c = copy.deepcopy(cfg)
    at = c
    for k in path[:-1]:
        at = at[k]
    at[path[-1]] = value
    return c
