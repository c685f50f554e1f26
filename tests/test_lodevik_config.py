"""Lodevik without a GPU: the configuration (reading, refusing, writing back, lowering to parts), the checkpoint's
tensor names, and the oracle's own invariants (small cases by hand, whole sequences against their prefixes)."""
import copy
import math

import pytest
import torch

import plain_lodevik as P
from lodevik_helpers import LODE, LODE_A, LODE_B, make_tensors


def test_architecture_is_chosen_by_its_string_key():
    from zlm_b200 import LodevikConfig
    from zlm_b200.registry import config_from_dict
    for d in (LODE_A, LODE_B):
        cfg = config_from_dict(d)
        assert isinstance(cfg, LodevikConfig)
        assert config_from_dict(cfg.to_dict()) == cfg
        assert len(cfg.to_dict()["layers"]) == len(d["layers"])


@pytest.mark.parametrize("name", sorted(LODE))
def test_lowering_names_parts_and_tensors(name):
    from zlm_b200.parts.model import DecoderModel
    from zlm_b200.registry import config_from_dict
    d = LODE[name]
    spec = config_from_dict(d).to_model_spec()
    assert [l.mixer.kind for l in spec.layers] == [{"latent_attention": "latent_attention", "attention": "diff_attention"}[l["type"]]
                                                   for l in d["layers"]]
    specs = {n: tuple(s.shape) for n, s in DecoderModel(spec).param_specs().items() if not s.ignorable}
    W = d["width"]
    want = {"embed": (d["vocab"], W), "final.norm": (W,)}
    bg = (d.get("embedding") or {}).get("bigram")
    if bg:
        want["bigram"] = (bg["buckets"] + 1, W)
    for i, l in enumerate(d["layers"]):
        m, p = l["mixer"], f"l{i}."
        want[p + "norm1"] = want[p + "ls1"] = (W,)
        if l["type"] == "latent_attention":
            H = m["heads"]
            want.update({p + "mix.q": (H * (m["dim"] + m["rot_dim"]), W), p + "mix.dkv": (m["kv_rank"] + m["rot_dim"], W),
                         p + "mix.dkv.norm": (m["kv_rank"],), p + "mix.uk": (H * m["dim"], m["kv_rank"]),
                         p + "mix.uv": (H * m["vdim"], m["kv_rank"]), p + "mix.sink": (H,), p + "mix.g": (H, W),
                         p + "mix.o": (W, H * m["vdim"])})
        else:
            H, G, D = m["heads"], m["kv_heads"], m["dim"]
            want.update({p + "mix.q": (H * 2 * D, W), p + "mix.k": (G * 2 * D, W), p + "mix.v": (G * m["vdim"], W),
                         p + "mix.o": (W, H * m["vdim"]), p + "mix.q.norm": (D,), p + "mix.k.norm": (D,)})
            for n in ("lq1", "lk1", "lq2", "lk2"):
                want[p + "mix." + n] = (D,)
        if l["mlp"] is not None:
            want[p + "norm2"] = want[p + "ls2"] = (W,)
            want[p + "mlp.gate"] = want[p + "mlp.up"] = (l["mlp"]["ff"], W)
            want[p + "mlp.down"] = (W, l["mlp"]["ff"])
    assert specs == want


def _bad(change):
    d = copy.deepcopy(LODE_A)
    change(d)
    return d


@pytest.mark.parametrize("change, word", [
    (lambda d: d.pop("vocab"), "vocab"),
    (lambda d: d["norm"].pop("eps"), "eps"),
    (lambda d: d["layers"][0].update(type="retention"), "type"),
    (lambda d: d["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=26), "rot.dims"),
    (lambda d: d["layers"][0]["mixer"]["mask"].update(size=0), "mask.size"),
    (lambda d: d["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda d: d["layers"][0]["mixer"].pop("diff"), "diff"),
    (lambda d: d["layers"][0]["mlp"].update(kind="moe"), "mlp.kind"),
    (lambda d: d["layers"][0]["mlp"].update(ff=0), "mlp.ff"),
    (lambda d: d["embedding"]["bigram"].update(buckets=0), "bigram"),
    (lambda d: d.update(layers=[]), "layers"),
])
def test_refusals_name_the_key(change, word):
    from zlm_b200 import ConfigError
    from zlm_b200.registry import config_from_dict
    with pytest.raises(ConfigError) as e:
        config_from_dict(_bad(change))
    assert word in str(e.value)


def test_optional_keys_have_their_plain_meaning():
    from zlm_b200.registry import config_from_dict
    d = copy.deepcopy(LODE_A)
    d.pop("logit_scale")
    d["embedding"].pop("bigram")
    d["embedding"].pop("scale")
    for l in d["layers"]:
        l["mixer"].pop("rot", None)
        l["mixer"].pop("mask", None)
        l["mixer"].pop("softcap", None)
    spec = config_from_dict(d).to_model_spec()
    back = config_from_dict(d).to_dict()
    assert back.get("logit_scale", 1.0) == 1.0 and (back.get("embedding") or {}).get("scale", 1.0) == 1.0
    assert not (back.get("embedding") or {}).get("bigram")
    from zlm_b200.parts.model import DecoderModel
    assert "bigram" not in DecoderModel(spec).param_specs()


# ------------------------------------------------------------------------------------------------ the oracle by hand
def test_visible_by_hand():
    ok = P.visible(5, 2).tolist()
    assert ok == [[True, False, False, False, False], [True, True, False, False, False],
                  [False, False, True, False, False], [False, False, True, True, False],
                  [False, False, False, False, True]]
    assert P.visible(3).tolist() == [[True, False, False], [True, True, False], [True, True, True]]


def test_softmax_with_sink_by_hand():
    s = torch.zeros(1, 1, 1, dtype=P.F)
    ok = torch.ones(1, 1, dtype=torch.bool)
    assert float(P.softmax_with_sink(s, ok)[0, 0, 0]) == 1.0
    assert abs(float(P.softmax_with_sink(s, ok, torch.zeros(1))[0, 0, 0]) - 0.5) < 1e-15
    # a sink of ln 3 against one key of score 0: the key keeps a quarter
    assert abs(float(P.softmax_with_sink(s, ok, torch.tensor([math.log(3.0)], dtype=P.F))[0, 0, 0]) - 0.25) < 1e-15


def test_rotation_and_activation_by_hand():
    x = torch.tensor([[1.0, 0.0, 5.0, 7.0, 2.0, 3.0]], dtype=P.F).repeat(2, 1)
    # base 1: every pair turns by the position itself; dims 4 leaves the last two coordinates alone
    y = P.rotate_pairs(x, torch.tensor([0, 1]), 1.0, 4)
    assert torch.equal(y[0], x[0])
    c, s = math.cos(1.0), math.sin(1.0)
    want = torch.tensor([c, s, 5 * c - 7 * s, 7 * c + 5 * s, 2.0, 3.0], dtype=P.F)
    assert float((y[1] - want).abs().max()) < 1e-15
    assert abs(float(P.gelu_tanh(torch.tensor(1.0, dtype=P.F))) - 0.8411919906082768) < 1e-12
    assert abs(float(P.unit_rms(torch.tensor([3.0, 4.0], dtype=P.F), 0.0)[0]) - 3.0 / math.sqrt(12.5)) < 1e-15


def test_pair_table_rows_by_hand():
    table = torch.arange(10, dtype=P.F)[:, None].repeat(1, 2)
    pair = 100.0 * torch.arange(8, dtype=P.F)[:, None].repeat(1, 2)
    x = P.embed([3, 4, 9], table, 2.0, pair, 7, 5, 3)
    # first token: the last row (7); then (3 * 5 + 4 * 3) % 7 = 6 and (4 * 5 + 9 * 3) % 7 = 5
    assert x[:, 0].tolist() == [6.0 + 700.0, 8.0 + 600.0, 18.0 + 500.0]


def test_diff_lambda_by_hand():
    w = {"lq1": torch.tensor([1.0, 2.0]), "lk1": torch.tensor([0.5, 0.25]), "lq2": torch.tensor([0.0, 1.0]),
         "lk2": torch.tensor([3.0, 0.0])}
    assert abs(P.diff_lambda(w, 0.3) - (math.e - 1.0 + 0.3)) < 1e-12


@pytest.mark.parametrize("name", sorted(LODE))
def test_a_prefix_gives_the_same_logits(name):
    """Causality of the whole oracle: the logits of a prefix are the first rows of the whole sequence's."""
    cfg = LODE[name]
    ref = {n: t.double() for n, t in make_tensors(cfg, 3).items()}
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, cfg["vocab"], (150,), generator=g).tolist()
    whole = P.forward(cfg, ref, ids)
    for k in (1, 2, 49, 71, 131):
        part = P.forward(cfg, ref, ids[:k])
        assert float((part - whole[:k]).abs().max()) < 1e-9


def test_chunks_hide_what_lies_before_them():
    """A one-layer differential model with chunks of 8: the logits from position 8 on do not depend on the tokens
    before position 7 (position 7 is the token before position 8 in the pair table), and do depend on them without
    chunks."""
    cfg = copy.deepcopy(LODE_A)
    cfg["layers"] = cfg["layers"][:1]
    cfg["layers"][0]["mixer"]["mask"] = {"size": 8}
    ref = {n: t.double() for n, t in make_tensors(cfg, 4).items()}
    a = [5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15, 16]
    b = [50, 60, 70, 80, 90, 100, 110, 12, 13, 14, 15, 16]
    la, lb = P.forward(cfg, ref, a), P.forward(cfg, ref, b)
    assert float((la[8:] - lb[8:]).abs().max()) < 1e-9 and float((la[7] - lb[7]).abs().max()) > 1e-3
    cfg["layers"][0]["mixer"].pop("mask")
    la, lb = P.forward(cfg, ref, a), P.forward(cfg, ref, b)
    assert float((la[8:] - lb[8:]).abs().max()) > 1e-3
