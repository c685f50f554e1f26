"""Sudupel without a GPU: the configuration reader (defaults, refusals, round trip, tensor names), and the plain
implementation checked by hand on tiny inputs and against itself."""
import copy
import math

import pytest
import torch

import plain_sudupel as P
from sudupel_helpers import SUDU, changed, make_tensors


def test_the_reader_round_trips_and_lowers_every_layer():
    from zlm_b200.registry import config_from_dict
    from zlm_b200.parts.model import DecoderModel
    for name, d in SUDU.items():
        cfg = config_from_dict(d)
        again = config_from_dict(cfg.to_dict())
        assert again == cfg, name
        spec = cfg.to_model_spec()
        assert [l.arrangement for l in spec.layers] == ["sandwich_norm"] * len(d["layers"])
        kinds = [l.mixer.kind for l in spec.layers]
        assert kinds == ["parallel" if l["type"] != "lightning" else "retention" for l in d["layers"]]
        names = DecoderModel(spec).param_specs()
        for i, l in enumerate(d["layers"]):
            assert f"l{i}.norm1" in names and f"l{i}.norm1b" in names
            assert (f"l{i}.norm2b" in names) == (l["mlp"] is not None)
            if l["type"] == "parallel":
                assert names[f"l{i}.mix.left.q.norm"].shape == (l["mixer"]["left"]["heads"] * l["mixer"]["left"]["dim"],)
                assert names[f"l{i}.mix.right.ra"].shape[0] == l["mixer"]["right"]["blocks"]
                assert f"l{i}.mix.left.q.conv" not in names
            if l["type"] == "parallel_2":
                assert names[f"l{i}.mix.left.k.norm"].shape == (l["mixer"]["left"]["dim"],)
                assert names[f"l{i}.mix.right.a2"].shape == (l["mixer"]["right"]["heads"] * l["mixer"]["right"]["dim"],
                                                              l["mixer"]["right"]["rank"])
            if l["type"] == "lightning":
                assert names[f"l{i}.mix.norm"].shape == (l["mixer"]["heads"] * l["mixer"]["vdim"],)
        assert "embed" in names and "head" in names and "final.norm" in names


def test_a_rank_that_no_key_names_is_left_to_the_checkpoint():
    from zlm_b200.registry import config_from_dict
    from zlm_b200.parts.model import DecoderModel
    d = copy.deepcopy(SUDU["A"])
    del d["layers"][1]["mixer"]["right"]["rank"]
    names = DecoderModel(config_from_dict(d).to_model_spec()).param_specs()
    a1, a2 = names["l1.mix.right.a1"], names["l1.mix.right.a2"]
    assert a1.shape == (-1, 64) and a2.shape == (48, -1)
    assert a1.fits((5, 64)) and a1.fits((16, 64)) and not a1.fits((5, 63)) and a2.fits((48, 7)) and not a2.fits((47, 7))


def test_defaults_and_refusals():
    from zlm_b200 import ConfigError
    from zlm_b200.registry import config_from_dict
    cfg = config_from_dict(SUDU["B"])
    assert cfg.embedding_scale == 1.0 and cfg.logit_softcap == 0.0
    assert cfg.layers[3].mlp.groups == 3 and config_from_dict(SUDU["A"]).layers[3].mlp.groups == 1
    assert config_from_dict(SUDU["A"]).layers[4].mixer.left.rot is None
    bad = [(("layers", 0, "type"), "parallel_3", "type"), (("layers", 0, "mixer", "left", "kv_heads"), 3, "kv_heads"),
           (("layers", 0, "mixer", "right", "blocks"), 5, "blocks"), (("layers", 0, "mlp", "limit"), 0.0, "limit"),
           (("layers", 1, "mlp", "router", "top"), 9, "top"), (("layers", 1, "mlp", "router", "groups", "keep"), 5, "groups"),
           (("layers", 2, "mixer", "decay"), [0.5], "decay"), (("layers", 0, "mixer", "left", "rot", "dims"), 26, "dims"),
           (("layers", 1, "mixer", "right", "tau"), 0.0, "tau"), (("layers", 0, "mlp", "kind"), "sparse", "kind")]
    for path, value, word in bad:
        with pytest.raises(ConfigError, match=word):
            config_from_dict(changed(SUDU["A"], path, value))
    d = copy.deepcopy(SUDU["A"])
    del d["layers"][0]["mixer"]["left"]["scale"]
    with pytest.raises(ConfigError, match="scale"):
        config_from_dict(d)


def test_rotation_frequencies_by_hand():
    f, m = P.rotary_frequencies({"base": 100.0, "dims": 4})
    assert torch.allclose(f, torch.tensor([1.0, 0.1], dtype=torch.float64)) and m == 1.0
    # the blend: where(t) = dims ln(original / (2 pi t)) / (2 ln base)
    r = {"base": 10000.0, "dims": 8, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}}
    f, m = P.rotary_frequencies(r)
    where = lambda t: 8 * math.log(64 / (2 * math.pi * t)) / (2 * math.log(10000.0))
    lo, hi = max(math.floor(where(8.0)), 0), min(math.ceil(where(1.0)), 7)
    assert (lo, hi) == (0, 2) and abs(m - (0.1 * math.log(4.0) + 1.0)) < 1e-15
    plain = [10000.0 ** (-2 * i / 8) for i in range(4)]
    ramp = [0.0, 0.5, 1.0, 1.0]
    for i in range(4):
        assert abs(float(f[i]) - (plain[i] / 4.0 * ramp[i] + plain[i] * (1 - ramp[i]))) < 1e-15
    # the rotation turns the pair (i, i + dims/2) and leaves what lies beyond dims
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0]]], dtype=torch.float64)
    y = P.rotate(x, torch.tensor([3]), {"base": 100.0, "dims": 4})[0, 0]
    a0, a1 = 3.0, 0.3
    want = [math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1), 3 * math.cos(a0) + math.sin(a0),
            4 * math.cos(a1) + 2 * math.sin(a1), 5.0]
    assert torch.allclose(y, torch.tensor(want, dtype=torch.float64))


def test_softmax_with_a_sink_and_a_window_by_hand():
    q = torch.zeros(3, 1, 2, dtype=torch.float64)
    k = torch.zeros(3, 1, 2, dtype=torch.float64)
    v = torch.tensor([[[1.0]], [[2.0]], [[4.0]]], dtype=torch.float64)
    # all scores 0: the sink holds one share of n + 1
    o = P.softmax_attention(q, k, v, 1.0, 0, True)
    assert torch.allclose(o[:, 0], torch.tensor([1 / 2, 3 / 3, 7 / 4], dtype=torch.float64))
    o = P.softmax_attention(q, k, v, 1.0, 2, False)          # itself and one token before it
    assert torch.allclose(o[:, 0], torch.tensor([1.0, 1.5, 3.0], dtype=torch.float64))


def test_recurrences_by_hand():
    # one head, one key channel, one value: S_t = a_t S + k_t v_t, o = S q
    q = torch.tensor([1.0, 2.0, 1.0], dtype=torch.float64).view(3, 1, 1)
    k = torch.tensor([1.0, 1.0, 3.0], dtype=torch.float64).view(3, 1, 1)
    v = torch.tensor([2.0, 1.0, 1.0], dtype=torch.float64).view(3, 1, 1)
    a = torch.tensor([0.5, 0.5, 0.1], dtype=torch.float64).view(3, 1, 1)
    o = P.linear_recurrence(q, k, v, a).flatten()
    assert torch.allclose(o, torch.tensor([2.0, 2 * (0.5 * 2 + 1), 0.1 * 2 + 3], dtype=torch.float64))
    # the convolution: the last column is the current token's
    u = torch.tensor([[1.0], [2.0], [3.0]], dtype=torch.float64)
    y = P.causal_conv(u, torch.tensor([[10.0, 1.0]], dtype=torch.float64), torch.tensor([0.5], dtype=torch.float64))
    assert torch.allclose(y.flatten(), torch.tensor([1.5, 12.5, 23.5], dtype=torch.float64))


def test_routing_by_hand():
    # two groups of three; the first group has the single best expert, the second the best two: the second is kept
    s = torch.tensor([[0.9, 0.2, 0.1, 0.6, 0.55, 0.15]], dtype=torch.float64)
    z = torch.log(s / (1 - s))
    idx, wgt, margin = P.route(z, torch.zeros(6, dtype=torch.float64), 2, 2, 1)
    assert idx.tolist() == [[3, 4]] and torch.allclose(wgt, s[:, 3:5])
    assert abs(float(margin) - min(1.15 - 1.1, 0.55 - 0.15)) < 1e-12
    # the correction moves the choice and not the weight; refused groups do not come back although the scores left
    # are negative
    corr = torch.tensor([0.0, 0.0, 0.0, -2.0, -2.0, -2.0], dtype=torch.float64)
    idx, wgt, _ = P.route(z, corr, 2, 2, 1)
    assert idx.tolist() == [[0, 1]] and torch.allclose(wgt, s[:, :2])
    corr = torch.tensor([-3.0, -3.0, -3.0, -2.0, -2.0, -2.0], dtype=torch.float64)
    idx, wgt, _ = P.route(z, corr, 3, 2, 1)
    assert sorted(idx.tolist()[0]) == [3, 4, 5]


def test_dense_feed_forward_clamps_by_hand():
    t = {"gate": torch.tensor([[2.0], [-3.0]], dtype=torch.float64), "up": torch.tensor([[3.0], [-3.0]], dtype=torch.float64),
         "down": torch.eye(2, dtype=torch.float64)}
    y = P.dense_ff(torch.ones(1, 1, dtype=torch.float64), "", {"limit": 1.5}, t)[0]
    g0, g1 = 1.5, -3.0
    want = [g0 / (1 + math.exp(-1.702 * g0)) * (1.5 + 1), g1 / (1 + math.exp(-1.702 * g1)) * (-1.5 + 1)]
    assert torch.allclose(y, torch.tensor(want, dtype=torch.float64))


def test_the_whole_model_is_causal_and_what_a_window_hides_stays_hidden():
    cfg = SUDU["A"]
    ref = {n: t.double() for n, t in make_tensors(cfg, 3).items()}
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, cfg["vocab"], (40,), generator=g).tolist()
    full = P.forward(cfg, ref, ids)[0]
    head = P.forward(cfg, ref, ids[:25])[0]
    assert torch.allclose(full[:25], head, atol=1e-9)
