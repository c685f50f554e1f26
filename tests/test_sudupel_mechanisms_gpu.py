"""Sudupel's mechanisms one at a time on the GPU, each as a model of one layer run through the engine (or as the
kernel alone) against the function of the plain implementation, with weights and inputs made so that a fault shows:
attention so peaked that single keys carry a query's weight (the plain implementation is first asked whether a window
that is one token off, a missing sink or another group mark would change the answer: it must), decays so close to 1
that a state from hundreds of tokens back still counts, routers whose groups decide."""
import copy
import math

import pytest
import torch

import plain_sudupel as P
from sudupel_helpers import (assert_rows_close, att, changed, dense, engine_for, gla, light, make_tensors, moe, one_layer,
                             pair, prompts, rec, rot)

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]


def run_cut(eng, ids, cuts, then_single=0):
    """The sequence in portions of the given sizes, then ``then_single`` tokens one by one; logits at every place."""
    from zlm_b200 import StepEntry
    s = eng.new_sequence()
    at, got = 0, []
    for c in list(cuts) + [1] * then_single:
        got.append(eng.step([StepEntry(s, ids[at:at + c], list(range(c)))]).clone())
        at += c
    eng.release(s)
    return torch.cat(got)


def peaked(tensors, names, by):
    out = dict(tensors)
    for n in names:
        out[n] = (out[n] * by).to(torch.bfloat16).float()
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [9, 64, 70, 130])
def test_windowed_attention_sees_exactly_its_window(tmp_path, dtype, window):
    """The windowed side alone (the other side's scale is 0), its norm weights scaled up so that the softmax is
    peaked: the plain implementation with a window one token longer or shorter gives other logits, the engine gives
    those of the right one, inside prompts, in portions that start inside a window and token by token."""
    left = att(2, 1, 16, 24, 0.9, rot(300.0, 8), conv=2, window=window)
    cfg = one_layer("parallel_2", pair(left, gla(1, 8, 8, 4.0, 4), 1.0, 0.0))
    t = peaked(make_tensors(cfg, 11), ["l0.mix.left.q.norm", "l0.mix.left.k.norm"], 1.7)
    ref = {n: x.double() for n, x in t.items()}
    n = window + 75
    (ids,) = prompts(cfg["vocab"], [n], seed=window)
    want = P.forward(cfg, ref, ids)[0]
    for other in (window + 1, window - 1):
        moved = P.forward(changed(cfg, ("layers", 0, "mixer", "left", "mask", "size"), other), ref, ids)[0]
        rel = (moved - want)[window:].norm(dim=-1) / want[window:].norm(dim=-1)
        assert int((rel > 0.02).sum()) >= 2, "the test would not see a window that is off by one"
    eng = engine_for(tmp_path, cfg, t, dtype, f"win{window}")
    tol = None if dtype == "float32" else 0.12          # (peaked attention multiplies bfloat16's rounding of q and k)
    assert_rows_close(run_cut(eng, ids, [n]), want, dtype, "whole", tol)
    assert_rows_close(run_cut(eng, ids, [window - 1, 2, 3, n - window - 4]), want, dtype, "portions", tol)
    assert_rows_close(run_cut(eng, ids, [window - 3], then_single=n - window + 3), want, dtype, "token by token", tol)


@pytest.mark.parametrize("dtype", DTYPES)
def test_full_attention_far_keys_sink_and_scaled_rotation(tmp_path, dtype):
    """The side with the norm over the whole projection, a sink and blended frequencies, 400 tokens: far keys count
    (a window would change the answer), the sink counts, the blend and its factor on cos and sin count."""
    left = att(4, 2, 16, 8, 0.8, rot(10000.0, 12, (8.0, 32, 16.0, 1.0)))
    cfg = one_layer("parallel", pair(left, rec(16, 2, 2), 1.0, 0.0))
    t = peaked(make_tensors(cfg, 12), ["l0.mix.left.q.norm", "l0.mix.left.k.norm"], 2.5)
    ref = {n: x.double() for n, x in t.items()}
    (ids,) = prompts(cfg["vocab"], [400], seed=5)
    want = P.forward(cfg, ref, ids)[0]
    no_scaling = copy.deepcopy(cfg)
    del no_scaling["layers"][0]["mixer"]["left"]["rot"]["scaling"]
    moved = P.forward(no_scaling, ref, ids)[0]
    assert float(((moved - want)[250:].norm(dim=-1) / want[250:].norm(dim=-1)).median()) > 0.05, "the blend does not show"
    # other tokens in the first 150 places change the logits 100 and more places later: far keys count
    moved = P.forward(cfg, ref, prompts(cfg["vocab"], [150], seed=6)[0] + ids[150:])[0]
    assert int(((moved - want)[250:].norm(dim=-1) / want[250:].norm(dim=-1) > 0.05).sum()) >= 10, "far keys do not show"
    eng = engine_for(tmp_path, cfg, t, dtype, "full")
    tol = None if dtype == "float32" else 0.12
    assert_rows_close(run_cut(eng, ids, [400]), want, dtype, "whole", tol)
    assert_rows_close(run_cut(eng, ids, [190, 2, 140], then_single=68), want, dtype, "portions and single tokens", tol)


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_sink_takes_its_share(dtype):
    """The attention kernels with and without the sink on one cache, prompts and single tokens, against the plain
    function: with all scores near zero the sink holds 1 / (n + 1) of the weight."""
    from zlm_b200.kernels import get_kernels, PAGE_TOKENS
    k = get_kernels()
    dt = torch.float32 if dtype == "float32" else torch.bfloat16
    g = torch.Generator().manual_seed(3)
    T, H, G, D = 70, 4, 2, 16
    q = (0.05 * torch.randn(T, H, D, generator=g)).to(dt).float()
    kk = (0.05 * torch.randn(T, G, D, generator=g)).to(dt).float()
    v = torch.randn(T, G, D, generator=g).to(dt).float()
    pool = torch.zeros(4, 2, G, PAGE_TOKENS, D, dtype=dt, device="cuda")
    table = torch.tensor([[2, 1, 0, 3]], dtype=torch.int32, device="cuda")
    for t in range(T):
        pool[int(table[0, t // PAGE_TOKENS]), 0, :, t % PAGE_TOKENS] = kk[t].to(dt).cuda()
        pool[int(table[0, t // PAGE_TOKENS]), 1, :, t % PAGE_TOKENS] = v[t].to(dt).cuda()
    pos = torch.arange(T, dtype=torch.int32, device="cuda")
    slot = torch.zeros(T, dtype=torch.int32, device="cuda")
    for sink in (True, False):
        out = torch.empty(T, H * D, dtype=dt, device="cuda")
        k.attention(out, q.reshape(T, H * D).to(dt).cuda(), pool, table, pos, slot, H, G, D, 1.0, 0, None, sink=sink)
        want = P.softmax_attention(q.double(), kk.double(), v.double(), 1.0, 0, sink)
        assert_rows_close(out.float().cpu(), want.float(), dtype, f"sink={sink}", 2e-5 if dtype == "float32" else 2e-2)
    with_sink = P.softmax_attention(q.double(), kk.double(), v.double(), 1.0, 0, True)
    without = P.softmax_attention(q.double(), kk.double(), v.double(), 1.0, 0, False)
    assert float((with_sink[0] / without[0]).mean()) == pytest.approx(0.5, rel=0.05)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", [(16, 1, 1), (48, 3, 2), (64, 8, 4), (40, 5, 8)])
def test_recurrent_block_remembers_from_far_back(tmp_path, dtype, sizes):
    """The recurrent side alone with decays close to 1 (lam far below zero): 500 tokens whole, in portions shorter
    than the convolution, then token by token; two sequences side by side; a slot used again starts from zero."""
    from zlm_b200 import StepEntry
    width, blocks, taps = sizes
    cfg = one_layer("parallel", pair(att(1, 1, 8, 8, 0.3), rec(width, blocks, taps), 0.0, 1.0), dense(32, 2.0))
    t = make_tensors(cfg, 21)
    t["l0.mix.right.lam"] = (t["l0.mix.right.lam"] - 3.0).to(torch.bfloat16).float()       # a = exp(-8 r softplus(lam)) near 0.99
    ref = {n: x.double() for n, x in t.items()}
    a, b = prompts(cfg["vocab"], [500, 37], seed=9)
    want = P.forward(cfg, ref, a)[0]
    forgetful = dict(ref)
    forgetful["l0.mix.right.lam"] = ref["l0.mix.right.lam"] + 6.0
    assert float(((P.forward(cfg, forgetful, a)[0] - want)[300:].norm(dim=-1) / want[300:].norm(dim=-1)).median()) > 0.05
    eng = engine_for(tmp_path, cfg, t, dtype, f"rec{width}")
    assert_rows_close(run_cut(eng, a, [500]), want, dtype, "whole")
    assert_rows_close(run_cut(eng, a, [1, 2, 1, 3, 250, 2, 200], then_single=41), want, dtype, "portions, then single tokens")
    s1, s2 = eng.new_sequence(), eng.new_sequence()
    got = eng.step([StepEntry(s1, b, [36]), StepEntry(s2, a[:200], [99, 199])]).clone()          # (pieces, unequal sequences)
    assert_rows_close(got, torch.stack([P.forward(cfg, ref, b)[0][36], want[99], want[199]]), dtype, "side by side")
    got = eng.step([StepEntry(s1, a[:5], []), StepEntry(s2, a[200:210], [9])]).clone()
    assert_rows_close(got, want[209:210], dtype, "going on from the pieces' state")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", [(1, 8, 8, 3), (2, 24, 20, 6), (3, 48, 200, 16), (1, 128, 16, 5), (2, 72, 40, 1)])
def test_gated_linear_attention_remembers_from_far_back(tmp_path, dtype, sizes):
    """The gated side alone, with a temperature that keeps the decays near 1: 450 tokens whole, in portions, token by
    token; key sizes that are not powers of two, values wider than a block of the kernel."""
    heads, dim, vdim, rank = sizes
    cfg = one_layer("parallel_2", pair(att(1, 1, 8, 8, 0.3, conv=2, window=5), gla(heads, dim, vdim, 32.0, rank), 0.0, 1.0))
    t = make_tensors(cfg, 31)
    ref = {n: x.double() for n, x in t.items()}
    (a,) = prompts(cfg["vocab"], [450], seed=13)
    want = P.forward(cfg, ref, a)[0]
    short = P.forward(changed(cfg, ("layers", 0, "mixer", "right", "tau"), 0.5), ref, a)[0]
    assert float(((short - want)[300:].norm(dim=-1) / want[300:].norm(dim=-1)).median()) > 0.05
    eng = engine_for(tmp_path, cfg, t, dtype, f"gla{dim}")
    assert_rows_close(run_cut(eng, a, [450]), want, dtype, "whole")
    assert_rows_close(run_cut(eng, a, [17, 2, 300, 1, 90], then_single=40), want, dtype, "portions, then single tokens")
    # two sequences of unequal length side by side, both in pieces, one of them going on from a state
    from zlm_b200 import StepEntry
    (b,) = prompts(cfg["vocab"], [140], seed=14)
    s1, s2 = eng.new_sequence(), eng.new_sequence()
    eng.step([StepEntry(s1, a[:70], [])])
    got = eng.step([StepEntry(s2, b, [139]), StepEntry(s1, a[70:400], [0, 129, 329])]).clone()
    assert_rows_close(got, torch.stack([P.forward(cfg, ref, b)[0][139], want[70], want[199], want[399]]), dtype, "side by side")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", [(1, 16, 8), (2, 40, 12), (4, 64, 64), (3, 72, 200)])
def test_lightning_attention_over_a_long_prompt(tmp_path, dtype, sizes):
    """Fixed decays near 1 over 700 tokens (the kernel runs the prompt in pieces), then a portion on a state that is
    not zero, then token by token."""
    heads, dim, vdim = sizes
    decay = [1.0 - 0.3 ** (h + 1) for h in range(heads)]
    cfg = one_layer("lightning", light(heads, dim, vdim, decay), dense(48, 1.5))
    t = make_tensors(cfg, 41)
    ref = {n: x.double() for n, x in t.items()}
    (a,) = prompts(cfg["vocab"], [760], seed=17)
    want = P.forward(cfg, ref, a)[0]
    eng = engine_for(tmp_path, cfg, t, dtype, f"light{dim}")
    assert_rows_close(run_cut(eng, a, [760]), want, dtype, "whole")
    assert_rows_close(run_cut(eng, a, [300, 2, 400], then_single=58), want, dtype, "pieces, a portion, single tokens")


def test_groups_marked_by_their_two_best():
    """Made scores: the group with the single best expert is not the group with the best two; both router kernels
    follow the sum of two, and with ``group_top`` 1 the other group."""
    from zlm_b200.kernels import get_kernels
    k = get_kernels()
    g = torch.Generator().manual_seed(2)
    T, E, groups, keep, top = 40, 12, 4, 2, 3
    s = 0.05 + 0.9 * torch.rand(T, E, generator=g, dtype=torch.float64)
    s[0] = torch.tensor([0.95, 0.05, 0.05, 0.6, 0.55, 0.05, 0.5, 0.45, 0.05, 0.3, 0.05, 0.05])
    z = torch.log(s / (1 - s)).float()
    corr = (0.1 * torch.randn(E, generator=g)).float()
    corr[:3] = 0.0
    idx_w, wgt_w, margin = P.route(z.double(), corr.double(), top, groups, keep)
    idx = torch.empty(T, top, dtype=torch.int32, device="cuda")
    wgt = torch.empty(T, top, dtype=torch.float32, device="cuda")
    k.moe_choose(idx, wgt, z.cuda().contiguous(), E, top, None, "sigmoid", False, corr.cuda(), groups, keep, 1.0, 2)
    sure = margin > 1e-4
    assert sure.sum() > 30
    assert torch.equal(idx.cpu().long().sort(-1).values[sure], idx_w.sort(-1).values[sure])
    assert torch.allclose(wgt.cpu().double().sort(-1).values[sure], wgt_w.sort(-1).values[sure], atol=1e-6)
    assert sorted(idx[0].tolist()) == [3, 4, 6]            # groups 1 and 2 by their sums; group 0 has the best single expert
    k.moe_choose(idx, wgt, z.cuda().contiguous(), E, top, None, "sigmoid", False, corr.cuda(), groups, keep, 1.0, 1)
    assert 0 in idx[0].tolist()
    # the kernel that computes the logits itself
    x = torch.randn(T, 32, generator=g)
    w = torch.randn(E, 32, generator=g) / 2
    idx_w, wgt_w, margin = P.route(x.double() @ w.double().T, corr.double(), top, groups, keep)
    k.moe_route(idx, wgt, x.cuda(), w.cuda(), top, None, None, "sigmoid", False, corr.cuda(), groups, keep, 1.0, 2)
    sure = margin > 1e-4
    assert torch.equal(idx.cpu().long().sort(-1).values[sure], idx_w.sort(-1).values[sure])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("r", [(8, 3, 4, 2), (6, 1, None, None), (12, 4, 3, 2), (4, 4, 2, 2)])
def test_routed_layer_against_the_plain_one(tmp_path, dtype, r):
    """A layer whose feed-forward is routed, few tokens and many (the grouped product), positions with a close call
    left out in bfloat16."""
    from sudupel_helpers import oracle
    experts, top, count, keep = r
    cfg = one_layer("lightning", light(2, 16, 16, [0.9, 0.5]), moe(24, experts, top, count, keep))
    t = make_tensors(cfg, 51)
    ref = {n: x.double() for n, x in t.items()}
    eng = engine_for(tmp_path, cfg, t, dtype, f"moe{experts}")
    for n in (3, 150):
        (a,) = prompts(cfg["vocab"], [n], seed=n)
        oracle(ref, cfg, a, dtype).check(run_cut(eng, a, [n]), range(n), dtype, f"{n} tokens")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("limit", [0.3, 1.5, 50.0])
def test_dense_feed_forward_with_limits_that_bite(tmp_path, dtype, limit):
    cfg = one_layer("lightning", light(1, 16, 16, [0.8]), dense(72, limit), embedding={"scale": 3.0}, logit_softcap=4.0)
    t = make_tensors(cfg, 61)
    ref = {n: x.double() for n, x in t.items()}
    (a,) = prompts(cfg["vocab"], [90], seed=3)
    want = P.forward(cfg, ref, a)[0]
    other = P.forward(changed(cfg, ("layers", 0, "mlp", "limit"), limit * 2), ref, a)[0]
    if limit < 10:
        assert float(((other - want).norm(dim=-1) / want.norm(dim=-1)).median()) > 0.02
    assert float(want.abs().max()) > 2.0            # the cap bites
    eng = engine_for(tmp_path, cfg, t, dtype, f"dense{limit}")
    assert_rows_close(run_cut(eng, a, [90]), want, dtype, "whole")
    assert_rows_close(run_cut(eng, a, [5], then_single=85), want, dtype, "single tokens")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("mode", ["none", "unit", "head", "row"])
def test_qkv_preparation_kernel(dtype, mode):
    """Convolution, the four norms, rotation over a part of a head with a factor on cos and sin, the cache's layout
    with padded heads, over two sequences of which one goes on from a state."""
    from types import SimpleNamespace
    from zlm_b200.kernels import get_kernels, PAGE_TOKENS
    k = get_kernels()
    dt = torch.float32 if dtype == "float32" else torch.bfloat16
    g = torch.Generator().manual_seed(7)
    H, G, D, V, taps, n_rot, eps, mscale = 3, 1, 24, 40, 3, 16, 1e-5, 1.2
    hdp = 48
    C = (H + G) * D + G * V
    lens, starts = [5, 70], [66, 0]
    T = sum(lens)
    proj = torch.randn(T, C + 8, generator=g).to(dt).float()
    conv_w = torch.randn(C, taps, generator=g).to(dt).float()
    state = torch.randn(2, taps - 1, C, generator=g).to(dt).float()
    qw = (1 + 0.2 * torch.randn(H * D if mode == "row" else D, generator=g)).to(dt).float()
    kw = (1 + 0.2 * torch.randn(G * D if mode == "row" else D, generator=g)).to(dt).float()
    inv = torch.tensor([30.0 ** (-2 * i / n_rot) for i in range(n_rot // 2)], dtype=torch.float32)
    pos = torch.tensor([starts[0] + i for i in range(lens[0])] + [starts[1] + i for i in range(lens[1])], dtype=torch.int32)
    seq = torch.tensor([0] * lens[0] + [1] * lens[1], dtype=torch.int32)
    slots = torch.tensor([1, 0], dtype=torch.int32)
    plan = SimpleNamespace(token_pos=pos.cuda(), token_slot=slots[seq.long()].cuda(), token_seq=seq.cuda(),
                           seq_start=torch.tensor(starts, dtype=torch.int32).cuda(),
                           cu_seqlens=torch.tensor([0, lens[0], T], dtype=torch.int32).cuda(), seq_slot=slots.cuda(), R=2)
    pool = torch.zeros(6, 2, G, PAGE_TOKENS, hdp, dtype=dt, device="cuda")
    table = torch.tensor([[0, 1, 2], [3, 4, 5]], dtype=torch.int32, device="cuda")
    q_out = torch.empty(T, H * hdp, dtype=dt, device="cuda")
    st = state.to(dt).cuda().contiguous()
    k.attn_prep(q_out, proj.to(dt).cuda(), conv_w.to(dt).cuda(), st, plan, table, pool, H, G, D, V, taps, mode,
                qw.to(dt).cuda() if mode in ("head", "row") else None, kw.to(dt).cuda() if mode in ("head", "row") else None,
                eps, inv.cuda(), n_rot, mscale)
    at = 0
    for r, (n, start) in enumerate(zip(lens, starts)):
        u = proj[at:at + n, :C].double()
        before = state[int(slots[r])].double() if start > 0 else torch.zeros(taps - 1, C, dtype=torch.float64)
        y = P.causal_conv(torch.cat([before, u]), conv_w.double())[taps - 1:]
        qq, kk, vv = y[:, :H * D], y[:, H * D:(H + G) * D], y[:, (H + G) * D:]
        if mode == "row":
            qq, kk = P.rms_norm(qq, qw.double(), eps), P.rms_norm(kk, kw.double(), eps)
        qq, kk = qq.view(n, H, D), kk.view(n, G, D)
        if mode in ("unit", "head"):
            qq = P.rms_norm(qq, qw.double() if mode == "head" else None, eps)
            kk = P.rms_norm(kk, kw.double() if mode == "head" else None, eps)
        p = pos[at:at + n].long()
        a = p.double()[:, None] * inv.double()[None, :]
        cos, sin = (torch.cos(a) * mscale)[:, None, :], (torch.sin(a) * mscale)[:, None, :]
        def turn(x):
            u1, u2 = x[..., :n_rot // 2], x[..., n_rot // 2:n_rot]
            return torch.cat([u1 * cos - u2 * sin, u2 * cos + u1 * sin, x[..., n_rot:]], -1)
        qq, kk = turn(qq), turn(kk)
        tol = 2e-5 if dtype == "float32" else 1e-2
        got_q = q_out[at:at + n].float().cpu().view(n, H, hdp)
        assert_rows_close(got_q[..., :D].reshape(n, -1), qq.reshape(n, -1).float(), dtype, f"q of sequence {r}", tol)
        assert float(got_q[..., D:].abs().max()) == 0.0
        for i in range(n):
            page, off = int(table[int(slots[r]), int(p[i]) // PAGE_TOKENS]), int(p[i]) % PAGE_TOKENS
            assert_rows_close(pool[page, 0, :, off, :D].float().cpu().reshape(1, -1), kk[i].reshape(1, -1).float(), dtype, "k", tol)
            assert_rows_close(pool[page, 1, :, off, :V].float().cpu().reshape(1, -1), vv[i].reshape(1, -1).float(), dtype, "v", tol)
            assert float(pool[page, 1, :, off, V:].abs().max()) == 0.0
        # the state: the newest taps - 1 projected rows
        hist = torch.cat([before, u])[-(taps - 1):]
        assert torch.allclose(st[int(slots[r])].float().cpu().double(), hist.to(dt).double(), atol=0)
        at += n


@pytest.mark.parametrize("dtype", DTYPES)
def test_small_kernels(dtype):
    """The scaled sum of two sides, the cap on logits, silu in place on the first columns, the clamped gated
    activation, the norm-and-gate kernel with every grouping."""
    from zlm_b200.kernels import get_kernels
    k = get_kernels()
    dt = torch.float32 if dtype == "float32" else torch.bfloat16
    g = torch.Generator().manual_seed(1)
    a, b, out = (torch.randn(7, 50, generator=g).cuda() for _ in range(3))
    keep = out.clone()
    k.scaled_sum(out, a, 0.7, b, -1.3, accumulate=True)
    assert torch.allclose(out, keep + 0.7 * a - 1.3 * b, atol=1e-6)
    k.expect_blank(out)
    k.scaled_sum(out, a, 0.7, b, -1.3)
    assert torch.allclose(out, 0.7 * a - 1.3 * b, atol=1e-6)
    x = (20 * torch.randn(5, 33, generator=g)).cuda()
    want = 7.0 * torch.tanh(x / 7.0)
    k.softcap_(x, 7.0)
    assert torch.allclose(x, want, atol=1e-5)
    y = torch.randn(9, 40, generator=g).to(dt).cuda()
    want = y.clone().float()
    want[:, :24] = torch.nn.functional.silu(want[:, :24])
    k.silu_rows(y, 24)
    assert torch.allclose(y.float(), want, atol=1e-6 if dtype == "float32" else 2e-2)
    gu = (2 * torch.randn(11, 2 * 24, generator=g)).to(dt).cuda()
    act = torch.empty(11, 24, dtype=dt, device="cuda")
    k.gated_limit(act, gu, 1.1, 1.702)
    gg, uu = gu.float()[:, :24].clamp(max=1.1), gu.float()[:, 24:].clamp(-1.1, 1.1)
    assert torch.allclose(act.float(), gg * torch.sigmoid(1.702 * gg) * (uu + 1), atol=1e-5 if dtype == "float32" else 3e-2)
    H, V = 3, 20
    o = torch.randn(6, H * V, generator=g).cuda()
    gate = torch.randn(6, H * V + 4, generator=g).to(dt).cuda()
    for group, w in (("head", (1 + 0.1 * torch.randn(V, generator=g))), ("row", (1 + 0.1 * torch.randn(H * V, generator=g))), ("none", None)):
        for act_name in ("sigmoid", "silu", "none"):
            res = torch.empty(6, H * V, dtype=dt, device="cuda")
            k.norm_gate(res, o, gate[:, :H * V] if act_name != "none" else None, H, V, group, None if w is None else w.cuda(), 1e-5,
                        act_name, 0.5)
            ref = o.double().cpu()
            if group == "head":
                ref = P.rms_norm(ref.view(6, H, V), w.double(), 1e-5).reshape(6, -1)
            elif group == "row":
                ref = P.rms_norm(ref, w.double(), 1e-5)
            gz = gate[:, :H * V].double().cpu()
            ref = ref * (torch.sigmoid(gz) if act_name == "sigmoid" else P.silu(gz) if act_name == "silu" else 1.0) * 0.5
            assert torch.allclose(res.double().cpu(), ref, atol=1e-5 if dtype == "float32" else 3e-2), (group, act_name)


@pytest.mark.parametrize("T", [1, 3, 8, 16, 17, 40, 64, 100, 128, 300, 500])
@pytest.mark.parametrize("I, K_", [(64, 40), (200, 1000), (1536, 512)])
def test_clamped_gate_in_the_epilogue_of_the_products(T, I, K_):
    """``linear_swiglu(act="swish_limit")`` on the streaming product, the tcgen05 forms and the mma.sync fallback against
    the plain clamped halves, with two different pairs of constants one after the other (each product gets its own), and
    the silu form of the same call after it still is silu."""
    from zlm_b200.kernels import get_kernels, interleave_gate_up
    k = get_kernels()
    g = torch.Generator().manual_seed(71)
    x = (1.5 * torch.randn(T, K_, generator=g)).to(torch.bfloat16)
    gate = (torch.randn(I, K_, generator=g) * K_ ** -0.5).to(torch.bfloat16)
    up = (torch.randn(I, K_, generator=g) * K_ ** -0.5).to(torch.bfloat16)
    w = interleave_gate_up(gate.cuda(), up.cuda())
    g64, u64 = x.double() @ gate.double().T, x.double() @ up.double().T
    for impl in (None, "mma", "gemv" if T <= 16 else None):
        for limit, alpha in ((0.8, 1.702), (2.5, 1.0)):
            out = torch.zeros(T, I, dtype=torch.bfloat16, device="cuda")
            k.linear_swiglu(out, x.cuda(), w, impl=impl, act="swish_limit", limit=limit, alpha=alpha)
            gg, uu = g64.clamp(max=limit), u64.clamp(-limit, limit)
            want = gg * torch.sigmoid(alpha * gg) * (uu + 1.0)
            assert torch.allclose(out.double().cpu(), want, atol=2e-2, rtol=2e-2), f"impl={impl} limit={limit}"
        k.linear_swiglu(out, x.cuda(), w, impl=impl)
        assert torch.allclose(out.double().cpu(), g64 * torch.sigmoid(g64) * u64, atol=2e-2, rtol=2e-2), f"silu impl={impl}"
    assert k.gemm_tc_status() == 0
