"""Lodevik's mechanisms one by one, each kernel beside a plain function of tests/plain_lodevik.py (float64, no cache):
the attention kernels' options (keys of the query's own chunk only, a cap on the scores, a learned sink per head,
several key heads on one value head) on every kernel that has them (the 32-bit kernel, the split decode kernel, the
mma.sync and the tcgen05 prompt kernels), the latent attention's kernels with sinks and chunks, the two kernels around
the differential attention, the embedding with its table of token pairs and its per-sequence state, the norm of a
sublayer's output with scale and residual add, the gated gelu (alone and in the products' epilogues), the gate per
head.  Where random numbers would hide a fault, one query and two keys are scaled so that the key just inside a
chunk holds all the weight and the key just outside it would hold even more if it were seen."""
import math

import pytest
import torch

import plain_lodevik as P

pytestmark = pytest.mark.gpu

PAGE = 64
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-5, "bfloat16": 2e-2}
F = torch.float64


@pytest.fixture(scope="module")
def K():
    from zlm_b200.kernels import get_kernels
    return get_kernels()


def close(got, want, dtype, what="", tol=None):
    """Rows as vectors: |got - want| <= tol * |want| for every row (rows of the last axis)."""
    got, want = got.double().cpu().reshape(-1, got.shape[-1]), want.double().cpu().reshape(-1, want.shape[-1])
    err = (got - want).norm(dim=1) / want.norm(dim=1).clamp_min(1e-9)
    t = tol or TOL[dtype]
    assert float(err.max()) <= t, f"{what}: row {int(err.argmax())} differs by {err.max():.3e} of its norm"


def rnd(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g) * scale


class Plan:
    """What the attention dispatchers read of a step's context: packed sequences with their slots, first positions
    and numbers of new tokens."""

    def __init__(self, slots, starts, news):
        self.is_decode = all(n == 1 for n in news)
        cu = [0]
        for n in news:
            cu.append(cu[-1] + n)
        self.R, self.max_new = len(slots), max(news)
        self.max_len = max(s + n for s, n in zip(starts, news))
        self.h_seq_start, self.h_seq_new = list(starts), list(news)
        self.cu_seqlens = torch.tensor(cu, dtype=torch.int32).cuda()
        self.seq_slot = torch.tensor(slots, dtype=torch.int32).cuda()
        self.seq_start = torch.tensor(starts, dtype=torch.int32).cuda()
        self.attention_impl = None
        self._bufs = {}

    def scratch(self, name, shape, dtype):
        n = 1
        for s in shape:
            n *= int(s)
        if name not in self._bufs or self._bufs[name].numel() < n:
            self._bufs[name] = torch.empty(n, dtype=dtype, device="cuda")
        return self._bufs[name][:n].view(*shape)


# ---------------------------------------------------------------------------------------------------------------
# the attention kernels' options
# ---------------------------------------------------------------------------------------------------------------
def shared_value_pool(keys, values, slots, n_pages, hd, seed):
    """keys [seq][n, nk, hd], values [seq][n, nv, hd] -> (pool [pages, nk + nv, PAGE, hd], table): the pages dealt in
    a shuffled order among pages of other content, slots that are not 0, 1, 2 ..."""
    g = torch.Generator().manual_seed(seed)
    nk, nv = keys[0].shape[1], values[0].shape[1]
    pool = torch.randn(n_pages, nk + nv, PAGE, hd, generator=g) * 2.0
    order = torch.randperm(n_pages, generator=g).tolist()
    table = torch.zeros(max(slots) + 1, 16, dtype=torch.int32)
    for s, k, v in zip(slots, keys, values):
        for lp in range((k.shape[0] + PAGE - 1) // PAGE):
            page = order.pop()
            table[s, lp] = page
            kk, vv = k[lp * PAGE:(lp + 1) * PAGE], v[lp * PAGE:(lp + 1) * PAGE]
            pool[page, :nk, :kk.shape[0]] = kk.transpose(0, 1)
            pool[page, nk:, :vv.shape[0]] = vv.transpose(0, 1)
    return pool, table


def plain_attention(q, k, v, pos, scale, chunk, softcap, sinks, group, v_share):
    """One query token: q [nq, hd] at position ``pos`` over k [n, nk, hd], v [n, nk / v_share, hd]; query head h reads
    key head h // group, and key head j reads value head j // v_share."""
    n = pos + 1
    kh = torch.arange(q.shape[0]) // group
    ok = P.visible(n, chunk)[pos:pos + 1]                                         # [1, n]: the last row of the mask
    out = P.attend(q[None].to(F), k[:n, kh].to(F), v[:n, kh // v_share].to(F), scale, ok, softcap, sinks)
    return out[0]


CASES = [
    # nq, nkv (key heads), hd, v_share, chunk, softcap, sink
    (8, 4, 16, 2, 70, 0.0, False),
    (6, 6, 48, 2, 64, 20.0, False),
    (4, 2, 128, 2, 128, 20.0, False),
    (16, 4, 128, 2, 100, 0.0, False),
    (4, 4, 128, 1, 0, 25.0, True),
    (3, 1, 64, 1, 48, 0.0, True),
    (12, 2, 32, 1, 130, 15.0, True),
    (5, 5, 80, 1, 0, 0.0, True),
]


def make_attention_case(nq, nkv, hd, v_share, chunk, softcap, sink, lens, news, probe, dtype, seed):
    """Random keys, values and queries of several sequences (``lens`` after the step, of which ``news`` new); for the
    query at position ``probe`` of the first sequence's last head, the first key that it may see is scaled to a score
    of 30 and the key before that one (which the chunk hides) to a score of 60."""
    group = nq // nkv
    nv = nkv // v_share
    keys = [rnd((n, nkv, hd), seed + i).to(dtype).double() for i, n in enumerate(lens)]
    values = [rnd((n, nv, hd), seed + 50 + i).to(dtype).double() for i, n in enumerate(lens)]
    starts = [l - n for l, n in zip(lens, news)]
    pos = [p for s, n in zip(starts, news) for p in range(s, s + n)]
    seq = [i for i, n in enumerate(news) for _ in range(n)]
    q = rnd((len(pos), nq, hd), seed + 99).to(dtype).double()
    scale = 1.0 / math.sqrt(hd)
    row = pos.index(probe)                       # the first sequence's tokens come first
    first = probe - probe % chunk if chunk else 0
    qh = q[row, nq - 1]
    unit = qh / (float(qh @ qh) * scale)
    keys[0][first, nkv - 1] = (unit * 30.0).to(dtype).double()
    if first > 0:
        keys[0][first - 1, nkv - 1] = (unit * 60.0).to(dtype).double()
    sinks = rnd((nq,), seed + 7, 2.0).float() if sink else None
    return keys, values, q, pos, seq, starts, scale, sinks, row, first, group


def run_attention_case(K, case, lens, news, probe, dtype, plan_of, seed=1, v_dim=None):
    """``v_dim``: the values are that wide; the columns beyond them in the pool hold numbers that nobody may read, and
    the output's columns beyond them must come out as zeros."""
    nq, nkv, hd, v_share, chunk, softcap, sink = case
    dt = DT[dtype]
    keys, values, q, pos, seq, starts, scale, sinks, row, first, group = make_attention_case(
        nq, nkv, hd, v_share, chunk, softcap, sink, lens, news, probe, dt, seed)
    slots = [3, 0, 5, 1, 4][:len(lens)]
    pool, table = shared_value_pool(keys, values, slots, 40, hd, seed)
    vd = v_dim or hd
    want = torch.stack([plain_attention(q[t], keys[seq[t]], values[seq[t]][..., :vd], pos[t], scale, chunk, softcap,
                                        sinks.double() if sinks is not None else None, group, v_share)
                        for t in range(len(pos))])
    T = len(pos)
    out = torch.zeros(T, nq * hd, dtype=dt, device="cuda")
    plan = plan_of(slots, starts, news)
    K.attention(out, q.to(dt).view(T, nq * hd).cuda(), pool.to(dt).cuda(), table.cuda(),
                torch.tensor(pos, dtype=torch.int32).cuda(), torch.tensor([slots[s] for s in seq], dtype=torch.int32).cuda(),
                nq, nkv, hd, scale, 0, plan, chunk=chunk, softcap=softcap,
                sinks=sinks.cuda() if sinks is not None else None, v_share=v_share, v_dim=v_dim)
    assert K.gemm_tc_status() == 0
    close(out.view(T, nq, hd)[..., :vd], want, dtype, f"{case}", tol=3e-2 if dtype == "bfloat16" else None)
    assert not bool(out.view(T, nq, hd)[..., vd:].any()), f"{case}: the columns beyond the values are not zeros"
    # the key just inside holds the weight of the probe's last head (beside the sink, if any): its value comes out
    got = out.view(T, nq, hd)[row, nq - 1].double().cpu()
    share = 1.0
    if sinks is not None:
        s_in = softcap * math.tanh(30.0 / softcap) if softcap else 30.0
        share = 1.0 / (1.0 + math.exp(float(sinks[nq - 1]) - s_in))
    v_in = values[0][first, (nkv - 1) // v_share][:vd] * share
    got = got[:vd]
    assert float((got - v_in).abs().max()) <= 0.05 * float(v_in.abs().max()) + 0.05, f"{case}: the probe reads another key"


def no_plan(slots, starts, news):
    return None


LENS, NEWS = [300, 5, 129, 64, 65], [300, 5, 70, 1, 65]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", CASES)
def test_attention_options_on_the_kernel_for_any_shape(K, case, dtype):
    run_attention_case(K, case, LENS, NEWS, 299, dtype, no_plan)


@pytest.mark.parametrize("impl", ["mma", None, "tc1", "tc2"])
@pytest.mark.parametrize("probe", [299, 256, 130])
@pytest.mark.parametrize("case", CASES)
def test_attention_options_on_the_prompt_kernels(K, case, impl, probe):
    """Whole prompts, a portion after a cached prefix, a single token, over tile and page borders; the probe sits at
    the end of the sequence, at the first position of a tile, and in the middle of one.  ``None``: the tcgen05 kernel
    where it takes the shape (heads of 128), "tc1" / "tc2" with one or two heads of a group in a block."""
    if impl in ("tc1", "tc2") and case[2] != 128:
        pytest.skip("the tcgen05 kernel is built for heads of 128")

    def plan_of(slots, starts, news):
        plan = Plan(slots, starts, news)
        plan.attention_impl = "mma" if impl == "mma" else None
        return plan
    K.set_prefill_attention_heads({"tc1": 1, "tc2": 2}.get(impl, 0))
    try:
        run_attention_case(K, case, LENS, NEWS, probe, "bfloat16", plan_of, seed=probe)
    finally:
        K.set_prefill_attention_heads(0)


@pytest.mark.parametrize("impl", ["mma", None])
@pytest.mark.parametrize("probe", [299, 256, 130])
@pytest.mark.parametrize("case", [(5, 5, 192, 1, 0, 0.0, True), (4, 4, 192, 1, 100, 0.0, True), (3, 3, 192, 1, 0, 0.0, False),
                                  (4, 2, 192, 1, 64, 30.0, False)])
def test_keys_wider_than_values_on_the_prompt_kernels(K, case, impl, probe):
    """Keys of 192 over values of 128 (what latent attention's whole prompts run on): the mma.sync kernel and, where
    ``None`` lets the library choose, the tcgen05 kernel with three slabs of key dimensions."""
    def plan_of(slots, starts, news):
        plan = Plan(slots, starts, news)
        plan.attention_impl = impl
        return plan
    run_attention_case(K, case, LENS, NEWS, probe, "bfloat16", plan_of, seed=probe + 1, v_dim=128)


@pytest.mark.parametrize("blocks", [None, 8, 4000])
@pytest.mark.parametrize("length", [700, 641, 640, 577])
@pytest.mark.parametrize("case", [c for c in CASES if c[0] // c[1] <= 16 and c[2] <= 128])
def test_attention_options_on_the_decode_kernel(K, case, length, blocks):
    """One token a sequence, few and many splits of the pages; the first sequence ends in the middle of a chunk, on
    its first position, on the last position of the chunk before, and just behind a page border."""
    lens = [length, 5, 129, 64, 65]
    K.decode_blocks = blocks
    try:
        run_attention_case(K, case, lens, [1] * 5, length - 1, "bfloat16", Plan, seed=length)
    finally:
        K.decode_blocks = None


# ---------------------------------------------------------------------------------------------------------------
# latent attention over records, with a sink per head and chunks
# ---------------------------------------------------------------------------------------------------------------
def record_pool(recs, seed):
    """Records [seq][n, D] -> (pool [pages, PAGE, D] bf16 on the GPU, table with a row per sequence)."""
    g = torch.Generator().manual_seed(seed)
    D = recs[0].shape[1]
    need = [(r.shape[0] + PAGE - 1) // PAGE for r in recs]
    order = torch.randperm(sum(need) + 2, generator=g).tolist()
    pool = torch.randn(sum(need) + 2, PAGE, D, generator=g) * 3.0
    table = torch.zeros(len(recs), max(need) + 1, dtype=torch.int32)
    for s, rec in enumerate(recs):
        for lp in range(need[s]):
            page = order.pop()
            table[s, lp] = page
            part = rec[lp * PAGE:(lp + 1) * PAGE]
            pool[page, :len(part)] = part.float()
    return pool, table


def plain_record_attention(q, rec, r, scale, pos, chunk, sinks):
    """q [H, D] at ``pos`` over the records rec [n, D] (keys: all D columns, values: the first r), every head alike."""
    n, H = pos + 1, q.shape[0]
    k = rec[:n, None, :].expand(n, H, rec.shape[1])
    return P.attend(q[None], k, k[:, :, :r], scale, P.visible(n, chunk)[pos:pos + 1], 0.0, sinks)[0]


@pytest.mark.parametrize("impl", ["plain32", "plain", "tensor"])
@pytest.mark.parametrize("decode", [True, False])
@pytest.mark.parametrize("H, r, dr, chunk, sink", [(3, 32, 16, 70, True), (16, 96, 32, 64, True), (17, 64, 64, 0, True),
                                                    (2, 48, 16, 128, False), (5, 16, 48, 130, True)])
def test_latent_attention_with_sinks_and_chunks(K, H, r, dr, chunk, sink, decode, impl):
    """Decode steps (ends in the middle of a chunk, on a chunk's first and last position, around page borders; few and
    many splits) and packed prompts and portions.  In the first sequence the first record that its last query may see
    is scaled to hold the weight of the last head, the record before it (hidden by the chunk) to hold even more."""
    dtype = "float32" if impl == "plain32" else "bfloat16"
    dt, D = DT[dtype], r + dr
    if decode:
        spans = [(699, 700), (0, 1), (63, 64), (64, 65), (129, 130), (255, 256), (127, 128), (128, 129)]
    else:
        spans = [(0, 300), (0, 5), (100, 131), (64, 65), (3, 9)]
    recs = [rnd((e, D), 11 * H + i).to(dt).double() for i, (_, e) in enumerate(spans)]
    pos = [p for s, e in spans for p in range(s, e)]
    seq = [i for i, (s, e) in enumerate(spans) for _ in range(s, e)]
    T = len(pos)
    q = rnd((T, H, D), 5, 0.4).to(dt).double()
    probe = spans[0][1] - 1
    row = pos.index(probe)
    first = probe - probe % chunk if chunk else 0
    qh = q[row, H - 1]
    unit = qh / (float(qh @ qh) * 0.25)
    # (every head reads the same records: the scaled record is the last head's alone as far as its own query goes)
    recs[0][first] = (unit * 30.0).to(dt).double()
    if first > 0:
        recs[0][first - 1] = (unit * 60.0).to(dt).double()
    sinks = rnd((H,), 3, 2.0).float() if sink else None
    want = torch.stack([plain_record_attention(q[t], recs[seq[t]], r, 0.25, pos[t], chunk,
                                               sinks.double() if sink else None) for t in range(T)])
    pool, table = record_pool(recs, seed=r)
    plan = Plan(list(range(len(spans))), [s for s, _ in spans], [e - s for s, e in spans])
    for blocks in ((None, 8, 2000) if decode and impl == "tensor" else (None,)):
        K.decode_blocks = blocks
        try:
            out = torch.zeros(T, H * r, dtype=dt, device="cuda")
            K.latent_attention(out, q.to(dt).view(T, H * D).cuda(), pool.to(dt).cuda(), table.cuda(),
                               torch.tensor(pos, dtype=torch.int32).cuda(), torch.tensor(seq, dtype=torch.int32).cuda(),
                               H, r, dr, 0.25, 0, plan if impl == "tensor" else None,
                               impl="plain" if impl != "tensor" else None, chunk=chunk,
                               sinks=sinks.cuda() if sink else None)
        finally:
            K.decode_blocks = None
        close(out.view(T, H, r), want, dtype, f"H={H} r={r} dr={dr} chunk={chunk} blocks={blocks}",
              tol=3e-2 if dtype == "bfloat16" else None)
        got = out.view(T, H, r)[row, H - 1].double().cpu()
        share = 1.0 / (1.0 + math.exp(float(sinks[H - 1]) - 30.0)) if sink else 1.0
        v_in = recs[0][first, :r] * share
        assert float((got - v_in).abs().max()) <= 0.05 * float(v_in.abs().max()) + 0.05, "the probe reads another record"


# ---------------------------------------------------------------------------------------------------------------
# the kernels around the differential attention
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H, G, dim, vdim, n_rot", [(4, 2, 24, 40, 8), (3, 3, 40, 8, 40), (2, 1, 16, 16, 0), (6, 1, 32, 64, 16),
                                                     (1, 1, 64, 128, 32)])
def test_maps_are_normed_rotated_and_written(K, dtype, H, G, dim, vdim, n_rot):
    """``diff_prep``: every map of q and k normed over dim with one weight each, neighbouring pairs of the first n_rot
    coordinates turned by the position, q out as query heads (g * 2 + m) * rep + j, k and v into the token's place of
    the pool [2G key heads | G value heads], padded with zeros to a multiple of 16."""
    dt = DT[dtype]
    hdp = (max(dim, vdim) + 15) // 16 * 16
    rep = H // G
    spans = [(60, 70), (0, 3), (127, 130)]
    pos = [p for s, e in spans for p in range(s, e)]
    seq = [i for i, (s, e) in enumerate(spans) for _ in range(s, e)]
    slots = [2, 0, 1]
    T = len(pos)
    N = (2 * H + 2 * G) * dim + G * vdim
    proj = rnd((T, N + 8 - N % 8), 21).to(dt)
    qw, kw = (1.0 + 0.1 * rnd((dim,), 22)).to(dt), (1.0 + 0.1 * rnd((dim,), 23)).to(dt)
    base, eps = 500.0, 1e-5
    inv_freq = torch.pow(torch.tensor(base, dtype=F), -2.0 * torch.arange(n_rot // 2, dtype=F) / max(n_rot, 1)).float()
    table = torch.zeros(3, 4, dtype=torch.int32)
    order = torch.randperm(9, generator=torch.Generator().manual_seed(4)).tolist()
    for s, (_, e) in zip(slots, spans):
        for lp in range((e + PAGE - 1) // PAGE):
            table[s, lp] = order.pop()
    pool = torch.full((9, 3 * G, PAGE, hdp), 7.0, dtype=dt, device="cuda")
    q_out = torch.full((T, 2 * H * hdp), 7.0, dtype=dt, device="cuda")
    K.diff_prep(q_out, proj.cuda(), qw.cuda(), kw.cuda(), eps, inv_freq.cuda() if n_rot else None, n_rot,
                torch.tensor(pos, dtype=torch.int32).cuda(), torch.tensor([slots[s] for s in seq], dtype=torch.int32).cuda(),
                table.cuda(), pool, H, G, dim, vdim)
    p64 = proj.double()
    posv = torch.tensor(pos)
    q = P.rotate_pairs(P.rms_norm(p64[:, :2 * H * dim].view(T, H, 2, dim), qw.double(), eps), posv, base, n_rot)
    k = P.rotate_pairs(P.rms_norm(p64[:, 2 * H * dim:(2 * H + 2 * G) * dim].view(T, G, 2, dim), kw.double(), eps), posv, base, n_rot)
    v = p64[:, (2 * H + 2 * G) * dim:N].view(T, G, vdim)
    got_q = q_out.view(T, 2 * H, hdp).double().cpu()
    for h in range(H):
        for m in range(2):
            at = ((h // rep) * 2 + m) * rep + h % rep
            close(got_q[:, at, :dim], q[:, h, m], dtype, f"q head {h} map {m}")
            assert float(got_q[:, at, dim:].abs().max() if hdp > dim else 0.0) == 0.0
    pool = pool.double().cpu()
    for t in range(T):
        page, place = int(table[slots[seq[t]], pos[t] // PAGE]), pos[t] % PAGE
        for g in range(G):
            for m in range(2):
                close(pool[page, g * 2 + m, place, :dim][None], k[t, g, m][None], dtype, f"k of token {t}")
                assert float(pool[page, g * 2 + m, place, dim:].abs().sum()) == 0.0
            close(pool[page, 2 * G + g, place, :vdim][None], v[t, g][None], dtype, f"v of token {t}")
            assert float(pool[page, 2 * G + g, place, vdim:].abs().sum()) == 0.0
    # nothing but the tokens' own places was written
    written = sum(1 for _ in pos) * 3 * G * hdp
    assert int((pool != 7.0).sum()) <= written


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H, G, vdim, hdp", [(4, 2, 40, 48), (3, 3, 8, 48), (6, 1, 64, 64), (1, 1, 128, 128)])
def test_maps_are_subtracted_and_the_head_normed(K, dtype, H, G, vdim, hdp):
    dt = DT[dtype]
    T, rep, lam, diff, eps = 37, H // G, 0.37, 0.3, 1e-5
    a = rnd((T, 2 * H, hdp), 31).to(dt)
    out = torch.zeros(T, H * vdim, dtype=dt, device="cuda")
    K.diff_combine(out, a.view(T, -1).cuda(), H, G, vdim, hdp, lam, 1.0 - diff, eps)
    a64 = a.double()
    for h in range(H):
        g, j = h // rep, h % rep
        a1, a2 = a64[:, (g * 2) * rep + j, :vdim], a64[:, (g * 2 + 1) * rep + j, :vdim]
        close(out.view(T, H, vdim)[:, h], P.unit_rms(a1 - lam * a2, eps) * (1.0 - diff), dtype, f"head {h}")


# ---------------------------------------------------------------------------------------------------------------
# the embedding with a scale and a table of token pairs
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("buckets, mul_prev, mul_cur", [(37, 11, 5), (1, 3, 2), (65521, 48271, 16807), (7, 0, 1)])
def test_embedding_with_pairs_keeps_the_token_before_a_step(K, dtype, buckets, mul_prev, mul_cur):
    """Three sequences cut into steps differently (whole, token by token, portions), in slots that are not 0, 1, 2;
    then a slot that is used again by a new sequence, whose first token must take the table's last row whatever the
    slot remembers.  Products of ids and multipliers pass 2^31."""
    dt = DT[dtype]
    V, H = 50000, 72
    table, pair = rnd((V, H), 41).to(dt), rnd((buckets + 1, H), 42).to(dt)
    g = torch.Generator().manual_seed(43)
    seqs = [torch.randint(0, V, (n,), generator=g).tolist() for n in (9, 6, 12)]
    seqs[0][3], seqs[0][4] = V - 1, V - 2                              # the largest products
    slots = [4, 1, 2]
    cuts = [[9], [1] * 6, [2, 5, 1, 4]]
    state = torch.full((6,), 12345, dtype=torch.int32, device="cuda")      # what a slot's earlier user left
    want = [P.embed(s, table.double(), 1.5, pair.double(), buckets, mul_prev, mul_cur) for s in seqs]
    done = [0, 0, 0]
    got = [[], [], []]
    for step in range(6):
        live = [i for i in range(3) if step < len(cuts[i])]
        news = [cuts[i][step] for i in live]
        plan = Plan([slots[i] for i in live], [done[i] for i in live], news)
        ids = [t for i, n in zip(live, news) for t in seqs[i][done[i]:done[i] + n]]
        plan.token_pos = torch.tensor([p for i, n in zip(live, news) for p in range(done[i], done[i] + n)], dtype=torch.int32).cuda()
        plan.token_seq = torch.tensor([j for j, n in enumerate(news) for _ in range(n)], dtype=torch.int32).cuda()
        out = torch.zeros(len(ids), H, dtype=torch.float32, device="cuda")
        K.embed_scaled(out, table.cuda(), torch.tensor(ids, dtype=torch.int32).cuda(), 1.5, pair.cuda(), buckets, mul_prev,
                       mul_cur, plan=plan, prev_state=state)
        at = 0
        for i, n in zip(live, news):
            got[i].append(out[at:at + n].cpu())
            at += n
            done[i] += n
    for i in range(3):
        close(torch.cat(got[i]), want[i], "float32", f"sequence {i}", tol=1e-6)
    assert state[4].item() == seqs[0][-1] and state[1].item() == seqs[1][-1] and state[2].item() == seqs[2][-1]
    # slot 4 again, by a new sequence
    plan = Plan([4], [0], [3])
    plan.token_pos = torch.arange(3, dtype=torch.int32).cuda()
    plan.token_seq = torch.zeros(3, dtype=torch.int32).cuda()
    out = torch.zeros(3, H, dtype=torch.float32, device="cuda")
    K.embed_scaled(out, table.cuda(), torch.tensor(seqs[1][:3], dtype=torch.int32).cuda(), 1.5, pair.cuda(), buckets,
                   mul_prev, mul_cur, plan=plan, prev_state=state)
    close(out, want[1][:3], "float32", "a slot used again", tol=1e-6)
    # without a pair table: the scale alone
    out = torch.zeros(4, H, dtype=torch.float32, device="cuda")
    K.embed_scaled(out, table.cuda(), torch.tensor(seqs[2][:4], dtype=torch.int32).cuda(), 0.25)
    close(out, table.double()[seqs[2][:4]] * 0.25, "float32", "scale alone", tol=1e-6)


# ---------------------------------------------------------------------------------------------------------------
# the norm of a sublayer's output, the layer's scale, the residual add
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("y_dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("R, H", [(1, 64), (37, 1000), (5, 4096), (3, 70), (2, 8192 + 4)])
@pytest.mark.parametrize("scaled, rounded", [(True, True), (True, False), (False, True)])
def test_sublayer_output_norm_scale_and_add(K, y_dtype, R, H, scaled, rounded):
    y = rnd((R, H), 51, 3.0).to(DT[y_dtype])
    x = rnd((R, H), 52)
    w, ls = 1.0 + 0.1 * rnd((H,), 53), 0.5 + 0.2 * rnd((H,), 54)
    stream = x.clone().cuda()
    copy = torch.zeros(R, H, dtype=torch.bfloat16, device="cuda") if rounded else None
    K.norm_scale_add(stream, y.cuda(), w.cuda(), 1e-5, ls.cuda() if scaled else None, cast_out=copy)
    want = x.double() + P.rms_norm(y.double(), w.double(), 1e-5) * (ls.double() if scaled else 1.0)
    close(stream, want, "float32", tol=2e-6)
    if rounded:
        assert torch.equal(copy, stream.to(torch.bfloat16))
    if y_dtype == "float32" and R > 1:
        # a row's result does not depend on the rows beside it
        alone = x[1:2].clone().cuda()
        K.norm_scale_add(alone, y[1:2].cuda(), w.cuda(), 1e-5, ls.cuda() if scaled else None)
        assert torch.equal(alone[0], stream[1])


def test_stream_rounded_to_bfloat16(K):
    x = rnd((7, 1003), 55, 5.0)
    out = torch.zeros(7, 1003, dtype=torch.bfloat16, device="cuda")
    K.cast_rows(out, x.cuda())
    assert torch.equal(out.cpu(), x.to(torch.bfloat16))


# ---------------------------------------------------------------------------------------------------------------
# the gated gelu, alone and in the products' epilogues; the gate per head
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gated_gelu(K, dtype):
    dt = DT[dtype]
    gu = rnd((13, 2 * 88), 61, 2.5).to(dt)
    out = torch.zeros(13, 88, dtype=dt, device="cuda")
    K.gated_act(out, gu.cuda(), "gelu_tanh")
    g64 = gu.double()
    close(out, P.gelu_tanh(g64[:, :88]) * g64[:, 88:], dtype, tol=1e-6 if dtype == "float32" else 6e-3)


@pytest.mark.parametrize("T", [1, 3, 8, 16, 17, 40, 64, 100, 128, 300, 500])
@pytest.mark.parametrize("I, K_", [(64, 40), (200, 1000), (1536, 512)])
def test_gated_gelu_in_the_epilogue_of_the_products(K, T, I, K_):
    """``linear_swiglu(act="gelu_tanh")`` on the streaming product, the tcgen05 forms and the mma.sync fallback, against
    the plain gated feed-forward's first half; the silu form of the same call still is silu."""
    from zlm_b200.kernels import interleave_gate_up
    x = rnd((T, K_), 71).to(torch.bfloat16)
    gate, up = rnd((I, K_), 72, K_ ** -0.5).to(torch.bfloat16), rnd((I, K_), 73, K_ ** -0.5).to(torch.bfloat16)
    w = interleave_gate_up(gate.cuda(), up.cuda())
    g64, u64 = x.double() @ gate.double().T, x.double() @ up.double().T
    for impl in (None, "mma", "gemv" if T <= 16 else None):
        out = torch.zeros(T, I, dtype=torch.bfloat16, device="cuda")
        K.linear_swiglu(out, x.cuda(), w, impl=impl, act="gelu_tanh")
        close(out, P.gelu_tanh(g64) * u64, "bfloat16", f"gelu impl={impl}", tol=1e-2)
        K.linear_swiglu(out, x.cuda(), w, impl=impl)
        close(out, g64 * torch.sigmoid(g64) * u64, "bfloat16", f"silu impl={impl}", tol=1e-2)
    assert K.gemm_tc_status() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H, V", [(3, 24), (1, 8), (16, 128), (5, 50)])
def test_one_gate_number_per_head(K, dtype, H, V):
    dt = DT[dtype]
    T = 11
    buf = rnd((T, H * V + H + 5), 81).to(dt).cuda()         # heads and gate numbers as columns of one projection
    x = buf[:, :H * V].as_strided((T, H, V), (buf.stride(0), V, 1))
    g = buf[:, H * V + 3:H * V + 3 + H]
    want = x.double().cpu() * torch.sigmoid(g.double().cpu())[:, :, None]
    K.head_scalar_gate(x, g)
    close(x.reshape(T, H * V), want.reshape(T, H * V), dtype, tol=1e-6 if dtype == "float32" else 6e-3)


# ---------------------------------------------------------------------------------------------------------------
# per-head keys and values of a step written out for the flash kernels
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H, dn, dr, dv, r", [(3, 32, 32, 48, 64), (2, 128, 64, 128, 96), (5, 12, 4, 10, 20), (1, 8, 8, 16, 8),
                                              (4, 48, 16, 20, 40)])
def test_keys_and_values_of_a_step_are_written_out(K, dtype, H, dn, dr, dv, r):
    """Two sequences of 70 and 5 tokens: K = [the head's unrotated key | the record's rotated part], V = [the head's
    value | zeros], at the token's place of its sequence's own pages; sizes that are multiples of 8 (pieces of 16
    bytes in bfloat16) and sizes that are not; a buffer that held other numbers before."""
    dt = DT[dtype]
    hd, lens = dn + dr, [70, 5]
    T = sum(lens)
    kv = rnd((T, H * (dn + dv)), 3).to(dt)
    rec = rnd((T, r + dr), 4).to(dt)
    pos = torch.tensor([p for n in lens for p in range(n)], dtype=torch.int32)
    seq = torch.tensor([i for i, n in enumerate(lens) for _ in range(n)], dtype=torch.int32)
    table = torch.tensor([[2, 0], [1, 0]], dtype=torch.int32)
    spool = torch.full((3, 2, H, PAGE, hd), 7.0, dtype=dt, device="cuda")
    K.latent_unfold(spool, table.cuda(), kv.cuda(), rec.cuda(), pos.cuda(), seq.cuda(), H, dn, dr, dv, r)
    got = spool.cpu()
    for t in range(T):
        page, place = int(table[seq[t], pos[t] // PAGE]), int(pos[t]) % PAGE
        for h in range(H):
            want_k = torch.cat([kv[t, h * dn:(h + 1) * dn], rec[t, r:]])
            want_v = torch.cat([kv[t, H * dn + h * dv: H * dn + (h + 1) * dv], torch.zeros(hd - dv, dtype=dt)])
            assert torch.equal(got[page, 0, h, place], want_k) and torch.equal(got[page, 1, h, place], want_v), (t, h)
    # places that no token has keep what they held
    assert bool((got[0, :, :, 6:] == 7.0).all()) and bool((got[1, :, :, 5:] == 7.0).all())
