"""The mechanisms of latent attention and of the routed feed-forward one by one: each kernel against the
oracle's function for it, at sizes of their own, with inputs made so that a fault shows: one key among
hundreds that holds almost all of the weight (far back, at a page's border, just inside and just outside a
window, in a prompt's portion and decoded alone), scores with a clear order for the router."""
import math

import pytest
import torch

import plain_nuvilorn as P

pytestmark = pytest.mark.gpu

PAGE = 64
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-5, "bfloat16": 2e-2}


def K():
    from zlm_b200.kernels import get_kernels
    return get_kernels()


def close(got, want, dtype, what=""):
    got, want = got.double().cpu(), want.double().cpu()
    err = (got - want).norm() / want.norm().clamp_min(1e-12)
    assert err <= TOL[dtype], f"{what}: differs by {err:.3e} of its norm"


def paged(records: torch.Tensor, dtype, shuffle_seed=0):
    """records [n, D] of one sequence -> (pool, block_table) with the pages in a shuffled order among
    pages of another content."""
    n, D = records.shape
    pages = (n + PAGE - 1) // PAGE
    g = torch.Generator().manual_seed(shuffle_seed)
    order = torch.randperm(pages + 3, generator=g)[:pages]
    pool = torch.randn(pages + 3, PAGE, D, generator=g) * 3.0
    for lp in range(pages):
        chunk = records[lp * PAGE:(lp + 1) * PAGE]
        pool[order[lp], :len(chunk)] = chunk
    table = torch.zeros(2, pages + 1, dtype=torch.int32)
    table[1, :pages] = order.int()
    return pool.to(DT[dtype]).cuda(), table.cuda()


def plain_attention(q, rec, r, scale, pos, window=0):
    """q [H, D] at position pos over rec [n, D]: softmax over the window's keys, values rec[:, :r]."""
    lo = max(0, pos + 1 - window) if window else 0
    s = (rec[lo:pos + 1] @ q.t()) * scale                    # [keys, H]
    return torch.softmax(s, dim=0).t() @ rec[lo:pos + 1, :r]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H, r, dr", [(3, 40, 8), (1, 24, 16), (18, 72, 16), (5, 136, 0), (16, 512, 64)])
def test_attention_over_records(dtype, H, r, dr):
    k = K()
    D, n = r + dr, 300
    g = torch.Generator().manual_seed(H * 1000 + r)
    rec = torch.randn(n, D, generator=g).to(DT[dtype]).double()
    pool, table = paged(rec.float(), dtype)
    positions = [0, 1, 62, 63, 64, 65, 127, 128, 200, 299]
    q = (torch.randn(len(positions), H, D, generator=g) * 0.5).to(DT[dtype])
    out = torch.zeros(len(positions), H * r, dtype=DT[dtype], device="cuda")
    pos = torch.tensor(positions, dtype=torch.int32, device="cuda")
    slot = torch.ones(len(positions), dtype=torch.int32, device="cuda")
    k.latent_attention(out, q.cuda().view(len(positions), H * D), pool, table, pos, slot, H, r, dr, 0.3)
    want = torch.stack([plain_attention(q[i].double(), rec, r, 0.3, p) for i, p in enumerate(positions)])
    close(out.view(len(positions), H, r), want, dtype, f"attention H={H} r={r} dr={dr}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [0, 5, 64, 100])
def test_one_key_holds_the_weight(dtype, window):
    """For every place of the standing-out key (far back, page borders, the window's first key and the key
    just before it) the output must be that key's value, or must not contain it."""
    k = K()
    H, r, dr, n = 2, 32, 8, 260
    D = r + dr
    g = torch.Generator().manual_seed(7)
    rec = torch.randn(n, D, generator=g).to(DT[dtype]).double()
    pool, table = paged(rec.float(), dtype, 3)
    for pos in (259, 130):
        places = {0, 1, 63, 64, 65, 127, 128, pos - 1, pos}
        if window:
            places |= {pos - window, pos - window + 1, pos - window + 2}
        for j in sorted(p for p in places if 0 <= p <= pos):
            q = (rec[j] * (40.0 / rec[j].norm() ** 2)).to(DT[dtype])         # score 40 at key j, small elsewhere
            q2 = torch.stack([q, -q])                                       # a second head that avoids key j
            out = torch.zeros(1, H * r, dtype=DT[dtype], device="cuda")
            k.latent_attention(out, q2.cuda().view(1, H * D), pool, table,
                               torch.tensor([pos], dtype=torch.int32, device="cuda"),
                               torch.ones(1, dtype=torch.int32, device="cuda"), H, r, dr, 1.0, window)
            want = plain_attention(q2.double(), rec, r, 1.0, pos, window)
            close(out.view(H, r), want, dtype, f"key {j} seen from {pos}, window {window}")
            inside = not window or j > pos - window
            hit = (out.view(H, r)[0].double().cpu() - rec[j, :r]).norm() / rec[j, :r].norm()
            assert (hit < 0.05) == inside, f"key {j} from {pos} window {window}: inside={inside}, distance {hit:.3f}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H, dn, dr, r, n_rot", [(3, 16, 8, 40, 8), (2, 8, 16, 24, 12), (1, 0, 32, 16, 32), (4, 24, 6, 56, 0)])
def test_prep_norms_rotates_and_writes_records(dtype, H, dn, dr, r, n_rot):
    k = K()
    T, eps, base = 7, 1e-5, 300.0
    g = torch.Generator().manual_seed(11)
    Dq, R = dn + dr, r + dr
    qd = torch.randn(T, H * Dq + R, generator=g).to(DT[dtype])
    cw = (1 + 0.2 * torch.randn(r, generator=g)).to(DT[dtype])
    positions = torch.tensor([0, 1, 63, 64, 65, 700, 1500], dtype=torch.int32)
    table = torch.zeros(1, 32, dtype=torch.int32)
    table[0] = torch.randperm(32, generator=g).int()
    pool = torch.zeros(32, PAGE, R, dtype=DT[dtype], device="cuda")
    i = torch.arange(n_rot // 2, dtype=torch.float64)
    inv = (base ** (-2.0 * i / max(n_rot, 1))).float().cuda() if n_rot else None
    dev = qd.cuda()
    qrot = torch.zeros(T, H, dr, dtype=DT[dtype], device="cuda")
    rows = torch.zeros(T, R, dtype=DT[dtype], device="cuda")
    k.latent_prep(dev[:, :H * Dq], qrot, dev[:, H * Dq:], cw.cuda(), eps, inv, n_rot, positions.cuda(),
                  torch.zeros(T, dtype=torch.int32, device="cuda"), table.cuda(), pool, H, dn, dr, r, rec_out=rows)
    x = qd.double()
    c = P.vector_norm(x[:, H * Dq:H * Dq + r], cw.double(), eps)
    kr = P.rotate_pairs(x[:, H * Dq + r:], positions, base, n_rot)
    qr = P.rotate_pairs(x[:, :H * Dq].reshape(T, H, Dq)[..., dn:], positions, base, n_rot)
    close(qrot, qr, dtype, "rotated query parts")
    got = torch.stack([pool[table[0, p // PAGE], p % PAGE] for p in positions.tolist()])
    close(got, torch.cat([c, kr], dim=1), dtype, "records")
    assert torch.equal(rows, got), "the records' plain rows differ from the pages"
    # in place, and without a record (a layer that reads another layer's latents)
    q3 = dev[:, :H * Dq].view(T, H, Dq)
    before = dev.clone()
    k.latent_prep(dev[:, :H * Dq], q3[:, :, dn:], None, None, eps, inv, n_rot, positions.cuda(),
                  torch.zeros(T, dtype=torch.int32, device="cuda"), None, None, H, dn, dr, r)
    close(q3[:, :, dn:], qr, dtype, "rotated in place")
    assert torch.equal(q3[:, :, :dn], before[:, :H * Dq].view(T, H, Dq)[:, :, :dn]) and torch.equal(dev[:, H * Dq:], before[:, H * Dq:])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_per_head_products(dtype):
    k = K()
    g = torch.Generator().manual_seed(13)
    for T, H, N, Kd in [(1, 3, 40, 16), (9, 2, 24, 8), (70, 18, 8, 72), (5, 1, 7, 33), (300, 3, 136, 64), (129, 2, 16, 264)]:
        x = torch.randn(T, H, Kd + (8 if T > 100 else 5), generator=g).to(DT[dtype]).cuda()
        w = (torch.randn(H, N, Kd, generator=g) / Kd ** 0.5).to(DT[dtype]).cuda()
        out = torch.zeros(T, H, N + 3, dtype=DT[dtype], device="cuda")
        k.head_linear(out[:, :, 3:], x[:, :, :Kd], w)
        want = torch.einsum("thk,hnk->thn", x[:, :, :Kd].double(), w.double())
        close(out[:, :, 3:], want, dtype, f"per-head product {T}x{H}x{N}x{Kd}")
        assert float(out[:, :, :3].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E, top, F, SF", [(5, 2, 32, 48), (7, 3, 24, 0), (4, 4, 16, 8), (9, 1, 40, 64), (64, 6, 16, 0)])
def test_routed_feed_forward_kernels(dtype, E, top, F, SF):
    k = K()
    T, W = 37, 64
    g = torch.Generator().manual_seed(E * 10 + top)
    x = torch.randn(T, W, generator=g).to(DT[dtype])
    t = {"router": (torch.randn(E, W, generator=g) * 0.4).to(DT[dtype])}
    for e in range(E):
        t[f"e{e}.up"] = (torch.randn(F, W, generator=g) / W ** 0.5).to(DT[dtype])
        t[f"e{e}.down"] = (torch.randn(W, F, generator=g) / F ** 0.5).to(DT[dtype])
    mlp = {"router": {"experts": E, "top": top}}
    if SF:
        mlp["shared"] = {"ff": SF}
        t["shared.up"] = (torch.randn(SF, W, generator=g) / W ** 0.5).to(DT[dtype])
        t["shared.down"] = (torch.randn(W, SF, generator=g) / SF ** 0.5).to(DT[dtype])
        t["shared.sg"] = (torch.randn(1, W, generator=g) * 0.3).to(DT[dtype])
    t64 = {n: v.double() for n, v in t.items()}
    idx = torch.zeros(T, top, dtype=torch.int32, device="cuda")
    wgt = torch.zeros(T, top, dtype=torch.float32, device="cuda")
    gate = torch.zeros(T, dtype=torch.float32, device="cuda")
    xd = x.cuda()
    k.moe_route(idx, wgt, xd, t["router"].cuda(), top, gate if SF else None, t["shared.sg"].cuda() if SF else None)
    widx, ww = P.route(x.double(), t64["router"], top)
    assert torch.equal(idx.cpu().long(), widx), "chosen experts (in the order of their scores)"
    assert torch.allclose(wgt.cpu().double(), ww, atol=1e-6)
    if SF:
        assert torch.allclose(gate.cpu().double(), torch.sigmoid(x.double() @ t64["shared.sg"].t())[:, 0], atol=1e-6)
    # the same choice from logits that a product left in fp32
    rows = [t["router"]] + ([t["shared.sg"]] if SF else [])
    logits = (x.double() @ torch.cat(rows).double().t()).float().cuda()
    idx2, wgt2, gate2 = torch.zeros_like(idx), torch.zeros_like(wgt), torch.zeros_like(gate)
    k.moe_choose(idx2, wgt2, logits, E, top, gate2 if SF else None)
    assert torch.equal(idx2, idx) and torch.allclose(wgt2, wgt, atol=1e-6)
    if SF:
        assert torch.allclose(gate2, gate, atol=1e-6)
    act = torch.zeros(T, top, F, dtype=DT[dtype], device="cuda")
    w_up = torch.stack([t[f"e{e}.up"] for e in range(E)]).cuda()
    w_down = torch.stack([t[f"e{e}.down"] for e in range(E)]).cuda()
    k.moe_up(act, xd, w_up, idx, wgt)
    stream = torch.randn(T, W, generator=g).cuda()
    start = stream.clone()
    k.moe_down(stream, act, w_down, idx)
    want = torch.zeros(T, W, dtype=torch.float64)
    for i in range(T):
        for e, we in zip(widx[i].tolist(), ww[i]):
            want[i] += P.relu2_expert(we * x[i].double(), t64[f"e{e}.up"], t64[f"e{e}.down"])
    close(stream - start, want, dtype, "routed experts")
    if SF:
        u = torch.zeros(T, SF, dtype=DT[dtype], device="cuda")
        k.linear(u, xd, t["shared.up"].cuda())
        a = torch.zeros_like(u)
        k.relu2_scale(a, u, gate)
        k.linear(stream, a, t["shared.down"].cuda(), accumulate=True)
        close(stream - start, P.moe_ff(x.double(), t64, "", mlp), dtype, "routed and shared experts")


def test_router_prefers_the_lower_index_on_a_tie():
    k = K()
    x = torch.ones(1, 8, device="cuda")
    w = torch.zeros(6, 8, device="cuda")
    w[4] = 0.5
    w[2] = 0.5
    idx = torch.zeros(1, 3, dtype=torch.int32, device="cuda")
    wgt = torch.zeros(1, 3, dtype=torch.float32, device="cuda")
    k.moe_route(idx, wgt, x, w, 3)
    assert idx.tolist() == [[2, 4, 0]]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_single_gain_norms(tmp_path, dtype):
    """The embedding's norm and a layer's norm with one number as weight, through the parts."""
    from zlm_b200.parts.base import Runtime
    from zlm_b200.parts.embedding import TokenEmbedding
    from zlm_b200.parts.norm import RMSNorm
    rt = Runtime(torch.device("cuda"), DT[dtype], K())
    g = torch.Generator().manual_seed(3)
    V, H, eps = 50, 72, 1e-5
    table = torch.randn(V, H, generator=g).to(DT[dtype])
    gain = torch.tensor(1.3).to(DT[dtype])
    emb = TokenEmbedding(V, H, norm={"kind": "rms_norm", "eps": eps, "scalar": True})
    emb.attach(rt)
    assert {n: tuple(p.shape) for n, p in emb.param_specs().items()} == {"weight": (V, H), "norm.weight": ()}
    emb.bind({"weight": table.cuda(), "norm.weight": gain.cuda()})
    ids = torch.tensor([3, 49, 0, 3], dtype=torch.int32, device="cuda")
    out = torch.zeros(4, H, device="cuda")
    emb.forward(out, ids)
    close(out, P.scalar_norm(table.double()[ids.cpu().long()], gain.double(), eps), "float32", "embedding norm")
    assert emb.tensors()["norm.weight"].shape == ()
    n = RMSNorm(H, eps, scalar=True)
    n.attach(rt)
    n.bind({"weight": gain.cuda()})
    y = torch.zeros(4, H, dtype=DT[dtype], device="cuda")
    n.forward(y, out)
    close(y, P.scalar_norm(out.double().cpu(), gain.double(), eps), dtype, "layer norm with one gain")


class Plan:
    """What the attention dispatcher reads of a step's context."""

    def __init__(self, is_decode, max_len, max_new=1):
        self.is_decode, self.max_len, self.max_new = is_decode, max_len, max_new
        self._bufs = {}

    def scratch(self, name, shape, dtype):
        n = 1
        for s in shape:
            n *= int(s)
        if name not in self._bufs or self._bufs[name].numel() < n:
            self._bufs[name] = torch.empty(n, dtype=dtype, device="cuda")
        return self._bufs[name][:n].view(*shape)


def pooled(lengths, D, seed):
    """Records of several sequences in one pool, pages dealt in a shuffled order: (records per sequence
    as float64, pool bf16 on the GPU, block table with a row per slot)."""
    g = torch.Generator().manual_seed(seed)
    recs = [torch.randn(n, D, generator=g).to(torch.bfloat16).double() for n in lengths]
    need = [(n + PAGE - 1) // PAGE for n in lengths]
    order = torch.randperm(sum(need) + 2, generator=g).tolist()
    pool = torch.randn(sum(need) + 2, PAGE, D, generator=g) * 3.0
    table = torch.zeros(len(lengths), max(need) + 1, dtype=torch.int32)
    for s, rec in enumerate(recs):
        for lp in range(need[s]):
            page = order.pop()
            table[s, lp] = page
            chunk = rec[lp * PAGE:(lp + 1) * PAGE]
            pool[page, :len(chunk)] = chunk.float()
    return recs, pool.to(torch.bfloat16).cuda(), table.cuda()


@pytest.mark.parametrize("H, r, dr", [(3, 32, 16), (16, 96, 32), (18, 80, 0), (16, 512, 64), (6, 16, 48)])
@pytest.mark.parametrize("window", [0, 70])
def test_tensor_core_attention_decode_steps(H, r, dr, window):
    """One token per sequence, sequences of unequal lengths (ends at and around page borders), few and many
    splits of the pages."""
    k = K()
    D = r + dr
    lengths = [1, 64, 65, 130, 700, 256]
    recs, pool, table = pooled(lengths, D, seed=H + r)
    g = torch.Generator().manual_seed(5)
    T = len(lengths)
    q = (torch.randn(T, H, D, generator=g) * 0.4).to(torch.bfloat16)
    pos = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device="cuda")
    slot = torch.arange(T, dtype=torch.int32, device="cuda")
    want = torch.stack([plain_attention(q[i].double(), recs[i], r, 0.25, lengths[i] - 1, window) for i in range(T)])
    for blocks in (None, 8, 2000):
        k.decode_blocks = blocks
        try:
            out = torch.zeros(T, H * r, dtype=torch.bfloat16, device="cuda")
            k.latent_attention(out, q.cuda().view(T, H * D), pool, table, pos, slot, H, r, dr, 0.25, window,
                               Plan(True, max(lengths)))
        finally:
            k.decode_blocks = None
        close(out.view(T, H, r), want, "bfloat16", f"decode H={H} r={r} dr={dr} window={window} blocks={blocks}")


@pytest.mark.parametrize("H, r, dr", [(3, 32, 16), (16, 96, 32), (17, 512, 64), (2, 256, 16)])
@pytest.mark.parametrize("window", [0, 33])
def test_tensor_core_attention_prompts_and_portions(H, r, dr, window):
    """Packed tokens of several sequences (whole prompts, a portion that starts late, a single token), so
    that blocks of neighbouring tokens hold the end of one sequence and the start of the next."""
    k = K()
    D = r + dr
    spans = [(0, 5), (0, 70), (100, 131), (64, 65), (3, 9)]          # positions [start, end) of each sequence's tokens
    recs, pool, table = pooled([e for _, e in spans], D, seed=3 * H + dr)
    pos = torch.tensor([p for s, e in spans for p in range(s, e)], dtype=torch.int32)
    slot = torch.tensor([i for i, (s, e) in enumerate(spans) for _ in range(s, e)], dtype=torch.int32)
    T = len(pos)
    g = torch.Generator().manual_seed(9)
    q = (torch.randn(T, H, D, generator=g) * 0.4).to(torch.bfloat16)
    out = torch.zeros(T, H * r, dtype=torch.bfloat16, device="cuda")
    k.latent_attention(out, q.cuda().view(T, H * D), pool, table, pos.cuda(), slot.cuda(), H, r, dr, 0.25, window,
                       Plan(False, max(e for _, e in spans), max(e - s for s, e in spans)))
    want = torch.stack([plain_attention(q[i].double(), recs[int(slot[i])], r, 0.25, int(pos[i]), window) for i in range(T)])
    close(out.view(T, H, r), want, "bfloat16", f"prompts H={H} r={r} dr={dr} window={window}")
    rows = (out.view(T, H, r).double().cpu() - want).flatten(1).norm(dim=1) / want.flatten(1).norm(dim=1)
    assert float(rows.max()) < 3e-2, f"token {int(rows.argmax())} (position {int(pos[rows.argmax()])}) differs by {rows.max():.3e}"


@pytest.mark.parametrize("decode", [True, False])
@pytest.mark.parametrize("window", [0, 5, 64, 100])
def test_one_key_holds_the_weight_on_tensor_cores(decode, window):
    k = K()
    H, r, dr, n = 2, 32, 16, 260
    D = r + dr
    recs, pool, table = pooled([n], D, seed=21)
    rec = recs[0]
    for pos in (259, 130):
        places = {0, 1, 63, 64, 65, 127, 128, pos - 1, pos}
        if window:
            places |= {pos - window, pos - window + 1, pos - window + 2}
        for j in sorted(p for p in places if 0 <= p <= pos):
            q = (rec[j] * (40.0 / rec[j].norm() ** 2)).to(torch.bfloat16)
            q2 = torch.stack([q, -q])
            # (a portion of three tokens whose last one is the query, or the query decoded alone)
            T = 1 if decode else 3
            qs = torch.zeros(T, H, D, dtype=torch.bfloat16)
            qs[-1] = q2
            out = torch.zeros(T, H * r, dtype=torch.bfloat16, device="cuda")
            k.latent_attention(out, qs.cuda().view(T, H * D), pool, table,
                               torch.arange(pos - T + 1, pos + 1, dtype=torch.int32, device="cuda"),
                               torch.zeros(T, dtype=torch.int32, device="cuda"), H, r, dr, 1.0, window,
                               Plan(decode, pos + 1, T))
            got = out[-1].view(H, r)
            close(got, plain_attention(q2.double(), rec, r, 1.0, pos, window), "bfloat16", f"key {j} from {pos}, window {window}")
            inside = not window or j > pos - window
            hit = (got[0].double().cpu() - rec[j, :r]).norm() / rec[j, :r].norm()
            assert (hit < 0.05) == inside, f"key {j} from {pos} window {window}: inside={inside}, distance {hit:.3f}"


@pytest.mark.parametrize("T, E, top, F, W", [(17, 64, 1, 16, 64), (37, 5, 2, 32, 64), (300, 7, 3, 24, 72), (700, 4, 4, 136, 128),
                                            (2048, 16, 2, 64, 256), (64, 64, 6, 16, 64)])
def test_grouped_experts_equal_the_token_by_token_kernels(T, E, top, F, W):
    """Steps of many tokens sort their (token, choice) pairs by expert and run tiles of rows: the same sums
    as the kernels that stream an expert per pair, for few and many rows an expert, experts without any
    row, and tiles that are not full."""
    k = K()
    g = torch.Generator().manual_seed(T + E)
    x = torch.randn(T, W, generator=g).to(torch.bfloat16).cuda()
    w_up = (torch.randn(E, F, W, generator=g) / W ** 0.5).to(torch.bfloat16).cuda()
    w_down = (torch.randn(E, W, F, generator=g) / F ** 0.5).to(torch.bfloat16).cuda()
    router = (torch.randn(E, W, generator=g) * 0.4).to(torch.bfloat16)
    if E >= 16:
        router[-3:] = 0.0
        router[-3:, 0] = -50.0                 # three experts that no token chooses:
        x[:, 0] = x[:, 0].abs() + 0.5          # their logit is -50 times a positive number
    idx = torch.zeros(T, top, dtype=torch.int32, device="cuda")
    wgt = torch.zeros(T, top, dtype=torch.float32, device="cuda")
    k.moe_route(idx, wgt, x, router.cuda(), top)
    if E >= 16:
        assert int(idx.max()) < E - 3
    act = torch.zeros(T, top, F, dtype=torch.bfloat16, device="cuda")
    want = torch.zeros(T, W, device="cuda")
    k.moe_up(act, x, w_up, idx, wgt)
    k.moe_down(want, act, w_down, idx)
    got = torch.zeros(T, W, device="cuda")
    k.moe_grouped(got, x, w_up, w_down, idx, wgt, impl="mma")
    # (the two kernels sum in different orders, and an activation on the edge between two bf16 values may
    # fall either way)
    err = (got - want).double().norm() / want.double().norm()
    assert err < 3e-4, f"grouped experts T={T} E={E} top={top}: differs by {err:.3e} of its norm"
    # the tcgen05 form: the weight is multiplied into the bf16 input rows, so it differs by their rounding
    got_tc = torch.zeros(T, W, device="cuda")
    k.moe_grouped(got_tc, x, w_up, w_down, idx, wgt, impl="tc")
    k.check_status(sync=True)
    err = (got_tc - want).double().norm() / want.double().norm()
    assert err < 1e-2, f"grouped experts on tcgen05 T={T} E={E} top={top}: differs by {err:.3e} of its norm"
    rows = (got_tc - want).double().norm(dim=1) / want.double().norm(dim=1).clamp_min(1e-9)
    assert float(rows.max()) < 5e-2, f"grouped experts on tcgen05: token {int(rows.argmax())} differs by {rows.max():.3e}"
    # and against the plain implementation
    xs = x.double().cpu()
    ref = torch.zeros(T, W, dtype=torch.float64)
    for i in range(0, T, max(1, T // 40)):
        for e, we in zip(idx[i].tolist(), wgt[i].double().cpu()):
            ref[i] += P.relu2_expert(we * xs[i], w_up[e].double().cpu(), w_down[e].double().cpu())
        close(got[i], ref[i], "bfloat16", f"grouped experts row {i}")
