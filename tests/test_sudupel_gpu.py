"""Sudupel on the GPU against the plain implementation (tests/plain_sudupel.py), in 32-bit and in bfloat16: whole
prompts, prefill against token-by-token decoding, portions down to two tokens, batches of unequal requests against
each alone, slots, pages and states that are given back and used again, long decoding, the first tokens of a
sequence, and greedy generation through ``Engine.generate``."""
import pytest
import torch

from sudupel_helpers import SUDU, assert_rows_close, greedy_generate, make_model, oracle, prompts

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
NAMES = sorted(SUDU)


def build(tmp_path, name, dtype, max_tokens=2048, **kw):
    from zlm_b200 import Engine
    folder, cfg, ref = make_model(tmp_path, name, seed=5)
    return Engine.from_pretrained(folder, dtype=dtype, max_tokens=max_tokens, **kw), cfg, ref


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts(tmp_path, name, dtype):
    """Also a prompt long enough for the fixed-decay recurrence to run in pieces side by side."""
    from zlm_b200 import StepEntry
    eng, cfg, ref = build(tmp_path, name, dtype)
    for i, n in enumerate([1, 2, 63, 64, 65, 200, 333]):
        (p,) = prompts(cfg["vocab"], [n], seed=10 + i)
        s = eng.new_sequence()
        got = eng.step([StepEntry(s, p, list(range(n)))]).clone()
        eng.release(s)
        oracle(ref, cfg, p, dtype).check(got, range(n), dtype, f"{name} whole prompt of {n}")
    eng.check(sync=True)
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prefill_then_token_by_token(tmp_path, name, dtype):
    """Decoding crosses two page borders (64, 128), lets every window pass over decoded tokens, and goes on for 150
    steps."""
    from zlm_b200 import StepEntry
    eng, cfg, ref = build(tmp_path, name, dtype)
    n, head = 211, 61
    (p,) = prompts(cfg["vocab"], [n], seed=21)
    want = oracle(ref, cfg, p, dtype)
    s = eng.new_sequence()
    got = [eng.step([StepEntry(s, p[:head], [head - 1])]).clone()]
    for t in range(head, n):
        got.append(eng.step([StepEntry(s, [p[t]], [0])]).clone())
    want.check(torch.cat(got), range(head - 1, n), dtype, f"{name} token by token")
    # and a sequence decoded from its very first token (convolutions and states start from nothing)
    s2 = eng.new_sequence()
    got = torch.cat([eng.step([StepEntry(s2, [p[t]], [0])]).clone() for t in range(12)])
    want.check(got, range(12), dtype, f"{name} first tokens one by one")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("cuts", [[2, 2, 2, 59, 64, 1, 3, 37], [130, 40], [1, 63, 1, 105], [3, 300, 2]])
def test_portions(tmp_path, name, dtype, cuts):
    """Portions shorter than a convolution's taps, portions that end on page borders, and a long one after states
    that are not zero."""
    from zlm_b200 import StepEntry
    eng, cfg, ref = build(tmp_path, name, dtype)
    n = sum(cuts)
    (p,) = prompts(cfg["vocab"], [n], seed=33)
    want = oracle(ref, cfg, p, dtype)
    s = eng.new_sequence()
    at, got = 0, []
    for c in cuts:
        got.append(eng.step([StepEntry(s, p[at:at + c], list(range(c)))]).clone())
        at += c
    want.check(torch.cat(got), range(n), dtype, f"{name} portions {cuts}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_and_reuse(tmp_path, name, dtype):
    """Three batches of unequal prompts, decoded together with short requests ending early, in a cache that holds
    little more than one batch: slots, pages and per-slot states come back and are used again."""
    from zlm_b200 import StepEntry
    eng, cfg, ref = build(tmp_path, name, dtype, max_tokens=64 * 7, max_batch=4)
    for b in range(3):
        lens = [3, 70, 17, 1] if b % 2 == 0 else [65, 2, 128]
        extra = [4, 9, 1, 12][:len(lens)]
        full = prompts(cfg["vocab"], [l + e for l, e in zip(lens, extra)], seed=40 + b)
        want = [oracle(ref, cfg, p, dtype) for p in full]
        slots = [eng.new_sequence() for _ in full]
        got = eng.step([StepEntry(s, p[:l], [0, l - 1] if l > 1 else [0]) for s, p, l in zip(slots, full, lens)]).clone()
        row = 0
        for j, l in enumerate(lens):
            places = [0, l - 1] if l > 1 else [0]
            want[j].check(got[row:row + len(places)], places, dtype, f"{name} batch {b} prompt {j}")
            row += len(places)
        for step in range(max(extra)):
            for j in range(len(full)):
                if step == extra[j]:
                    eng.release(slots[j])
            live = [j for j in range(len(full)) if step < extra[j]]
            got = eng.step([StepEntry(slots[j], [full[j][lens[j] + step]], [0]) for j in live]).clone()
            for r, j in enumerate(live):
                want[j].check(got[r], [lens[j] + step], dtype, f"{name} batch {b} step {step} request {j}")
        for j in range(len(full)):
            if extra[j] == max(extra):
                eng.release(slots[j])
        eng.cache.check()
    assert eng.cache.tokens_held() == 0


@pytest.mark.parametrize("name", NAMES)
def test_fp32_logits_do_not_depend_on_cutting_or_batch_beyond_rounding(tmp_path, name):
    """32-bit: a position's logits whole, in portions, token by token or beside other requests agree to rounding."""
    from zlm_b200 import StepEntry
    eng, cfg, _ = build(tmp_path, name, "float32")
    a, b = prompts(cfg["vocab"], [290, 31], seed=50)
    s = eng.new_sequence()
    whole = eng.step([StepEntry(s, a, list(range(290)))]).clone()
    eng.release(s)
    s, s2 = eng.new_sequence(), eng.new_sequence()
    got = eng.step([StepEntry(s2, b, [30]), StepEntry(s, a[:270], list(range(270)))])[1:].clone()
    rest = [eng.step([StepEntry(s2, [b[0]], []), StepEntry(s, [a[t]], [0])]).clone() for t in range(270, 290)]
    assert_rows_close(torch.cat([got] + rest), whole, "float32", f"{name} cuttings", tol=2e-5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_greedy_generation(tmp_path, name, dtype):
    """``Engine.generate`` (scheduler, decode graphs with the per-slot states inside them, sampler) against the
    oracle's greedy continuation.  32-bit: the same tokens.  bfloat16: every chosen token is, for the oracle given the
    engine's own tokens so far, the best one or within rounding of it."""
    eng, cfg, ref = build(tmp_path, name, dtype)
    ps = prompts(cfg["vocab"], [5, 40, 1, 66], seed=60)
    n = 12
    out = eng.generate(ps, max_tokens=n).tokens
    assert [len(o) for o in out] == [n] * len(ps)
    for p, o in zip(ps, out):
        if dtype == "float32":
            assert o == greedy_generate(ref, cfg, p, n)
        else:
            full = oracle(ref, cfg, list(p) + list(o), dtype)          # (positions that hang on a router's close call are left out)
            lg, safe = full.logits[len(p) - 1:-1], full.safe[len(p) - 1:-1]
            gap = lg.max(dim=-1).values - lg[torch.arange(n), torch.tensor(o)]
            assert bool((gap <= 0.05 * lg.std(dim=-1))[safe].all()), f"{name}: a chosen token is {gap[safe].max():.3f} below the best"
    eng.check(sync=True)
    # a second run in the same engine: captured decode steps are replayed on slots whose states were used before
    again = eng.generate(ps, max_tokens=n).tokens
    assert again == out


def test_weights_read_back_by_name(tmp_path):
    eng, cfg, ref = build(tmp_path, "A", "float32")
    for n, t in ref.items():
        assert torch.equal(eng.tensor(n).cpu().double().reshape(t.shape), t), n


def test_trace_replay_runs_the_design(tmp_path):
    """bin/trace_run chooses the model class by config.json and replays a schedule with a batch."""
    from helpers import TraceRun
    import plain_sudupel as P
    folder, cfg, ref = make_model(tmp_path, "A", seed=7)
    a, b = prompts(cfg["vocab"], [20, 9], seed=70)
    out = str(tmp_path / "out")
    run = TraceRun(folder, "float32", out, 256)
    got0 = run.step(0, [{"id": "x", "tokens": a[:19], "want": [0, 18]}, {"id": "y", "tokens": b[:8], "want": [7]}])
    got1 = run.step(1, [{"id": "x", "tokens": a[19:], "want": [0]}, {"id": "y", "tokens": b[8:], "want": []}], end=["x", "y"])
    assert run.close() == 0
    wa, wb = P.forward(cfg, ref, a)[0].float(), P.forward(cfg, ref, b)[0].float()
    V = cfg["vocab"]
    assert_rows_close(torch.from_numpy(got0.reshape(-1, V).copy()), torch.stack([wa[0], wa[18], wb[7]]), "float32")
    assert_rows_close(torch.from_numpy(got1.reshape(-1, V).copy()), wa[19:20], "float32")


def test_command_line_writes_and_runs_a_random_model(tmp_path, capsys):
    """``random-model`` from a Sudupel config.json, then ``run`` on the folder it wrote: the tokens are those of
    ``Engine.generate`` on the same folder."""
    import json
    from zlm_b200 import Engine
    from zlm_b200.cli import main
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(SUDU["A"]))
    folder = str(tmp_path / "model")
    assert main(["random-model", "--config", str(cfg_path), "--seed", "3", "--out", folder]) == 0
    capsys.readouterr()
    assert main(["run", folder, "-p", "5 17 3", "-p", "9 9", "--max-tokens", "6", "--dtype", "float32"]) == 0
    lines = [l.split("\t") for l in capsys.readouterr().out.splitlines() if "\t" in l and l[0].isdigit()]
    got = {0: [], 1: []}
    for req, tok in lines:
        got[int(req)].append(int(tok))
    want = Engine.from_pretrained(folder, dtype="float32", max_tokens=256).generate([[5, 17, 3], [9, 9]], max_tokens=6).tokens
    assert [got[0], got[1]] == want


@pytest.mark.parametrize("name", NAMES)
def test_a_batch_of_many_requests_through_captured_steps(tmp_path, name):
    """24 unequal requests generated together (decode steps of more than 16 rows: the many-token forms of the kernels
    inside captured steps) give, in 32-bit, the tokens that each request gives alone."""
    eng, cfg, _ = build(tmp_path, name, "float32", max_tokens=64 * 64, max_batch=32)
    ps = prompts(cfg["vocab"], [3 + (7 * i) % 40 for i in range(24)], seed=9)
    together = eng.generate(ps, max_tokens=10).tokens
    alone = [eng.generate([p], max_tokens=10).tokens[0] for p in ps]
    assert together == alone
    eng.check(sync=True)
