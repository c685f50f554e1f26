"""Lodevik on the GPU against the plain implementation (tests/plain_lodevik.py), in 32-bit and in bfloat16: whole
prompts, prefill against token-by-token decoding, portions down to two tokens, batches of unequal requests against
each alone, slots, pages and per-slot state that are given back and used again, long decoding over every chunk's
edge, the first tokens of a sequence, and greedy generation through ``Engine.generate``."""
import pytest
import torch

from lodevik_helpers import LODE, MEDIAN_TOL, assert_rows_close, greedy_generate, make_model, oracle_logits, prompts

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
NAMES = sorted(LODE)


def build(tmp_path, name, dtype, max_tokens=2048, **kw):
    from zlm_b200 import Engine
    folder, cfg, ref = make_model(tmp_path, name, seed=5)
    return Engine.from_pretrained(folder, dtype=dtype, max_tokens=max_tokens, **kw), cfg, ref


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts(tmp_path, name, dtype):
    from zlm_b200 import StepEntry
    eng, cfg, ref = build(tmp_path, name, dtype)
    for i, n in enumerate([1, 2, 47, 48, 49, 64, 65, 131, 200, 333]):
        (p,) = prompts(cfg["vocab"], [n], seed=10 + i)
        s = eng.new_sequence()
        got = eng.step([StepEntry(s, p, list(range(n)))]).clone()
        eng.release(s)
        assert_rows_close(got, oracle_logits(ref, cfg, p), dtype, f"{name} whole prompt of {n}")
    eng.check(sync=True)
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prefill_then_token_by_token(tmp_path, name, dtype):
    """Decoding crosses page borders (64, 128, 192), the edges of every chunk (48, 64, 70, 96, 128, 130, 140 ...), and
    goes on for 170 steps; then a sequence decoded from its very first token (no token before it, no cache)."""
    from zlm_b200 import StepEntry
    eng, cfg, ref = build(tmp_path, name, dtype)
    n, head = 211, 41
    (p,) = prompts(cfg["vocab"], [n], seed=21)
    want = oracle_logits(ref, cfg, p)
    s = eng.new_sequence()
    got = [eng.step([StepEntry(s, p[:head], [head - 1])]).clone()]
    for t in range(head, n):
        got.append(eng.step([StepEntry(s, [p[t]], [0])]).clone())
    assert_rows_close(torch.cat(got), want[head - 1:], dtype, f"{name} token by token")
    s2 = eng.new_sequence()
    got = torch.cat([eng.step([StepEntry(s2, [p[t]], [0])]).clone() for t in range(12)])
    assert_rows_close(got, want[:12], dtype, f"{name} first tokens one by one")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("cuts", [[2, 2, 2, 59, 64, 1, 3, 37], [130, 40], [1, 63, 1, 105], [3, 300, 2], [47, 2, 21, 58, 2]])
def test_portions(tmp_path, name, dtype, cuts):
    """Portions of two tokens, portions that end on page borders and on chunk edges, portions that start one token
    after them, and a long one after a short one."""
    from zlm_b200 import StepEntry
    eng, cfg, ref = build(tmp_path, name, dtype)
    n = sum(cuts)
    (p,) = prompts(cfg["vocab"], [n], seed=33)
    s = eng.new_sequence()
    at, got = 0, []
    for c in cuts:
        got.append(eng.step([StepEntry(s, p[at:at + c], list(range(c)))]).clone())
        at += c
    assert_rows_close(torch.cat(got), oracle_logits(ref, cfg, p), dtype, f"{name} portions {cuts}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_and_reuse(tmp_path, name, dtype):
    """Three batches of unequal prompts, decoded together with short requests ending early, in a cache that holds
    little more than one batch: slots, pages and the slots' last tokens come back and are used again."""
    from zlm_b200 import StepEntry
    eng, cfg, ref = build(tmp_path, name, dtype, max_tokens=64 * 8, max_batch=4)
    for b in range(3):
        lens = [3, 70, 17, 1] if b % 2 == 0 else [65, 2, 128]
        extra = [4, 9, 1, 12][:len(lens)]
        full = prompts(cfg["vocab"], [l + e for l, e in zip(lens, extra)], seed=40 + b)
        want = [oracle_logits(ref, cfg, p) for p in full]
        slots = [eng.new_sequence() for _ in full]
        got = eng.step([StepEntry(s, p[:l], [0, l - 1] if l > 1 else [0]) for s, p, l in zip(slots, full, lens)]).clone()
        row = 0
        for j, l in enumerate(lens):
            places = [0, l - 1] if l > 1 else [0]
            assert_rows_close(got[row:row + len(places)], want[j][places], dtype, f"{name} batch {b} prompt {j}")
            row += len(places)
        for step in range(max(extra)):
            for j in range(len(full)):
                if step == extra[j]:
                    eng.release(slots[j])
            live = [j for j in range(len(full)) if step < extra[j]]
            got = eng.step([StepEntry(slots[j], [full[j][lens[j] + step]], [0]) for j in live]).clone()
            for r, j in enumerate(live):
                assert_rows_close(got[r], want[j][lens[j] + step], dtype, f"{name} batch {b} step {step} request {j}")
        for j in range(len(full)):
            if extra[j] == max(extra):
                eng.release(slots[j])
        eng.cache.check()
    assert eng.cache.tokens_held() == 0


@pytest.mark.parametrize("name", NAMES)
def test_fp32_logits_do_not_depend_on_cutting_or_batch_beyond_rounding(tmp_path, name):
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


def test_chunk_pages_come_back_while_a_sequence_grows(tmp_path):
    """A model whose layers all see their own chunk only gives the pages of the chunks before back as it goes: a
    sequence several times as long as the cache still runs, and agrees with the oracle."""
    from zlm_b200 import Engine, StepEntry
    from lodevik_helpers import _att, _lat, _layer
    cfg = {"architecture": "Lodevik", "vocab": 90, "width": 32, "norm": {"eps": 1e-5},
           "embedding": {"scale": 2.0, "bigram": {"buckets": 7, "mul_prev": 3, "mul_cur": 1}},
           "layers": [_layer("attention", _att(2, 1, 16, 16, 0.3, 0.25, 0.0, 100.0, 8, 64), 24),
                      _layer("latent_attention", _lat(2, 8, 8, 8, 16, 0.3, 100.0, 8, 128), 0)]}
    folder, cfg, ref = make_model(tmp_path, cfg, seed=3)
    eng = Engine.from_pretrained(folder, dtype="float32", max_tokens=64 * 4, max_seq_len=1024, max_batch=1)
    (p,) = prompts(cfg["vocab"], [700], seed=8)
    want = oracle_logits(ref, cfg, p)
    s = eng.new_sequence()
    got, at = [], 0
    for c in [100, 60, 1, 1, 130, 90] + [1] * 40 + [150, 128]:
        got.append(eng.step([StepEntry(s, p[at:at + c], [c - 1])]).clone())
        at += c
        eng.cache.check()
        assert eng.cache.tokens_held() <= 64 * 4
    ends = torch.tensor([100, 160, 161, 162, 292, 382] + list(range(383, 423)) + [572, 700]) - 1
    assert_rows_close(torch.cat(got), want[ends], "float32", "a sequence longer than the cache")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_greedy_generation(tmp_path, name, dtype):
    """``Engine.generate`` (scheduler, decode graphs with the slots' last tokens inside them, sampler) against the
    oracle's greedy continuation.  32-bit: the same tokens.  bfloat16: every chosen token is, for the oracle given the
    engine's own tokens so far, the best one or within rounding of it: a bfloat16 row differs from the oracle's by
    MEDIAN_TOL of its norm, which is that share of the row's root mean square a logit; two logits differ by sqrt(2)
    times that, and four such deviations are allowed."""
    eng, cfg, ref = build(tmp_path, name, dtype)
    ps = prompts(cfg["vocab"], [5, 40, 1, 66], seed=60)
    n = 12
    out = eng.generate(ps, max_tokens=n).tokens
    assert [len(o) for o in out] == [n] * len(ps)
    for p, o in zip(ps, out):
        if dtype == "float32":
            assert o == greedy_generate(ref, cfg, p, n)
        else:
            lg = oracle_logits(ref, cfg, list(p) + list(o))[len(p) - 1:-1]
            gap = lg.max(dim=-1).values - lg[torch.arange(n), torch.tensor(o)]
            allowed = 4 * 2 ** 0.5 * MEDIAN_TOL["bfloat16"] * lg.pow(2).mean(dim=-1).sqrt()
            assert bool((gap <= allowed).all()), f"{name}: a chosen token is {gap.max():.3f} below the best"
    eng.check(sync=True)
    # a second run in the same engine: captured decode steps are replayed on slots that were used before
    again = eng.generate(ps, max_tokens=n).tokens
    assert again == out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_replayed_decode_steps_give_the_logits_of_the_plain_implementation(tmp_path, name, dtype):
    """The sampler's decode steps (captured once, then replayed) against the oracle row by row: a captured step must
    contain every kernel of the eager one, also those that a note left in the step's context could make it skip."""
    from zlm_b200.sampling import SamplingParams
    eng, cfg, ref = build(tmp_path, name, dtype)
    ps = prompts(cfg["vocab"], [9, 70, 33], seed=77)
    more = prompts(cfg["vocab"], [10, 10, 10], seed=78)
    greedy = SamplingParams(temperature=0.0)
    for _ in range(2):          # the second round replays from its first step on
        slots = [eng.new_sequence() for _ in ps]
        eng.prefill_sample(slots, ps, greedy, [0, 1, 2])
        rows = []
        for t in range(10):
            eng.decode_sample(slots, [m[t] for m in more], greedy, [0, 1, 2])
            rows.append(eng.last_logits[: len(ps)].clone())
        for i, (p, m) in enumerate(zip(ps, more)):
            want = oracle_logits(ref, cfg, list(p) + list(m))[len(p):]
            assert_rows_close(torch.stack([r[i] for r in rows]), want, dtype, f"{name} replayed decode, request {i}")
        for s in slots:
            eng.release(s)
    assert eng.decoder.replays > 0 or not eng.decoder.use_graphs


def test_weights_read_back_by_name(tmp_path):
    eng, cfg, ref = build(tmp_path, "A", "float32")
    for n, t in ref.items():
        assert torch.equal(eng.tensor(n).cpu().double().reshape(t.shape), t), n


def test_trace_replay_runs_the_design(tmp_path):
    """bin/trace_run chooses the model class by config.json and replays a schedule with a batch."""
    from helpers import TraceRun
    folder, cfg, ref = make_model(tmp_path, "A", seed=7)
    a, b = prompts(cfg["vocab"], [20, 9], seed=70)
    out = str(tmp_path / "out")
    run = TraceRun(folder, "float32", out, 256)
    got0 = run.step(0, [{"id": "x", "tokens": a[:19], "want": [0, 18]}, {"id": "y", "tokens": b[:8], "want": [7]}])
    got1 = run.step(1, [{"id": "x", "tokens": a[19:], "want": [0]}, {"id": "y", "tokens": b[8:], "want": []}], end=["x", "y"])
    assert run.close() == 0
    wa, wb = oracle_logits(ref, cfg, a), oracle_logits(ref, cfg, b)
    V = cfg["vocab"]
    assert_rows_close(torch.from_numpy(got0.reshape(-1, V).copy()), torch.stack([wa[0], wa[18], wb[7]]), "float32")
    assert_rows_close(torch.from_numpy(got1.reshape(-1, V).copy()), wa[19:20], "float32")


def test_command_line_writes_and_runs_a_random_model(tmp_path, capsys):
    """``random-model`` from a Lodevik config.json, then ``run`` on the folder it wrote: the tokens are those of
    ``Engine.generate`` on the same folder."""
    import json
    from zlm_b200 import Engine
    from zlm_b200.cli import main
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(LODE["A"]))
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
