"""The Mifolorn decoder in the engine against the plain implementation under every way of cutting the work:
whole prompts, the last tokens one by one (through captured decode graphs), portions down to two tokens, mixed
batches of unequal requests over a pool so small that pages and state slots are used again; then greedy generation
through the entry point and the scheduler, long decoding from a first token on, and the replay program."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers
import mifolorn_models as M
import plain_mifolorn as P
from test_replay_gpu import families

# float32: (largest, mean) |difference| relative to the largest |logit|.
TOL32 = (2e-5, 2e-6)
# bfloat16: a position's error is the root mean square over the vocabulary of the difference (its mean taken off) relative
# to that of the plain logits, and it is held against what rounding alone does at the same position (`rounding_alone`).
# These models run their layers two or three times and norm every head of the recurrent mixers' small outputs, so a head
# whose output is near zero before its norm amplifies rounding at single positions: the engine's error may be up to
# SINGLE times the model's there (the largest seen is 6), at most OVER_SHARE of the positions may be beyond OVER times
# it, and the median of the ratio stays below MEDIAN.  A lost key, state or tap moves every later position by several
# tenths, tens of times what rounding does.
FLOOR, SINGLE, OVER, OVER_SHARE, MEDIAN = 2e-3, 10.0, 3.0, 0.05, 1.5

pytestmark = pytest.mark.gpu
ROOT = os.path.join(os.path.dirname(os.path.abspath(__file__)), os.pardir)

CASES = {
    "U": dict(lengths=[7, 30, 61, 2, 45], page_tokens=4),
    "V": dict(lengths=[90, 5, 33, 140], page_tokens=16),
    "W": dict(lengths=[150, 20, 75, 210], page_tokens=16),
    "X": dict(lengths=[66, 3, 131, 40], page_tokens=8),
}
_cache = {}


def setup_case(tmp_path_factory, which, dtype):
    key = (which, dtype)
    if key not in _cache:
        d = M.make_model_dir(tmp_path_factory.mktemp("mifolorn"), which, dtype)
        cfg, weights = M.load_plain(d)
        seqs = {f"r{i}": p for i, p in enumerate(M.prompts(which, np.random.default_rng(17), CASES[which]["lengths"]))}
        ref = {rid: P.forward(cfg, weights, ids) for rid, ids in seqs.items()}
        _cache[key] = (d, cfg, weights, seqs, ref)
    return _cache[key]


def to_bfloat16(x):
    return torch.from_numpy(np.ascontiguousarray(x)).to(torch.bfloat16).double().numpy()


def centred_rms(x):
    x = x - x.mean(axis=-1, keepdims=True)
    return np.sqrt((x * x).mean(axis=-1))


def rounding_alone(cfg, weights, seqs, ref):
    """What rounding alone does to the plain logits, per request and position (by a coarse model: the inputs of the
    matrix products, the queries and the cache narrowed, nothing else), as a centred root mean square."""
    P.round_inputs = to_bfloat16
    try:
        return {rid: centred_rms(P.forward(cfg, weights, ids) - ref[rid]) for rid, ids in seqs.items()}
    finally:
        P.round_inputs = None


def compare(got, ref, seqs, dtype, slack=None):
    """Every position against the plain logits; the FIRST position out of tolerance is reported, since its place says
    what is special about it."""
    assert len(got) == sum(len(v) for v in seqs.values())
    for (rid, p), v in got.items():
        assert np.isfinite(v).all(), f"non-finite logits at {rid}:{p}"
    if dtype == torch.float32:
        scale = max(np.abs(r).max() for r in ref.values())
        means = []
        for (rid, p), v in sorted(got.items()):
            d = np.abs(v.astype(np.float64) - ref[rid][p])
            means.append(d.mean())
            assert d.max() <= TOL32[0] * scale, f"first wrong position: request {rid} position {p}: |diff| {d.max():.3g}"
        assert np.mean(means) <= TOL32[1] * scale
        return
    scale = np.sqrt(np.mean(np.concatenate([centred_rms(r) ** 2 for r in ref.values()])))
    ratios, over = [], []
    for (rid, p), v in sorted(got.items()):
        e = centred_rms(v.astype(np.float64) - ref[rid][p]) / scale
        s = slack[rid][p] / scale + FLOOR
        assert e <= SINGLE * s, f"first wrong position: request {rid} position {p}: error {e:.3g}, rounding alone {s:.3g}"
        ratios.append(e / s)
        if e > OVER * s:
            over.append((rid, p))
    assert len(over) <= max(1, OVER_SHARE * len(ratios)), f"{len(over)} of {len(ratios)} positions are beyond rounding, the first {over[0]}"
    assert np.median(ratios) <= MEDIAN, f"the median error is {np.median(ratios):.2f} times what rounding alone does"


def check(got, cfg, weights, seqs, ref, dtype):
    compare(got, ref, seqs, dtype, rounding_alone(cfg, weights, seqs, ref) if dtype == torch.bfloat16 else None)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("which", ["U", "V", "W", "X"])
@pytest.mark.parametrize("family", ["whole", "tail", "portions", "mixed", "mixed_tight"])
def test_replay_matches_plain(tmp_path_factory, which, dtype, family):
    from hk_b200.engine import Engine
    d, cfg, weights, seqs, ref = setup_case(tmp_path_factory, which, dtype)
    steps = families(seqs)[family]
    max_tokens = helpers.peak_tokens(steps)
    engine = Engine(d, dtype=dtype, max_tokens=max_tokens, page_tokens=CASES[which]["page_tokens"], max_requests=4,
                    max_context=max_tokens)
    check(helpers.run_trace_on_engine(engine, steps), cfg, weights, seqs, ref, dtype)
    engine.cache.books.audit()
    assert all(f == engine.cache.num_pages for f in engine.free_pages()), "pages were not all given back"
    if family == "tail":
        assert engine.decode_graphs and engine._graphs[1].graph is not None      # single tokens replayed a captured graph


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("which", ["U", "W"])
def test_captured_decode_steps_equal_eager_ones(tmp_path_factory, which, dtype):
    from hk_b200.engine import Engine
    d, _, _, seqs, _ = setup_case(tmp_path_factory, which, dtype)
    steps = helpers.trace_mixed(seqs, np.random.default_rng(8), max_live=3, decode_tail=25)
    runs = []
    for graphs in (True, False):
        engine = Engine(d, dtype=dtype, max_tokens=helpers.peak_tokens(steps), page_tokens=8, max_requests=3, decode_graphs=graphs)
        runs.append(helpers.run_trace_on_engine(engine, steps))
        if graphs:
            assert any(g.graph is not None for g in engine._graphs.values())
    if dtype == torch.float32:
        for key, v in runs[0].items():
            assert np.array_equal(v, runs[1][key]), key
    else:
        # a captured step cuts a request's keys into a fixed number of ranges, an eager one by the batch: other sums, and
        # so other roundings downstream; the two runs differ as either differs from the plain logits
        _, cfg, weights, seqs, ref = setup_case(tmp_path_factory, which, dtype)
        eager = {rid: np.stack([runs[1][(rid, p)] for p in range(len(ids))]).astype(np.float64) for rid, ids in seqs.items()}
        compare(runs[0], eager, seqs, dtype, rounding_alone(cfg, weights, seqs, ref))


@pytest.mark.parametrize("which", ["U", "W"])
def test_logits_do_not_depend_on_the_cut_the_batch_or_the_slot(tmp_path_factory, which):
    from hk_b200.engine import Engine
    d, _, _, seqs, ref = setup_case(tmp_path_factory, which, torch.float32)
    runs = {}
    for family in ("whole", "portions", "mixed_tight"):
        steps = families(seqs)[family]
        engine = Engine(d, dtype="float32", max_tokens=helpers.peak_tokens(steps), page_tokens=8, max_requests=2 if family == "mixed_tight" else 4)
        runs[family] = helpers.run_trace_on_engine(engine, steps)
    scale = max(np.abs(r).max() for r in ref.values())
    for key, v in runs["whole"].items():
        for family in ("portions", "mixed_tight"):
            assert np.abs(runs[family][key] - v).max() <= 4e-6 * scale, (family, key)


def plain_greedy(cfg, w, prompt, n):
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(np.argmax(P.forward(cfg, w, ids)[-1])))
    return ids[len(prompt):]


@pytest.mark.parametrize("which", ["U", "V"])
def test_greedy_generation_through_the_entry_point_and_the_scheduler(tmp_path_factory, which):
    import hk_b200
    from hk_b200.api import GenerationStats, generate_with_engine
    d, cfg, w, _, _ = setup_case(tmp_path_factory, which, torch.float32)
    prompts = M.prompts(which, np.random.default_rng(5), [5, 19, 40, 33, 2])
    want = [plain_greedy(cfg, w, p, 6) for p in prompts]
    assert hk_b200.generate(d, prompts, max_new_tokens=6, temperature=0, dtype="float32") == want
    # two slots and a tight pool: requests wait for a slot, portions are short, pages and state slots are used again
    eng = hk_b200.Engine(d, dtype="float32", max_tokens=128, page_tokens=8, max_requests=2, max_context=64, max_batch_tokens=24)
    st = GenerationStats()
    assert generate_with_engine(eng, prompts, 6, temperature=0, prefill_chunk=11, stats=st) == want
    assert st.generated_tokens == 30 and all(f == eng.cache.num_pages for f in eng.free_pages())
    assert generate_with_engine(eng, prompts[::-1], 6, temperature=0, prefill_chunk=7) == want[::-1]     # the same engine again


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_long_decoding_and_first_tokens(tmp_path_factory, dtype):
    """A prompt of one token, then 170 tokens one by one (over many pages), beside a second request that starts
    later: every position against the plain implementation."""
    from hk_b200.engine import Engine
    d, cfg, w, _, _ = setup_case(tmp_path_factory, "W", dtype)
    a, b = M.prompts("W", np.random.default_rng(9), [171, 60])
    ref = {"a": P.forward(cfg, w, a), "b": P.forward(cfg, w, b)}
    steps = [{"entries": [("a", a[:1], [0])], "end": []}]
    for i in range(1, 171):
        entries = [("a", [a[i]], [0])]
        if i == 100:
            entries.append(("b", b[:3], [0, 1, 2]))
        elif 100 < i <= 157:
            entries.append(("b", [b[i - 98]], [0]))
        steps.append({"entries": entries, "end": (["a"] if i == 170 else []) + (["b"] if i == 157 else [])})
    engine = Engine(d, dtype=dtype, max_tokens=helpers.peak_tokens(steps), page_tokens=16, max_requests=2)
    check(helpers.run_trace_on_engine(engine, steps), cfg, w, {"a": a, "b": b}, ref, dtype)
    assert all(f == engine.cache.num_pages for f in engine.free_pages())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(tmp_path_factory, tmp_path, dtype):
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    d, cfg, weights, seqs, ref = setup_case(tmp_path_factory, "U", tdt)
    steps = families(seqs)["mixed"]
    out = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", str(out),
         "--max-tokens", str(helpers.peak_tokens(steps))],
        input=helpers.trace_to_jsonl(steps), capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split("\n")[:len(steps)] == [f"done {i}" for i in range(len(steps))]
    vocab = M.CONFIGS["U"]["vocab"]
    got, pos = {}, {}
    for i, st in enumerate(steps):
        wanted = sum(len(w) for _, _, w in st["entries"])
        if wanted:
            arr = np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(wanted, vocab)
            r = 0
            for rid, toks, want in st["entries"]:
                for w in want:
                    got[(rid, pos.get(rid, 0) + w)] = arr[r]
                    r += 1
        for rid, toks, _ in st["entries"]:
            pos[rid] = pos.get(rid, 0) + len(toks)
    check(got, cfg, weights, seqs, ref, tdt)


def test_command_line_generates_with_this_design(tmp_path_factory):
    d, cfg, w, _, _ = setup_case(tmp_path_factory, "V", torch.float32)
    prompt = M.prompts("V", np.random.default_rng(2), [9])[0]
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "hk"), "run", d, "-p", ",".join(map(str, prompt)), "-n", "5",
                           "--temp", "0", "--dtype", "float32"], capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [int(t) for t in proc.stdout.replace(",", " ").split()] == plain_greedy(cfg, w, prompt, 5)
