"""The Zazulix decoder in the engine against the plain implementation under every way of cutting the work:
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
import plain_zazulix as P
import zazulix_models as M
from test_kedanex_replay_gpu import run_logging_routes
from test_replay_gpu import families

# float32: (largest, mean) |difference| relative to the largest |logit|.
TOL32 = (2e-5, 2e-6)
# bfloat16: a position's error is the root mean square over the vocabulary of the difference (its mean taken off) relative
# to that of the plain logits, and it is held against what rounding alone does at the same position (`rounding_alone`):
# no position beyond SINGLE times it, at most OVER_SHARE of the positions beyond OVER times it, the median of the ratio
# below MEDIAN.  A head of a retention layer whose output is near zero before its norm (the first tokens of a sequence)
# amplifies rounding at single positions; a lost key, state or tap moves every later position by several tenths.
FLOOR, SINGLE, OVER, OVER_SHARE, MEDIAN = 2e-3, 10.0, 3.0, 0.05, 1.5
CLOSE_CALL = 0.03      # a router's margin (in choice scores) below this may fall either way in bfloat16

pytestmark = pytest.mark.gpu
ROOT = os.path.join(os.path.dirname(os.path.abspath(__file__)), os.pardir)

CASES = {
    "A": dict(lengths=[7, 30, 61, 2, 45], page_tokens=4),
    "B": dict(lengths=[90, 5, 33, 140], page_tokens=16),
    "C": dict(lengths=[150, 20, 75, 210], page_tokens=16),
    "D": dict(lengths=[66, 3, 131, 40], page_tokens=8),
}
_cache = {}


def setup_case(tmp_path_factory, which, dtype):
    key = (which, dtype)
    if key not in _cache:
        d = M.make_model_dir(tmp_path_factory.mktemp("zazulix"), which, dtype)
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


def plain_along(cfg, weights, ids, routes, rounded=False):
    """The plain logits with the routed feed-forwards using the experts `routes` names (per routed layer [T, top];
    None: its own choices); `rounded`: with the inputs of the products, the queries and the cache narrowed."""
    P.route_choices = dict(zip(M.routed_prefixes(cfg), routes)) if routes else None
    P.round_inputs = to_bfloat16 if rounded else None
    try:
        return P.forward(cfg, weights, ids)
    finally:
        P.route_choices = P.round_inputs = None


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


def run_and_compare(engine, steps, cfg, weights, seqs, ref, dtype):
    """float32: the engine against the plain logits.  bfloat16: a close call of a router may fall the other way than in
    the plain implementation, and the request then goes on differently; so the engine's choices are logged, held against
    the plain ones wherever the margin is clear, and the plain implementation runs again along the engine's choices:
    every position is compared, none left out."""
    if dtype == torch.float32:
        got = helpers.run_trace_on_engine(engine, steps)
        compare(got, ref, seqs, dtype)
        return got
    got, routes = run_logging_routes(engine, steps, seqs)
    followed, slack = {}, {}
    for rid, ids in seqs.items():
        followed[rid] = plain_along(cfg, weights, ids, routes[rid])
        slack[rid] = centred_rms(plain_along(cfg, weights, ids, routes[rid], rounded=True) - followed[rid])
        free = _free_choices(cfg, weights, ids, routes[rid])
        for k, prefix in enumerate(M.routed_prefixes(cfg)):
            mine, margins = free[prefix]
            clear = margins >= CLOSE_CALL
            assert (np.sort(mine[clear], axis=1) == np.sort(routes[rid][k][clear], axis=1)).all(), \
                f"request {rid}: the experts of {prefix} differ where the choice was clear"
    compare(got, followed, seqs, dtype, slack)
    return got


def _free_choices(cfg, weights, ids, routes):
    """What the plain router would choose by itself at every token along the engine's path (the feed-forwards use the
    engine's experts): per routed feed-forward (choices [T, top], margins [T])."""
    seen = {}
    orig, orig_ff = P.route, P.routed_feed_forward

    def spy(z, correction, top, groups):
        out = orig(z, correction, top, groups)
        spy.rows.append((out[0], out[2]))
        return out

    def ff(h, w, p, mlp):
        spy.rows = []
        y = orig_ff(h, w, p, mlp)
        seen[p] = (np.asarray([r[0] for r in spy.rows], dtype=np.int64), np.asarray([r[1] for r in spy.rows]))
        return y

    P.route, P.routed_feed_forward = spy, ff
    P.route_choices = dict(zip(M.routed_prefixes(cfg), routes))
    try:
        P.forward(cfg, weights, ids)
    finally:
        P.route, P.routed_feed_forward, P.route_choices = orig, orig_ff, None
    return seen


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("which", ["A", "B", "C", "D"])
@pytest.mark.parametrize("family", ["whole", "tail", "portions", "mixed", "mixed_tight"])
def test_replay_matches_plain(tmp_path_factory, which, dtype, family):
    from hk_b200.engine import Engine
    d, cfg, weights, seqs, ref = setup_case(tmp_path_factory, which, dtype)
    steps = families(seqs)[family]
    max_tokens = helpers.peak_tokens(steps)
    engine = Engine(d, dtype=dtype, max_tokens=max_tokens, page_tokens=CASES[which]["page_tokens"], max_requests=4,
                    max_context=max_tokens, decode_graphs=dtype == torch.float32)     # the routers' choices are logged from
    # Python, which a replayed graph does not run: bfloat16 steps run eagerly here, and captured steps have a test of their own
    run_and_compare(engine, steps, cfg, weights, seqs, ref, dtype)
    engine.cache.books.audit()
    assert all(f == engine.cache.num_pages for f in engine.free_pages()), "pages were not all given back"
    if family == "tail" and dtype == torch.float32:
        assert engine.decode_graphs and engine._graphs[1].graph is not None      # single tokens replayed a captured graph


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("which", ["A", "C"])
def test_captured_decode_steps_equal_eager_ones(tmp_path_factory, which, dtype):
    from hk_b200.engine import Engine
    d, cfg, weights, seqs, ref = setup_case(tmp_path_factory, which, dtype)
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
        # so other roundings downstream (and now and then another expert); the two runs differ as either differs from the
        # plain logits
        eager = {rid: np.stack([runs[1][(rid, p)] for p in range(len(ids))]).astype(np.float64) for rid, ids in seqs.items()}
        slack = {rid: 2 * centred_rms(plain_along(cfg, weights, ids, None, rounded=True) - ref[rid]) for rid, ids in seqs.items()}
        compare(runs[0], eager, seqs, dtype, slack)


@pytest.mark.parametrize("which", ["A", "B", "D"])
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


@pytest.mark.parametrize("which", ["A", "B"])
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
    """A prompt of one token, then 170 tokens one by one (over many pages and past the window), beside a second
    request that starts later: every position against the plain implementation."""
    from hk_b200.engine import Engine
    d, cfg, w, _, _ = setup_case(tmp_path_factory, "C", dtype)
    a, b = M.prompts("C", np.random.default_rng(9), [171, 60])
    seqs = {"a": a, "b": b}
    ref = {"a": P.forward(cfg, w, a), "b": P.forward(cfg, w, b)}
    steps = [{"entries": [("a", a[:1], [0])], "end": []}]
    for i in range(1, 171):
        entries = [("a", [a[i]], [0])]
        if i == 100:
            entries.append(("b", b[:3], [0, 1, 2]))
        elif 100 < i <= 157:
            entries.append(("b", [b[i - 98]], [0]))
        steps.append({"entries": entries, "end": (["a"] if i == 170 else []) + (["b"] if i == 157 else [])})
    engine = Engine(d, dtype=dtype, max_tokens=helpers.peak_tokens(steps), page_tokens=16, max_requests=2,
                    decode_graphs=dtype == torch.float32)
    run_and_compare(engine, steps, cfg, w, seqs, ref, dtype)
    assert all(f == engine.cache.num_pages for f in engine.free_pages())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(tmp_path_factory, tmp_path, dtype):
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    d, cfg, weights, seqs, ref = setup_case(tmp_path_factory, "A", tdt)
    steps = families(seqs)["mixed"]
    out = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", str(out),
         "--max-tokens", str(helpers.peak_tokens(steps))],
        input=helpers.trace_to_jsonl(steps), capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split("\n")[:len(steps)] == [f"done {i}" for i in range(len(steps))]
    vocab = M.CONFIGS["A"]["vocab"]
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
    if tdt == torch.float32:
        compare(got, ref, seqs, tdt)
        return
    # The engine's choices are not at hand here, and a close call of a router may fall the other way than in the plain
    # implementation (the tests above follow the engine's choices).  The program must give what an engine gives that is
    # set up and driven as the program does it: the same kernels on the same numbers.
    from hk_b200.engine import Engine
    max_tokens = helpers.peak_tokens(steps)
    engine = Engine(d, dtype=dtype, max_tokens=max_tokens, page_tokens=16, max_requests=4, max_context=max_tokens,
                    max_batch_tokens=max_tokens)
    same = helpers.run_trace_on_engine(engine, steps)
    assert set(same) == set(got)
    scale = max(np.abs(r).max() for r in ref.values())
    off = [key for key in got if np.abs(got[key] - same[key]).max() > 1e-3 * scale]
    assert len(off) <= 0.03 * len(got), f"{len(off)} of {len(got)} positions differ from the engine's own, the first {sorted(off)[0]}"


def test_command_line_generates_with_this_design(tmp_path_factory):
    d, cfg, w, _, _ = setup_case(tmp_path_factory, "B", torch.float32)
    prompt = M.prompts("B", np.random.default_rng(2), [9])[0]
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "hk"), "run", d, "-p", ",".join(map(str, prompt)), "-n", "5",
                           "--temp", "0", "--dtype", "float32"], capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [int(t) for t in proc.stdout.replace(",", " ").split()] == plain_greedy(cfg, w, prompt, 5)
