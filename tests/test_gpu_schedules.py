"""Schedules that serving runs and the small traces do not: a live set that grows past and shrinks
below what decode graphs were captured with; prompt portions of hundreds of tokens on top of cached
tokens (the scheduler's default chunking); sixteen and sixty-four live requests in one step; a
request forked from another with a partly filled page (copy-on-write on the device); and an engine
whose pool is so small that it must preempt and evict. Everything against the plain implementation.
"""
import numpy as np
import pytest

import gpu_fixtures as gf
import plain_model as pm
import tiny_configs as tc
import trace_tools as tt

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


def _plain_rows(case, dtype, requests, wanted):
    """Plain logits of the wanted positions only: {request: {position: row}}."""
    w, cfg = pm.load_plain(gf.model_dir(case))
    rnd = pm.no_rounding
    if dtype == "bfloat16":
        w, rnd = pm.round_weights_bf16(w), pm.bf16_rounding
    out = {}
    for rid, positions in wanted.items():
        positions = sorted(set(positions))
        rows = pm.plain_forward(w, cfg, requests[rid], rnd, positions=positions).numpy()
        out[rid] = dict(zip(positions, rows))
    return out


def _plain_and_bound(case, dtype, requests, wanted):
    """The plain rows to compare with and the bound they must be met within. In bfloat16 the model's own
    noise (rounding against exact plain implementation) is measured on these very rows: it grows with
    the length of a request, and these requests are longer than the ones the case's standard noise is from."""
    plain = _plain_rows(case, dtype, requests, wanted)
    if dtype == "float32":
        return plain, gf.tolerance(dtype, case)
    exact = _plain_rows(case, "float32", requests, wanted)
    noise = max(tt.rel_err(plain[r][p], exact[r][p]) for r in plain for p in plain[r])
    return plain, gf.tolerance(dtype, case, noise=max(noise, gf.bf16_noise(case)))


def _check_greedy_continuation(w, cfg, rnd, prompt, generated, dtype, what):
    """Every generated token against the plain logits of its own past (teacher-forced: one plain pass over prompt
    and generated tokens gives the logits at every place, each depending only on the tokens before it); only a
    near-tie of the two candidates may differ."""
    tokens = list(prompt) + list(generated)
    places = list(range(len(prompt) - 1, len(tokens) - 1))
    logits = pm.plain_forward(w, cfg, tokens[:-1], rnd, positions=places).numpy()
    for k, t in enumerate(generated):
        best = int(np.argmax(logits[k]))
        if t != best:
            gap = float(logits[k][best] - logits[k][t])
            assert gap < (1e-4 if dtype == "float32" else 5e-2), f"{what} token {k}: {t} != {best} (gap {gap})"


def _wanted(steps):
    wanted = {}
    for rows in tt.wanted_positions(steps).values():
        for rid, pos in rows:
            wanted.setdefault(rid, []).append(pos)
    return wanted


def _finish(engine, dtype):
    if dtype == "bfloat16":
        from geneinfer_b200.ops import kernels
        assert kernels.gemm_tc_status(engine.device) == 0, "a bounded wait of a tensor-core kernel gave up"
    engine.check_status()
    engine.cache.check_invariants()
    assert not engine.cache.requests, "requests left open"
    assert all(g.pool.free_count == g.pool.n_pages for g in engine.cache.groups), "pages were lost"


# ------------------------------------------------------------------ graphs and a changing live set
@pytest.mark.parametrize("grow_on_demand", [False, True])
@pytest.mark.parametrize("dtype", DTYPES)
def test_live_set_grows_and_shrinks_under_graphs(dtype, grow_on_demand):
    """3 requests decode (their steps are captured into a graph), then 20, then the first 3 again:
    the replayed graph of the small batch must still read and write the buffers that are in use
    after the large batch. With ``grow_on_demand`` every scratch buffer starts small and is replaced
    by a larger one when the 20 arrive (what a large vocabulary does to the logits buffer): graphs
    captured before must not be replayed on the freed memory."""
    case = "c"
    vocab = gf.CASES[case][0]["vocab_size"]
    reqs = {f"g{i}": tc.random_tokens(60 + 3 * i, vocab, 300 + i) for i in range(20)}
    first, rest = list(reqs)[:3], list(reqs)[3:]
    steps, fed = [], {r: 0 for r in reqs}

    def step(entries, end=()):
        steps.append({"step": len(steps), "entries": entries, "end": list(end)})

    def decode(rids, end=()):
        entries = [{"id": r, "tokens": [reqs[r][fed[r]]], "want": [0]} for r in rids]
        for r in rids:
            fed[r] += 1
        step(entries, end)

    step([{"id": r, "tokens": reqs[r][:20], "want": [19]} for r in first])
    for r in first:
        fed[r] = 20
    for _ in range(5):
        decode(first)
    for k in range(0, len(rest), 4):                     # the others arrive, four prompts a step, beside the decoding ones
        new = rest[k:k + 4]
        entries = [{"id": r, "tokens": [reqs[r][fed[r]]], "want": [0]} for r in first]
        entries += [{"id": r, "tokens": reqs[r][:24], "want": [5, 23]} for r in new]
        for r in first:
            fed[r] += 1
        for r in new:
            fed[r] = 24
        step(entries)
    for k in range(6):
        decode(first + rest, end=rest if k == 5 else ())
    for k in range(8):
        decode(first, end=first if k == 7 else ())

    engine = gf.make_engine(case, dtype, n_pages=20 * 7, max_requests=20, max_step_tokens=128)
    assert engine.use_graphs
    if grow_on_demand:
        engine._SCRATCH_AT_ONCE = 1
    got = tt.run_in_process(engine, steps)
    assert engine.graph_replays >= 12, "the decode steps were not replayed from graphs"
    _finish(engine, dtype)
    tt.compare(got, _plain_rows(case, dtype, reqs, _wanted(steps)), gf.tolerance(dtype, case), f"grow and shrink {dtype}")


def test_bounded_caches_of_graphs_and_launch_programs():
    """With room for two graphs and three launch programs only, old entries are dropped and made again: the
    logits stay what they are with room for all."""
    case, dtype = "c", "bfloat16"
    reqs = gf.requests(case)
    steps = tt.trace_mixed(reqs, seed=7) + []
    roomy = gf.make_engine(case, dtype, n_pages=tt.max_tokens_of(steps, reqs) // 16)
    want = tt.run_in_process(roomy, steps)
    tight = gf.make_engine(case, dtype, n_pages=tt.max_tokens_of(steps, reqs) // 16)
    tight.max_graphs, tight.max_programs = 2, 3
    got = tt.run_in_process(tight, steps)
    assert len(tight._graphs) <= 2 and len(tight._programs) <= 3
    assert len(roomy._programs) > 3, "the trace was meant to meet more shapes than the tight engine keeps"
    for key, row in want.items():
        assert np.array_equal(row, got[key]), f"{key}: dropping and re-making a graph or a program changed the logits"
    _finish(tight, dtype)


# ------------------------------------------------------------------ long portions on a cache that is not empty
LONG_CUTS = {
    "c": [[1, 511], [17, 495], [300, 212]],
    "d": [[1, 383], [17, 367], [200, 184]],
    "w": [[1, 450], [17, 600], [300, 130, 500]],
    "w3": [[1, 200], [17, 330], [300, 131]],
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ["c", "d", "w", "w3"])
def test_long_portions_on_cached_tokens(case, dtype):
    """Portions of 130 to 600 tokens on top of 1, 17 and 300 cached tokens, the cuts the scheduler
    makes of long prompts: the many-token products, the rotation in their epilogue and the prefill
    attention start at a position that is not 0, on pages that are partly filled."""
    vocab = gf.CASES[case][0]["vocab_size"]
    reqs, steps = {}, []
    for i, cuts in enumerate(LONG_CUTS[case]):
        rid = f"long{i}"
        toks = tc.random_tokens(sum(cuts), vocab, 500 + i)
        reqs[rid] = toks
        p = 0
        for k, n in enumerate(cuts):
            # logits at the portion's first and last tokens, around the first page edge inside it and in its middle
            edge = (-(p) % 16) or 16
            want = sorted({0, 1, min(edge - 1, n - 1), min(edge, n - 1), n // 2, n - 2, n - 1} & set(range(n)))
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[p:p + n], "want": want}],
                          "end": [rid] if k == len(cuts) - 1 else []})
            p += n
    engine = gf.make_engine(case, dtype, n_pages=tt.max_tokens_of(steps, reqs) // 16, max_step_tokens=640)
    got = tt.run_in_process(engine, steps)
    _finish(engine, dtype)
    plain, bound = _plain_and_bound(case, dtype, reqs, _wanted(steps))
    tt.compare(got, plain, bound, f"long portions {case} {dtype}")


# ------------------------------------------------------------------ many live requests
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case,live", [("c", 16), ("c", 64), ("d", 16), ("d", 64)])
def test_many_live_requests(case, live, dtype):
    """Sixteen and sixty-four requests live at a time: steps with that many decode rows beside prompt
    portions, block tables of that many requests, products of 33 to 128 tokens, on a pool that cannot
    hold all requests at once."""
    vocab = gf.CASES[case][0]["vocab_size"]
    n = live + live // 2
    reqs = {f"m{i}": tc.random_tokens(int(34 + (i * 7) % 45), vocab, 700 + i) for i in range(n)}
    steps = tt.trace_mixed(reqs, seed=live, max_live=live, tail=24)
    assert max(len(s["entries"]) for s in steps) >= live // 2
    held = tt.max_tokens_of(steps, reqs)
    assert held < sum(tt.round_up(len(t)) for t in reqs.values())
    engine = gf.make_engine(case, dtype, n_pages=held // 16, max_requests=live, max_step_tokens=live * 40)
    got = tt.run_in_process(engine, steps)
    _finish(engine, dtype)
    tt.compare(got, _plain_rows(case, dtype, reqs, _wanted(steps)), gf.tolerance(dtype, case),
               f"{live} live requests {case} {dtype}")


# ------------------------------------------------------------------ copy-on-write on the device
@pytest.mark.parametrize("case,dtype", [("b", "float32"), ("c", "bfloat16")])
def test_forked_request_copies_the_shared_page_before_writing(case, dtype):
    """B starts on the first m positions of A, m inside a page both share, and goes on with tokens
    of its own while A goes on with its; then C forks all of A, its partly filled last page included,
    and both write into that page's next row. Each must equal its own whole sequence: the shared
    page was copied on the device before the first write (tools/multiseq_check_main.cpp:260-316)."""
    from geneinfer_b200.engine.step import StepEntry
    vocab = gf.CASES[case][0]["vocab_size"]
    a = tc.random_tokens(75, vocab, 901)
    m = 41                                                   # row 9 of the third page
    b = a[:m] + tc.random_tokens(30, vocab, 902)
    c = a[:70] + tc.random_tokens(5, vocab, 903)
    reqs = {"A": a, "B": b, "C": c}
    engine = gf.make_engine(case, dtype, n_pages=16)
    got = {}

    def run(entries):
        logits = engine.step([StepEntry(rid, toks, want) for rid, toks, want, _ in entries]).float().cpu().numpy()
        k = 0
        for rid, _, want, base in entries:
            for w in want:
                got[(rid, base + w)] = logits[k].copy()
                k += 1

    engine.open("A")
    run([("A", a[:60], [59], 0)])
    engine.fork("A", "B", m)
    ta, tb = engine.cache.requests["A"].tables[0], engine.cache.requests["B"].tables[0]
    assert list(tb[:3]) == list(ta[:3])
    run([("B", b[m:m + 12], list(range(12)), m), ("A", a[60:65], list(range(5)), 60)])   # B writes rows 9.. of the shared page
    assert tb[2] != ta[2] and tb[0] == ta[0] and tb[1] == ta[1], "B still shares the page it wrote into"
    run([("B", b[m + 12:], list(range(len(b) - m - 12)), m + 12), ("A", a[65:70], list(range(5)), 65)])
    engine.fork("A", "C")                                    # 70 positions: the fifth page holds 6 rows
    tc_ = engine.cache.requests["C"].tables[0]
    assert list(tc_[:5]) == list(ta[:5])
    run([("A", a[70:], list(range(5)), 70), ("C", c[70:], list(range(5)), 70)])
    assert tc_[4] != ta[4] and list(tc_[:4]) == list(ta[:4])
    for rid in ("A", "B", "C"):
        engine.close(rid)
    _finish(engine, dtype)
    plain = _plain_rows(case, dtype, reqs, {rid: [p for (r, p) in got if r == rid] for rid in reqs})
    tt.compare(got, plain, gf.tolerance(dtype, case), f"copy-on-write {case} {dtype}")


# ------------------------------------------------------------------ rewinding a request
@pytest.mark.parametrize("case,dtype", [("b", "float32"), ("c", "bfloat16")])
def test_a_rewound_request_goes_on_like_a_fresh_one(case, dtype):
    """A request is fed 70 tokens, rewound to 37 (into the middle of a page; the rows beyond stay in the page as
    they are) and fed other tokens: the logits are those of the new sequence as a whole."""
    from geneinfer_b200.engine.step import StepEntry
    vocab = gf.CASES[case][0]["vocab_size"]
    first = tc.random_tokens(70, vocab, 951)
    second = first[:37] + tc.random_tokens(40, vocab, 952)
    engine = gf.make_engine(case, dtype, n_pages=8)
    engine.open("r")
    engine.step([StepEntry("r", first, [69])])
    free = engine.cache.free_pages()
    engine.truncate("r", 37)
    assert engine.length("r") == 37 and engine.cache.free_pages() == free + 2      # 5 pages -> 3
    got = {}
    logits = engine.step([StepEntry("r", second[37:60], list(range(23)))]).float().cpu().numpy()
    got.update({("r", 37 + k): logits[k].copy() for k in range(23)})
    for p in range(60, 77):
        got[("r", p)] = engine.step([StepEntry("r", [second[p]], [0])]).float().cpu().numpy()[0].copy()
    engine.close("r")
    _finish(engine, dtype)
    plain = _plain_rows(case, dtype, {"r": second}, {"r": list(range(37, 77))})
    tt.compare(got, plain, gf.tolerance(dtype, case), f"rewound request {case} {dtype}")


# ------------------------------------------------------------------ preemption and eviction on the engine
@pytest.mark.parametrize("dtype", DTYPES)
def test_engine_preempts_and_evicts_when_pages_run_out(dtype):
    """A pool that cannot hold the running requests to their ends: the scheduler must evict pages of
    the prefix cache and preempt the youngest request, and every request must still generate what the
    plain implementation generates alone (the reference's engine test fails if neither ever happened,
    tests/verify_engine.py:98-103)."""
    from geneinfer_b200 import Engine
    case = "b"
    engine = Engine(gf.model_dir(case), dtype=dtype, max_running=4, kv_pages=14, step_tokens=64, prefill_chunk=24,
                    prefix_cache=True)
    common = tc.random_tokens(34, 384, 77)
    prompts = [common + tc.random_tokens(3 + 4 * i, 384, 80 + i) for i in range(7)]
    new = 40
    got = engine.generate(prompts, max_new_tokens=new, temperature=0.0)
    st = engine.stats
    assert st.preemptions > 0, "the pool was meant to be too small: no request was preempted"
    assert st.evicted_pages > 0, "no page of the prefix cache was evicted"
    assert st.prefix_hits > 0
    w, cfg = pm.load_plain(gf.model_dir(case))
    rnd = pm.no_rounding
    if dtype == "bfloat16":
        w, rnd = pm.round_weights_bf16(w), pm.bf16_rounding
    for i, (p, g) in enumerate(zip(prompts, got)):
        assert len(g) == new
        _check_greedy_continuation(w, cfg, rnd, p, g, dtype, f"request {i}")
    engine.clear_prefix_cache()
    assert engine.steps.cache.free_pages() == 14 and not engine.steps.cache.requests
    engine.steps.cache.check_invariants()


# ------------------------------------------------------------------ the entry point with sixteen running requests
@pytest.mark.parametrize("dtype", DTYPES)
def test_engine_with_sixteen_running_requests_across_context_buckets(dtype, tmp_path):
    """Twenty requests through ``Engine`` with sixteen running at a time: prompts from 3 to 1,030 tokens, so that
    decode steps cross the context buckets their graphs are keyed by (256, 1,024, 2,048), a stop token for some,
    more requests than places. The tokens must be the ones the engine gives without CUDA graphs and launch
    programs, and the ones the plain implementation's logits name (teacher-forced; only a near-tie may differ)."""
    from geneinfer_b200 import Engine, SamplingParams
    config = dict(tc.TINY_C, max_position_embeddings=1280)
    folder = tc.make_model_dir(config, tc.SHARP_C, str(tmp_path / "c_long"))
    vocab = config["vocab_size"]
    lengths = [3, 250, 1030, 17, 260, 1000, 64, 255, 1019, 129, 5, 300, 980, 31, 240, 1024, 90, 270, 33, 512]
    prompts = [tc.random_tokens(n, vocab, 1200 + i) for i, n in enumerate(lengths)]
    new = 24

    def run(plain_launches):
        engine = Engine(folder, dtype=dtype, max_running=16, kv_pages=16 * 40 + 200, step_tokens=512, prefill_chunk=300,
                        prefix_cache=False)
        if plain_launches:
            engine.steps.use_graphs = engine.steps.use_programs = False
        ids = [engine.submit(p, len(p) + new - 1, SamplingParams(0.0), stop_ids=[7, 11] if i % 3 == 0 else ())
               for i, p in enumerate(prompts)]
        engine.run_until_idle()
        out = [engine.result(i) for i in ids]
        assert all(not r.error for r in out)
        assert engine.stats.max_running_seen == 16 and not engine.steps.cache.requests
        engine.steps.check_status()
        return engine, [list(r.generated_tokens) for r in out], [r.stopped_by_end_token for r in out]

    fast, got, stopped = run(False)
    assert fast.steps.graph_replays > 10 and fast.steps.program_runs > 10
    _, want, want_stopped = run(True)
    assert got == want and stopped == want_stopped, "graphs or launch programs change the tokens"
    assert any(stopped) or all(len(g) == new for g in got)
    w, cfg = pm.load_plain(folder)
    rnd = pm.no_rounding
    if dtype == "bfloat16":
        w, rnd = pm.round_weights_bf16(w), pm.bf16_rounding
    for i in (0, 2, 5, 8, 15, 19):                           # the shortest, the longest, the ones at the buckets' edges
        _check_greedy_continuation(w, cfg, rnd, prompts[i], got[i], dtype, f"request {i}")
