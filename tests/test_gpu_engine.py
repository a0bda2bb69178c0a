"""The engine against the plain implementation under every way of cutting the work, in 32-bit and
in bfloat16: whole, tail decoded one by one, portions of changing size, mixed batches on so few
pages that they are used again, long decoding, the first tokens; and through bin/trace_run."""
import numpy as np
import pytest

import gpu_fixtures as gf
import trace_tools as tt

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
CASES = ["a", "b", "c", "d"]


def _play(case, dtype, steps, page_size=16):
    reqs = gf.requests(case)
    max_tokens = tt.max_tokens_of(steps, reqs)
    engine = gf.make_engine(case, dtype, n_pages=max_tokens // page_size, page_size=page_size)
    got = tt.run_in_process(engine, steps)
    if dtype == "bfloat16":
        from geneinfer_b200.ops import kernels
        assert kernels.gemm_tc_status(engine.device) == 0, "a bounded wait of a tensor-core kernel gave up"
    engine.cache.check_invariants()
    assert not engine.cache.requests, "requests left open"
    assert all(g.pool.free_count == g.pool.n_pages for g in engine.cache.groups), "pages were lost"
    return got


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", CASES + ["a_named", "b_named"])
def test_whole(case, dtype):
    got = _play(case, dtype, tt.trace_whole(gf.requests(case)))
    tt.compare(got, gf.plain_logits(case, dtype), gf.tolerance(dtype, case), f"whole {case} {dtype}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", CASES)
def test_tail_decoded_one_by_one(case, dtype):
    got = _play(case, dtype, tt.trace_tail_decode(gf.requests(case), tail=32))
    tt.compare(got, gf.plain_logits(case, dtype), gf.tolerance(dtype, case), f"tail {case} {dtype}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", CASES)
def test_portions_of_changing_size(case, dtype):
    got = _play(case, dtype, tt.trace_portions(gf.requests(case)))
    tt.compare(got, gf.plain_logits(case, dtype), gf.tolerance(dtype, case), f"portions {case} {dtype}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("seed", [1, 2])
def test_mixed_batches_reusing_pages(case, dtype, seed):
    reqs = gf.requests(case)
    steps = tt.trace_mixed(reqs, seed=seed)
    assert max(len(s["entries"]) for s in steps) >= 3
    total = sum(tt.round_up(len(t)) for t in reqs.values())
    assert tt.max_tokens_of(steps, reqs) < total, "the pool must be too small to hold all requests at once"
    got = _play(case, dtype, steps)
    tt.compare(got, gf.plain_logits(case, dtype), gf.tolerance(dtype, case), f"mixed {case} {dtype} seed {seed}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ["w", "w3"])
def test_full_widths_of_the_1b_and_3b_shapes(case, dtype):
    """Two layers at the real widths of Llama-3.2-1B (hidden 2048, 32:8 heads of 64, intermediate 8192,
    vocabulary 128256) and one at those of Llama-3.2-3B (hidden 3072, 24:8 heads of 128): the sizes at
    which the products split over K, run in clusters and tile the vocabulary, whole, with the tail
    decoded and in portions beside each other."""
    reqs = gf.requests(case)
    plain, tol = gf.plain_logits(case, dtype), gf.tolerance(dtype, case)
    whole = None
    for name, steps in (("whole", tt.trace_whole(reqs)), ("tail", tt.trace_tail_decode(reqs, tail=32)),
                        ("mixed", tt.trace_mixed(reqs, seed=4, max_live=2))):
        got = _play(case, dtype, steps)
        tt.compare(got, plain, tol, f"full widths {case}, {name}, {dtype}")
        if whole is None:
            whole = got
        elif dtype == "float32":       # one fixed chain of operations per output, at these widths too
            for key, row in got.items():
                assert np.array_equal(row, whole[key]), f"{case} {key}: the {name} cut differs from the whole prompt in 32-bit"


@pytest.mark.parametrize("dtype", DTYPES)
def test_cuts_agree_bitwise_in_32bit_and_closely_in_bf16(dtype):
    """The same position computed whole, decoded and in portions: identical in 32-bit (every output
    is one fixed chain of operations), within rounding in bfloat16."""
    case = "b"
    a = _play(case, dtype, tt.trace_whole(gf.requests(case)))
    b = _play(case, dtype, tt.trace_portions(gf.requests(case)))
    c = _play(case, dtype, tt.trace_mixed(gf.requests(case), seed=5))
    for other in (b, c):
        for key, row in other.items():
            if dtype == "float32":
                assert np.array_equal(row, a[key]), f"{key}: cuts differ in 32-bit"
            else:
                assert tt.rel_err(row, a[key]) < float(gf.tolerance(dtype, case))


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_and_first_tokens(dtype):
    """A request decoded token by token from its very first token to the end of the context."""
    case = "b"
    toks = gf.requests(case)["r6"]              # 256 tokens = the whole context
    steps = [{"step": i, "entries": [{"id": "r6", "tokens": [t], "want": [0]}], "end": ["r6"] if i == len(toks) - 1 else []}
             for i, t in enumerate(toks)]
    got = _play(case, dtype, steps)
    assert len(got) == len(toks)
    tt.compare(got, gf.plain_logits(case, dtype), gf.tolerance(dtype, case), f"long decode {dtype}")


@pytest.mark.parametrize("case,dtype,page_size", [("a", "float32", 8), ("a", "float32", 64), ("c", "bfloat16", 8),
                                                  ("c", "bfloat16", 32), ("c", "bfloat16", 64), ("d", "bfloat16", 128),
                                                  ("b", "bfloat16", 24), ("a", "float32", 1), ("b", "float32", 3),
                                                  ("b", "float32", 7), ("a", "float32", 1000), ("c", "bfloat16", 3),
                                                  ("b", "bfloat16", 7), ("d", "bfloat16", 1), ("c", "bfloat16", 1000)])
def test_other_page_sizes(case, dtype, page_size):
    """Pages smaller than, equal to and larger than the kernels' key tiles (the TMA boxes follow the
    page size), and a page size that TMA boxes cannot tile (24: the cp.async kernels)."""
    reqs = gf.requests(case)
    steps = tt.trace_mixed(reqs, seed=3)
    max_tokens = tt.max_tokens_of(steps, reqs, unit=max(64, page_size))
    engine = gf.make_engine(case, dtype, n_pages=max_tokens // page_size, page_size=page_size)
    got = tt.run_in_process(engine, steps)
    tt.compare(got, gf.plain_logits(case, dtype), gf.tolerance(dtype, case), f"page size {page_size}")


def test_portions_around_tile_edges_agree_bitwise_with_token_by_token_in_32bit():
    """Portions of 1, 2, 7, 8, 9, 15, 16, 17, 63, 64, 65 and 149 tokens (the sizes around the kernels' tiles and the
    pages' edges, tests/verify_device.py:140-153 of the reference) against the same request fed token by token:
    the same bits in 32-bit."""
    case = "c"
    toks = gf.requests(case)["r2"]                          # 512 tokens
    sizes = [1, 2, 7, 8, 9, 15, 16, 17, 63, 64, 65, 149]
    assert sum(sizes) <= len(toks)
    steps, p = [], 0
    for n in sizes:
        steps.append({"step": len(steps), "entries": [{"id": "r2", "tokens": toks[p:p + n], "want": list(range(n))}],
                      "end": ["r2"] if n == sizes[-1] else []})
        p += n
    by_portions = _play(case, "float32", steps)
    single = [{"step": i, "entries": [{"id": "r2", "tokens": [t], "want": [0]}], "end": ["r2"] if i == p - 1 else []}
              for i, t in enumerate(toks[:p])]
    one_by_one = _play(case, "float32", single)
    assert set(by_portions) == set(one_by_one)
    for key, row in by_portions.items():
        assert np.array_equal(row, one_by_one[key]), f"{key}: a portion and single tokens differ in 32-bit"
    tt.compare(by_portions, gf.plain_logits(case, "float32"), gf.tolerance("float32", case), "portions around tile edges")


def test_step_refuses_bad_input_and_leaves_state_unchanged():
    from geneinfer_b200.cache import OutOfPages
    from geneinfer_b200.engine.step import StepEntry
    engine = gf.make_engine("a", "float32", n_pages=4)
    engine.open("x")
    engine.open("y")
    with pytest.raises(IndexError):
        engine.step([StepEntry("x", [256], [0])])                 # token outside the vocabulary
    with pytest.raises(IndexError):
        engine.step([StepEntry("x", [1, 2], [2])])                # wanted place outside the tokens
    with pytest.raises(KeyError):
        engine.step([StepEntry("nobody", [1], [0])])
    with pytest.raises(ValueError):
        engine.step([StepEntry("x", [1], [0]), StepEntry("x", [2], [0])])
    with pytest.raises(IndexError):
        engine.step([StepEntry("x", [1] * 129, [])])              # beyond the context length
    engine.step([StepEntry("x", [1] * 40, [39])])                 # 3 of 4 pages
    free = engine.cache.free_pages()
    with pytest.raises(OutOfPages):
        engine.step([StepEntry("x", [2], [0]), StepEntry("y", [3] * 20, [0])])   # y needs 2 pages, 1 is free
    assert engine.cache.free_pages() == free and engine.length("x") == 40 and engine.length("y") == 0
    engine.cache.check_invariants()
    out = engine.step([StepEntry("x", [2], [0]), StepEntry("y", [3] * 16, [15])])
    assert out.shape == (2, 256)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", CASES)
def test_trace_run_tool(case, dtype, tmp_path):
    """bin/trace_run as a child process: all four ways of cutting in one trace."""
    reqs = gf.requests(case)
    steps = []
    for part in (tt.trace_whole(reqs), tt.trace_tail_decode(reqs), tt.trace_portions(reqs),
                 tt.trace_mixed(reqs, seed=9)):
        base = len(steps)
        steps += [dict(s, step=base + s["step"]) for s in part]
    vocab = gf.CASES[case][0]["vocab_size"]
    got = tt.run_trace_tool(gf.model_dir(case), dtype, steps, tt.max_tokens_of(steps, reqs), str(tmp_path / "out"), vocab)
    tt.compare(got, gf.plain_logits(case, dtype), gf.tolerance(dtype, case), f"trace_run {case} {dtype}")


def test_trace_run_taps(tmp_path):
    """``--taps`` writes the residual stream of the wanted rows with the reference's tags
    (tools/forward_main.cpp:92-102): checked against the plain implementation layer by layer."""
    import json
    import os
    import subprocess
    import sys
    import torch
    import plain_model as pm
    case = "a"
    toks = gf.requests(case)["r0"]
    head = 25
    steps = [{"step": 0, "entries": [{"id": "t", "tokens": toks[:head], "want": [0, head - 1]}], "end": []},
             {"step": 1, "entries": [{"id": "t", "tokens": toks[head:head + 1], "want": [0]}], "end": ["t"]}]
    out = tmp_path / "out"
    cmd = [sys.executable, os.path.join(tt.ROOT, "bin", "trace_run"), "--model", gf.model_dir(case), "--dtype", "float32",
           "--out", str(out), "--max-tokens", "64", "--taps"]
    p = subprocess.run(cmd, input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    w, cfg = pm.load_plain(gf.model_dir(case))
    D = cfg["hidden"] if "hidden" in cfg else w["model.embed_tokens.weight"].shape[1]
    n = head + 1
    cos, sin = pm.plain_rope_table(range(n), cfg["head_dim"], cfg["theta"], cfg["scaling"])
    x = pm.plain_embedding(w["model.embed_tokens.weight"], toks[:n])
    want = {"embedding": x.clone()}
    for l in range(cfg["layers"]):
        x = pm.plain_layer(x, w, f"model.layers.{l}.", cfg, cos, sin, pm.no_rounding)
        want[f"layer{l:02d}_ffn_out"] = x.clone()
    want["final_norm"] = pm.plain_rmsnorm(x, w["model.norm.weight"], cfg["eps"])
    for step, rows in ((0, [0, head - 1]), (1, [head])):
        for tag, full in want.items():
            got = np.fromfile(out / f"{step}.{tag}.f32", dtype="<f4").reshape(len(rows), D)
            assert tt.rel_err(got, full[rows].numpy()) < gf.TOL_F32, f"step {step}, tap {tag}"
        for l in range(cfg["layers"]):
            assert (out / f"{step}.layer{l:02d}_attn_out.f32").stat().st_size == len(rows) * D * 4
