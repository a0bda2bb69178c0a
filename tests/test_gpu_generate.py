"""Generation through the Python entry point and the command line against the plain implementation:
greedy and temperature sampling with fixed seeds, several requests at once, few pages."""
import os
import subprocess
import sys

import numpy as np
import pytest

import gpu_fixtures as gf
import plain_model as pm
import tiny_configs as tc

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _plain_continue(case, dtype, prompt, n_new, sampler, stop_ids=()):
    w, cfg = pm.load_plain(gf.model_dir(case))
    if dtype == "bfloat16":
        w = pm.round_weights_bf16(w)
    rnd = pm.bf16_rounding if dtype == "bfloat16" else pm.no_rounding
    tokens, out, gaps = list(prompt), [], []
    for _ in range(n_new):
        logits = pm.plain_forward(w, cfg, tokens, rnd)[-1].numpy()
        top2 = np.sort(logits)[-2:]
        gaps.append(float(top2[1] - top2[0]))
        nxt = sampler.sample(logits)
        out.append(nxt)
        tokens.append(nxt)
        if nxt in stop_ids:
            break
    return out, gaps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_of_tiny_a(dtype):
    """BASELINE's first configuration: 3 requests of 7/16/33 random ids, 16 greedy tokens each."""
    from geneinfer_b200 import Engine
    engine = Engine(gf.model_dir("a"), dtype=dtype, max_running=3, kv_pages=12, step_tokens=24, nvtx=True, debug_checks=True)
    prompts = [tc.random_tokens(n, 256, 40 + n) for n in (7, 16, 33)]
    got = engine.generate(prompts, max_new_tokens=16, temperature=0.0)
    for p, g in zip(prompts, got):
        want, gaps = _plain_continue("a", dtype, p, 16, pm.PlainSampler(0.0))
        assert len(g) == 16
        if g != want:       # only a near-tie of the two best logits may differ, and only from there on
            i = next(k for k in range(16) if g[k] != want[k])
            assert gaps[i] < (1e-4 if dtype == "float32" else 5e-2), f"token {i}: {g} != {want}"
    assert engine.stats.steps > 16 and not engine.steps.cache.requests


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_temperature_sampling_of_tiny_b(dtype):
    """BASELINE's second configuration: 5 requests of 1/5/24/64/100 ids, temperature 0.8, fixed seeds."""
    from geneinfer_b200 import Engine
    engine = Engine(gf.model_dir("b"), dtype=dtype, max_running=4, kv_pages=20, step_tokens=48, prefill_chunk=32)
    prompts = [tc.random_tokens(n, 384, 60 + n) for n in (1, 5, 24, 64, 100)]
    got = engine.generate(prompts, max_new_tokens=12, temperature=0.8, seed=77)
    agree = 0
    for i, (p, g) in enumerate(zip(prompts, got)):
        want, _ = _plain_continue("b", dtype, p, 12, pm.PlainSampler(0.8, 0, 1.0, seed=77 + i))
        assert len(g) == 12
        agree += g == want
        if dtype == "float32":
            assert g == want, f"request {i}: {g} != {want}"
    assert agree >= (5 if dtype == "float32" else 3)     # bfloat16: a draw next to a boundary may fall either way
    assert engine.steps.cache.free_pages() + engine.cached_blocks() == 20


def test_top_k_top_p_and_stop_ids_through_the_engine():
    from geneinfer_b200 import Engine, SamplingParams
    engine = Engine(gf.model_dir("b"), dtype="float32", max_running=2, kv_pages=16)
    prompt = tc.random_tokens(9, 384, 5)
    want, _ = _plain_continue("b", "float32", prompt, 10, pm.PlainSampler(1.1, 20, 0.8, seed=3))
    rid = engine.submit(prompt, len(prompt) + 9, SamplingParams(1.1, 20, 0.8, 3))
    stop = want[4]
    rid2 = engine.submit(prompt, 0, SamplingParams(1.1, 20, 0.8, 3), stop_ids=[stop])
    engine.run_until_idle()
    assert engine.result(rid).generated_tokens == want
    first = want.index(stop)
    assert engine.result(rid2).generated_tokens == want[:first + 1] and engine.result(rid2).stopped_by_end_token
    assert engine.result(rid2).cached_tokens == 0
    assert engine.cached_blocks() == 1, "the one full page of the 18-position request is indexed"


def test_greedy_and_sampled_requests_in_one_batch_with_steps_launched_ahead():
    """A greedy and a sampled request decode side by side: the sampling kernel leaves the greedy row's
    argmax in place, and the ids stay on the device for the step that is launched ahead."""
    from geneinfer_b200 import Engine, SamplingParams
    engine = Engine(gf.model_dir("b"), dtype="float32", max_running=2, kv_pages=16, prefix_cache=False)
    assert engine.scheduler.lookahead
    p1, p2 = tc.random_tokens(6, 384, 21), tc.random_tokens(11, 384, 22)
    want1, _ = _plain_continue("b", "float32", p1, 14, pm.PlainSampler(0.0))
    want2, _ = _plain_continue("b", "float32", p2, 14, pm.PlainSampler(0.9, 0, 1.0, seed=5))
    launched = []
    run = engine.scheduler._launch_ahead
    engine.scheduler._launch_ahead = lambda cur: launched.append(run(cur)) or launched[-1]
    r1 = engine.submit(p1, len(p1) + 13, SamplingParams(0.0))
    r2 = engine.submit(p2, len(p2) + 13, SamplingParams(0.9, 0, 1.0, 5))
    engine.run_until_idle()
    assert engine.result(r1).generated_tokens == want1
    assert engine.result(r2).generated_tokens == want2
    assert sum(x is not None for x in launched) >= 10, "no step was launched ahead"
    assert engine.steps.cache.free_pages() == 16 and not engine.steps.cache.requests


def test_decoding_without_the_tiled_weight_copy_gives_the_same_tokens():
    """The tile-by-tile copy of the weights changes how decode steps fetch them, not what they compute."""
    from geneinfer_b200 import Engine
    prompts = [tc.random_tokens(n, 500, 70 + n) for n in (9, 40, 3)]
    with_copy = Engine(gf.model_dir("c"), dtype="bfloat16", max_running=3, kv_pages=24, prefix_cache=False)
    without = Engine(gf.model_dir("c"), dtype="bfloat16", max_running=3, kv_pages=24, prefix_cache=False,
                     decode_weight_copy=False)
    assert with_copy.model.head.weight_tiles is not None and without.model.head.weight_tiles is None
    assert with_copy.model.weight_bytes() == without.model.weight_bytes()
    assert with_copy.generate(prompts, 12) == without.generate(prompts, 12)


def test_prefix_cache_gives_the_same_tokens():
    from geneinfer_b200 import Engine
    common = tc.random_tokens(40, 256, 9)
    prompts = [common + tc.random_tokens(5, 256, 90 + i) for i in range(3)]
    with_cache = Engine(gf.model_dir("a"), dtype="float32", max_running=1, kv_pages=24, prefix_cache=True)
    without = Engine(gf.model_dir("a"), dtype="float32", max_running=1, kv_pages=24, prefix_cache=False)
    assert with_cache.generate(prompts, 8) == without.generate(prompts, 8)
    assert with_cache.stats.prefix_tokens == 2 * 32 and without.stats.prefix_tokens == 0
    assert with_cache.cached_blocks() > 0
    with_cache.clear_prefix_cache()
    assert with_cache.steps.cache.free_pages() == 24


def test_command_line(tmp_path):
    prompt = tc.random_tokens(7, 256, 47)
    want, _ = _plain_continue("a", "float32", prompt, 6, pm.PlainSampler(0.0))
    dump = tmp_path / "tokens.txt"
    cmd = [sys.executable, os.path.join(ROOT, "bin", "gi_generate"), "--model", gf.model_dir("a"), "--prompt-ids",
           " ".join(map(str, prompt)), "--steps", str(len(prompt) + 5), "--temperature", "0", "--weights", "f32",
           "--dump-tokens", str(dump)]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr
    lines = dump.read_text().splitlines()
    assert [int(t) for t in lines[0].split()] == prompt and [int(t) for t in lines[1].split()] == want
    assert p.stdout.strip().endswith(" ".join(map(str, want))) and "[stats]" in p.stderr
    # --profile: the per-operation report of one decode step, in 32-bit and with the bfloat16 kernels
    prof = subprocess.run(cmd + ["--profile"], capture_output=True, text=True, timeout=600)
    assert prof.returncode == 0, prof.stderr
    assert "device profile: one decode step at context" in prof.stderr and "matrix products (32-bit)" in prof.stderr
    long_prompt = tc.random_tokens(150, 500, 48)
    prof = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "gi_generate"), "--model", gf.model_dir("c"), "--prompt-ids",
                           " ".join(map(str, long_prompt)), "--steps", "154", "--temperature", "0", "--profile", "--quiet"],
                          capture_output=True, text=True, timeout=600)
    assert prof.returncode == 0, prof.stderr
    lines = {l.split("  ")[1].strip(): l for l in prof.stderr.splitlines() if l.startswith("  ") and "%" in l}
    for op in ("attention", "rmsnorm", "matrix products (tensor cores)", "q/k/v projections + rope + store", "sampling"):
        assert op in lines, f"--profile does not report '{op}':\n{prof.stderr}"
    assert float(lines["matrix products (tensor cores)"].split()[-1]) > 0, "no weight rate for the products"
    bad = subprocess.run(cmd[:4] + ["--prompt", "hello"], capture_output=True, text=True)
    assert bad.returncode == 2 and "tokenizer" in bad.stderr
    missing = subprocess.run(cmd[:2] + ["--model", str(tmp_path / "nothing"), "--prompt-ids", "1"], capture_output=True, text=True)
    assert missing.returncode == 1 and "config.json" in missing.stderr
    # the random-weights mode: a folder from a configuration and a seed, the same tokens from the same seed,
    # the folder kept when --model names it
    import json
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(tc.TINY_B))
    made = tmp_path / "made"
    runs = []
    for extra in (["--model", str(made)], [], ["--dtype", "fp32"]):
        r = subprocess.run(cmd[:2] + ["--random-weights", "11", "--config", str(cfg_file), "--prompt-ids", "5 9 2", "--steps", "9",
                                      "--temperature", "0", "--no-echo"] + extra, capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr
        runs.append([int(t) for t in r.stdout.split()])
    assert len(runs[0]) == 7 and runs[0] == runs[1]        # positions 3..8 fed, the token after the last one also sampled
    assert (made / "config.json").is_file() and (made / "model.safetensors").is_file()
    assert sum(a != b for a, b in zip(runs[0], runs[2])) <= 2          # 32-bit on the same weights: near-ties at most
    alone = subprocess.run(cmd[:2] + ["--random-weights", "11", "--prompt-ids", "1"], capture_output=True, text=True)
    assert alone.returncode == 2 and "go together" in alone.stderr
    assert subprocess.run(cmd[:2] + ["--help"], capture_output=True, text=True).returncode == 0


def test_decode_timeline_from_inside_the_kernels():
    """bench_kernels.py decode_timeline: the library variant with time stamps is built, a decode step is recorded,
    and every kernel of a layer shows up with its events in order."""
    cmd = [sys.executable, os.path.join(ROOT, "bench_kernels.py"), "decode_timeline", "--batch", "2", "--context", "64",
           "--layers", "2", "--from-launch", "0", "--to-launch", "20"]
    run = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-2000:]
    lines = [l for l in run.stdout.splitlines() if " blocks | " in l]
    kinds = {l.split(" blocks | ")[0].split(None, 1)[1].rsplit(None, 1)[0].strip() for l in lines}
    assert {"rmsnorm", "product qkv+rope", "attention_decode", "product add", "product store", "swiglu"} <= kinds, run.stdout
    for l in lines:
        if "product add" in l:
            # the events that every block records (the first block of a cluster alone waits for partial tiles)
            every = ("enter", "waited", "first operands", "last MMA issued", "accumulator ready", "leave")
            stamps = [float(cell.split()[-1].split("..")[0]) for cell in l.split(" | ")[1:] if cell.rsplit(" ", 1)[0] in every]
            assert len(stamps) == len(every) and stamps == sorted(stamps), f"events out of order: {l}"
    assert "status word: 0" in run.stdout
