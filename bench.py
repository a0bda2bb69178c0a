#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at the Llama-3.2-1B shape with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--shape 1b|3b|8b] [--layers L]
    python bench.py --scenario mixed|prefix [--shape ...] [--dtype bfloat16|float32]
                                        (continuous batching / shared prefixes through the scheduler, see run_scenario)
    python bench.py --scenario sizes [--shape ...]   (decode steps at a grid of batch sizes and contexts, see run_sizes)

Prints ONE JSON line. ``value`` is decoded tokens per second at batch 8 and context 8192, timed on
the device over exactly K decode steps (one step = one token for every request of the batch);
``e2e`` is the same through the Python entry point (``Engine.step``: token ids from the host in,
sampled ids back to the host, every step). ``prefill`` is one 2,048-token prompt in one step (its
``frac`` is of the cuBLAS burst figure, ``frac_of_sustained`` of the sustained one); ``roofline``
relates the decode step's bytes (every weight once plus the cache of the live requests) to the
measured copy bandwidth, and ``rooflines`` gives the same fraction for every decode point;
``points`` holds decode at batch 1 and 64, at context 128, the prefill in four portions, and
``short_requests_b*``: requests of 16 prompt + 64 generated tokens through ``Engine.generate``.

``--impl reference`` runs the unmodified reference: its own ``gi_serve_bench`` with its CUDA
backend, built with its CMake files into baseline/_ref/build when it is not there yet, on the same
random model folder, at 8 concurrent requests of 16 prompt + 64 generated tokens (the workload that
finishes; the line says ``same_config: false`` and names ``points.short_requests_b8`` as the figure
to compare with). When it cannot be built or gives no result, the line says ``unavailable`` and why.

This engine runs on one GPU: for --gpus > 1 it prints one line saying so and exits with 2.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# BASELINE.json configs[2]: the Llama-3.2-1B shape.
LLAMA_1B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_act": "silu",
    "hidden_size": 2048, "intermediate_size": 8192, "num_hidden_layers": 16, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 64, "vocab_size": 128256, "max_position_embeddings": 131072,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
}
# The other two shapes the baseline names (not the default run): --shape 3b | 8b, usually with --layers.
LLAMA_3B = dict(LLAMA_1B, hidden_size=3072, num_hidden_layers=28, num_attention_heads=24, head_dim=128)
LLAMA_8B = dict(LLAMA_1B, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32,
                head_dim=128, tie_word_embeddings=False,
                rope_scaling=dict(LLAMA_1B["rope_scaling"], factor=8.0))
SHAPES = {"1b": ("Llama-3.2-1B", LLAMA_1B), "3b": ("Llama-3.2-3B", LLAMA_3B), "8b": ("Llama-3.1-8B", LLAMA_8B)}
CONTEXT = 8192
PAGE = 16
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                p = json.load(f)
            out = dict(FALLBACK_PEAKS)
            out.update({k: float(v) for k, v in p.items() if k in out and isinstance(v, (int, float))})
            out["source"] = "measured"
            return out
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


def model_folder(config, seed=1):
    """The random-weights model folder (made once per box under the temporary directory)."""
    from geneinfer_b200.weights import write_random_model
    tag = (f"geneinfer_bench_{config['num_hidden_layers']}x{config['hidden_size']}x{config['intermediate_size']}_"
           f"{int(config['tie_word_embeddings'])}_{seed}_{os.getuid()}")
    path = os.path.join(tempfile.gettempdir(), tag)
    if not (os.path.isfile(os.path.join(path, "model.safetensors")) and os.path.isfile(os.path.join(path, "done"))):
        t0 = time.time()
        print(f"[bench] writing random bf16 weights to {path}", file=sys.stderr, flush=True)
        write_random_model(config, seed, path, "bfloat16", std=0.02, norm_mean=1.0, norm_std=0.02)
        open(os.path.join(path, "done"), "w").close()
        print(f"[bench] wrote them in {time.time() - t0:.0f} s", file=sys.stderr, flush=True)
    return path


def step_bytes(model, cfg, batch, context):
    """Bytes a decode step has to read: every weight it uses once, and the cache of the live requests."""
    elt = 2
    kv_per_token = 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * elt * cfg["num_hidden_layers"]
    return model.weight_bytes() + batch * context * kv_per_token


def prefill_flops(cfg, T):
    D, I, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"]
    A = cfg["num_attention_heads"] * cfg["head_dim"]
    K = cfg["num_key_value_heads"] * cfg["head_dim"]
    gemm = 2 * T * (D * (A + 2 * K) + A * D + 2 * D * I + I * D) * L
    attention = 2 * T * T * cfg["head_dim"] * cfg["num_attention_heads"] * L      # causal: half of 2 products
    head = 2 * D * cfg["vocab_size"]
    return gemm + attention + head


def fill_cache(engine, keys, length):
    """Gives each request ``length`` cached positions of random keys and values (setup, untimed):
    decoding reads them exactly as it would read real ones."""
    for t in engine.group_pages:
        t.normal_(0.0, 1.0)
    for key in keys:
        rc = engine.open(key)
        engine.cache.reserve(rc, length)
        engine.cache.advance(rc, length)


def time_decode_device(engine, batch, context, steps, warmup, vocab):
    """K decode steps of the step function with greedy sampling on the device, timed with CUDA events."""
    import torch
    from geneinfer_b200.engine.step import StepEntry
    from geneinfer_b200.ops import kernels
    keys = [f"b{i}" for i in range(batch)]
    fill_cache(engine, keys, context - steps - warmup)
    ids = torch.zeros(batch, dtype=torch.int32, device=engine.device)
    g = torch.Generator().manual_seed(3)
    toks = torch.randint(0, vocab, (steps + warmup, batch), generator=g).tolist()

    def one(i):
        logits = engine.step([StepEntry(k, [toks[i][j]], [0]) for j, k in enumerate(keys)])
        kernels.argmax(logits, ids)

    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = kernels.launch_count()
    start.record()
    for i in range(warmup, warmup + steps):
        one(i)
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end)
    launches = kernels.launch_count() - launches0
    for k in keys:
        engine.close(k)
    return ms / steps, launches


def time_decode_e2e(llm, batch, context, steps, warmup, vocab):
    """The same decode steps through Engine.step(): host token ids in, sampled ids out, every step."""
    import torch
    from geneinfer_b200 import SamplingParams
    import numpy as np
    rng = np.random.default_rng(5)
    sched = llm.scheduler
    prefill = context - steps - warmup - 1
    for t in llm.steps.group_pages:
        t.normal_(0.0, 1.0)
    rids = []
    for i in range(batch):
        prompt = [int(t) for t in rng.integers(0, vocab, prefill + 1)]
        rids.append(llm.submit(prompt, 0, SamplingParams(0.0)))
    sched._admit()
    for job in sched.running:                     # setup, untimed: the prompt's cache is filled with random values
        llm.steps.cache.reserve(job.cache, prefill)
        llm.steps.cache.advance(job.cache, prefill)
        job.fed = prefill
    for _ in range(warmup):
        llm.step()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    start.record()
    for _ in range(steps):
        llm.step()
    end.record()
    torch.cuda.synchronize()
    wall_ms = (time.perf_counter() - t0) * 1e3
    assert all(len(llm.result(r).generated_tokens) == warmup + steps for r in rids)
    h2d = llm.steps._desc_size * 4
    d2h = batch * 4
    for job in list(sched.running):
        sched._finish(job)
    return wall_ms / steps, h2d, d2h


def time_prefill(engine, tokens, warmup, vocab, portions=1):
    """One prompt of ``tokens`` ids in ``portions`` equal steps; the median of three, in ms."""
    import torch
    from geneinfer_b200.engine.step import StepEntry
    g = torch.Generator().manual_seed(7)
    times = []
    n = tokens // portions
    for i in range(warmup + 3):
        prompt = torch.randint(0, vocab, (tokens,), generator=g).tolist()
        engine.open("p")
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for c in range(portions):
            engine.step([StepEntry("p", prompt[c * n:(c + 1) * n], [n - 1] if c == portions - 1 else [])])
        end.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(start.elapsed_time(end))
        engine.close("p")
    return sorted(times)[len(times) // 2]


SHORT_PROMPT, SHORT_NEW = 16, 64      # the reference arm's workload (its serve bench's own defaults)


def time_short_requests(llm, batch, vocab, runs=3):
    """``batch`` requests of 16 random prompt ids and 64 greedy tokens each through ``Engine.generate``
    (host token ids in, generated ids out), all submitted together: generated tokens per second of
    wall time, prompts included; the median of ``runs`` after one warm-up run."""
    import numpy as np
    import torch
    rng = np.random.default_rng(7)
    prompts = [[int(t) for t in rng.integers(0, vocab, SHORT_PROMPT)] for _ in range(batch)]
    walls = []
    for run in range(-1, runs):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = llm.generate(prompts, max_new_tokens=SHORT_NEW, temperature=0.0)
        torch.cuda.synchronize()
        if run >= 0:
            walls.append(time.perf_counter() - t0)
        assert all(len(o) == SHORT_NEW for o in out)
    return round(batch * SHORT_NEW / sorted(walls)[len(walls) // 2], 1)


def run_ours(args):
    import torch
    from geneinfer_b200 import Engine
    shape_name, shape = SHAPES[args.shape]
    cfg = dict(shape)
    layers_full = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    pk = peaks()
    folder = model_folder(cfg)
    vocab = cfg["vocab_size"]
    batch = 8
    pages_per_request = CONTEXT // PAGE

    def make(b):
        return Engine(folder, dtype="bfloat16", max_seq_len=CONTEXT, page_size=PAGE, kv_pages=b * pages_per_request,
                      max_running=b, step_tokens=PREFILL_TOKENS, prefix_cache=False)

    llm = make(batch)
    model = llm.model
    clocks = ClockSampler()
    clocks.start()
    ms_step, launches = time_decode_device(llm.steps, batch, CONTEXT, args.steps, args.warmup, vocab)
    ms_e2e, h2d, d2h = time_decode_e2e(llm, batch, CONTEXT, args.steps, args.warmup, vocab)
    ms_prefill = time_prefill(llm.steps, PREFILL_TOKENS, max(1, args.warmup), vocab)
    ms_prefill_4 = time_prefill(llm.steps, PREFILL_TOKENS, 1, vocab, portions=4)
    ms_short, _ = time_decode_device(llm.steps, batch, 128, args.steps, args.warmup, vocab)
    short = {f"short_requests_b{batch}": time_short_requests(llm, batch, vocab)}
    clock_record = clocks.stop()          # sampled through the timed regions above, which follow one another under load
    flops = prefill_flops(cfg, PREFILL_TOKENS)

    def roofline(b, context, ms):
        achieved = step_bytes(model, cfg, b, context) / (ms * 1e-3) / 1e9
        return {"achieved": round(achieved, 1), "frac": round(achieved / pk["hbm_gbs"], 4)}

    rooflines = {"decode_b8": roofline(batch, CONTEXT, ms_step), "decode_b8_context128": roofline(batch, 128, ms_short)}
    del llm
    torch.cuda.empty_cache()

    points = {"decode_b8_context128": round(batch / (ms_short * 1e-3), 1),
              "prefill_2048_in_4_portions": round(PREFILL_TOKENS / (ms_prefill_4 * 1e-3), 1)}
    for b in (1, 64):
        e = make(b)
        ms_b, _ = time_decode_device(e.steps, b, CONTEXT, args.steps, args.warmup, vocab)
        points[f"decode_b{b}"] = round(b / (ms_b * 1e-3), 1)
        rooflines[f"decode_b{b}"] = roofline(b, CONTEXT, ms_b)
        short[f"short_requests_b{b}"] = time_short_requests(e, b, vocab)
        del e
        torch.cuda.empty_cache()
    points.update(short)

    value = batch / (ms_step * 1e-3)
    line = {
        "metric": f"decode tok/s at batch 8, context 8192 ({shape_name} shape, random bf16 weights)",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights N(0,0.02), random token ids, random cache contents",
        "impl": "ours",
        "config": {
            "model": f"{shape_name} shape", "global_batch": batch, "seq_len": CONTEXT, "parallelism": "single GPU",
            "layers": cfg["num_hidden_layers"], "layers_of_named_config": layers_full, "hidden": cfg["hidden_size"],
            "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "intermediate": cfg["intermediate_size"], "vocab": vocab, "tied_head": cfg["tie_word_embeddings"], "page_size": PAGE,
            "rope": f"theta 500000, llama3 {cfg['rope_scaling']['factor']:g}/1/4/8192", "rms_norm_eps": cfg["rms_norm_eps"],
            "decode_weight_copy": True,
            "l2": "step inputs (weights + cache) are larger than L2", "peaks": pk["source"],
        },
        "e2e": {"value": round(batch / (ms_e2e * 1e-3), 1), "unit": "tok/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": round(ms_e2e, 4)},
        "gpu_launches": launches,
        "prefill": {"value": round(PREFILL_TOKENS / (ms_prefill * 1e-3), 1), "tokens": PREFILL_TOKENS,
                    "ms": round(ms_prefill, 3), "frac": round(flops / (ms_prefill * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                    "peak": pk["bf16_tflops"], "peak_kind": "cuBLAS bf16 burst, TFLOP/s",
                    "frac_of_sustained": round(flops / (ms_prefill * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4)},
        "roofline": dict(rooflines["decode_b8"], bound="hbm", peak=pk["hbm_gbs"], unit="GB/s"),
        "rooflines": rooflines,
        "points": points,
        "short_requests": "points.short_requests_b*: generated tok/s of b requests of 16 prompt + 64 generated tokens through "
                          "Engine.generate, wall time with the prompts (the workload of the reference arm)",
        "clocks": clock_record,
    }
    print(json.dumps(line), flush=True)
    return 0


def run_sizes(args):
    """Decode steps of the step function at a grid of batch sizes and context lengths (device time per step with CUDA
    events, the same timing as the default run's), each with its fraction of the HBM roofline. Prints one JSON line."""
    import torch
    from geneinfer_b200 import Engine
    shape_name, shape = SHAPES[args.shape]
    cfg = dict(shape)
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    pk = peaks()
    folder = model_folder(cfg)
    vocab = cfg["vocab_size"]
    contexts = (128, 2048, CONTEXT, 4 * CONTEXT)
    points = []
    for batch in (1, 4, 8, 16, 32, 64):
        longest = max(c for c in contexts if batch * c <= 64 * CONTEXT)             # at most 512 Ki cached positions
        llm = Engine(folder, dtype="bfloat16", max_seq_len=longest, page_size=PAGE, kv_pages=batch * ((longest + PAGE - 1) // PAGE),
                     max_running=batch, step_tokens=max(batch, 16), prefix_cache=False)
        for context in contexts:
            if context > longest:
                continue
            ms, _ = time_decode_device(llm.steps, batch, context, args.steps, args.warmup, vocab)
            achieved = step_bytes(llm.model, cfg, batch, context) / (ms * 1e-3) / 1e9
            points.append({"batch": batch, "context": context, "ms_per_step": round(ms, 4), "tok_s": round(batch / ms * 1e3, 1),
                           "gb_s": round(achieved, 1), "frac": round(achieved / pk["hbm_gbs"], 4)})
        llm.steps.check_status()
        del llm
        torch.cuda.empty_cache()
    print(json.dumps({"metric": f"decode steps at a grid of sizes ({shape_name} shape, random bf16 weights)", "impl": "ours", "n_gpus": 1,
                      "dtype": "bf16", "steps": args.steps, "warmup": args.warmup, "peak_gb_s": pk["hbm_gbs"],
                      "peaks": pk["source"], "points": points}))
    return 0


def run_scenario(args):
    """Two workloads through the entry point, beside the default run: ``mixed`` (32 requests with
    prompts of 128 to 4096 random ids and 256 generated tokens each, admitted together, prompts cut
    into portions beside decoding requests) and ``prefix`` (64 requests with 2,048-token prompts of
    which the first 1,024 are one of four shared prefixes, 512 generated tokens each, with the
    prefix cache on and off). Prints one JSON line."""
    import numpy as np
    import torch
    from geneinfer_b200 import Engine, SamplingParams
    shape_name, shape = SHAPES[args.shape]
    cfg = dict(shape)
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    folder = model_folder(cfg)
    vocab = cfg["vocab_size"]
    rng = np.random.default_rng(11)

    def ids(n):
        return [int(t) for t in rng.integers(0, vocab, n)]

    if args.scenario == "mixed":
        n_req, new, running = 32, 256, 32
        prompts = [ids(int(n)) for n in rng.integers(128, 4097, n_req)]
        variants = [("prefix_cache_on", True)]
    else:
        n_req, new, running = 64, 512, 64
        prefixes = [ids(1024) for _ in range(4)]
        prompts = [prefixes[i % 4] + ids(1024) for i in range(n_req)]
        variants = [("prefix_cache_on", True), ("prefix_cache_off", False)]
    longest = max(len(p) for p in prompts) + new
    pages = sum((len(p) + new + PAGE - 1) // PAGE + 1 for p in prompts)
    out = {"metric": f"{args.scenario} workload, generated tok/s ({shape_name} shape, random bf16 weights)", "impl": "ours",
           "n_gpus": 1, "dtype": "bf16", "data": "synthetic: seeded random weights and token ids",
           "config": {"model": f"{shape_name} shape", "layers": cfg["num_hidden_layers"], "requests": n_req,
                      "prompt_tokens": sum(len(p) for p in prompts), "generated_per_request": new, "max_running": running,
                      "step_tokens": 2048, "page_size": PAGE}}
    dtype = "float32" if args.dtype == "float32" else "bfloat16"
    out["dtype"] = "fp32" if dtype == "float32" else "bf16"
    results = {}
    for name, cache_on in variants:
        llm = Engine(folder, dtype=dtype, max_seq_len=longest, page_size=PAGE, kv_pages=pages, max_running=running,
                     step_tokens=2048, prefix_cache=cache_on)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        if args.scenario == "prefix":
            # the first request of each prefix arrives first; the others once its prompt is in the cache
            rids = [llm.submit(p, len(p) + new - 1, SamplingParams(0.0)) for p in prompts[:4]]
            while any(llm.result(r).first_token_step < 0 for r in rids):
                llm.step()
            rids += [llm.submit(p, len(p) + new - 1, SamplingParams(0.0)) for p in prompts[4:]]
        else:
            rids = [llm.submit(p, len(p) + new - 1, SamplingParams(0.0)) for p in prompts]
        llm.run_until_idle()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        res = [llm.result(r) for r in rids]
        bad = [r.error or len(r.generated_tokens) for r in res if r.error or len(r.generated_tokens) != new]
        if bad:
            raise RuntimeError(f"scenario {args.scenario}: requests did not finish as expected: {bad[:4]}")
        results[name] = [list(r.generated_tokens) for r in res]
        st = llm.stats
        out[name] = {"seconds": round(dt, 3), "generated_tok_s": round(n_req * new / dt, 1),
                     "all_tok_s": round((sum(len(p) for p in prompts) + n_req * new) / dt, 1), "steps": st.steps,
                     "preemptions": st.preemptions, "prefix_hits": st.prefix_hits, "cached_positions": st.prefix_tokens,
                     "evicted_pages": st.evicted_pages, "max_tokens_in_step": st.max_tokens_in_step}
        llm.clear_prefix_cache()
        llm.steps.cache.check_invariants()
        if llm.steps.cache.free_pages() != pages:
            raise RuntimeError("scenario: pages were lost")
        del llm
        torch.cuda.empty_cache()
    # a sampled subset again, each request alone (the reference's serve bench compares every request with its run
    # alone, bench/serve_bench_main.cpp:18,202). In 32-bit every output is one fixed chain of operations, so the tokens
    # must be identical; in bfloat16 a product of 1 token and one of 2,048 round differently, and the nearly flat logits
    # of random weights let a near-tie fall either way: there the count is reported, with the first place that differs.
    order = sorted(range(n_req), key=lambda i: len(prompts[i]))
    subset = sorted({order[0], order[n_req // 2], order[-1]})
    alone = Engine(folder, dtype=dtype, max_seq_len=longest, page_size=PAGE, kv_pages=(longest + PAGE - 1) // PAGE + 1,
                   max_running=1, step_tokens=2048, prefix_cache=False)
    same, first_diff = 0, None
    for i in subset:
        got = alone.generate([prompts[i]], max_new_tokens=new, temperature=0.0)[0]
        batched = results[variants[0][0]][i]
        if got == batched:
            same += 1
        elif first_diff is None:
            k = next(k for k in range(new) if got[k] != batched[k])
            # how close the two candidates were: the logits at that place once more (the request alone, fed in portions of 2,048)
            from geneinfer_b200.engine.step import StepEntry
            fed = list(prompts[i]) + batched[:k]
            alone.steps.open("gap")
            for c in range(0, len(fed), 2048):
                part = fed[c:c + 2048]
                logits = alone.steps.step([StepEntry("gap", part, [len(part) - 1] if c + 2048 >= len(fed) else [])])
            row = logits[0].float().cpu()
            alone.steps.close("gap")
            first_diff = {"request": i, "token": k, "logit_gap": round(abs(float(row[got[k]] - row[batched[k]])), 5),
                          "logit_spread": round(float(row.max() - row.median()), 3)}
    out["alone"] = {"requests_checked": len(subset), "identical_to_running_alone": same, "first_difference": first_diff}
    if dtype == "float32" and same != len(subset):
        raise RuntimeError(f"scenario {args.scenario}: in 32-bit a request generated other tokens than alone: {first_diff}")
    out["value"] = out[variants[0][0]]["generated_tok_s"]
    out["unit"] = "tok/s"
    print(json.dumps(out), flush=True)
    return 0


REF_DIR = os.path.join(ROOT, "baseline", "_ref")
REF_RUNS = 3


def reference_binary():
    """Path of the reference's own serve bench built with its CUDA backend, or (None, why). The
    reference is a CMake project (pip has nothing to install); its stock ``gi_serve_bench`` is built
    from the unmodified source tree into baseline/_ref/build when it is not there yet."""
    exe = os.path.join(REF_DIR, "build", "gi_serve_bench")
    if os.path.isfile(exe) and os.access(exe, os.X_OK):
        return exe, None
    src = os.environ.get("GI_REFERENCE_SRC") or os.path.join(os.path.dirname(ROOT), "reference")
    if not os.path.isfile(os.path.join(src, "CMakeLists.txt")):
        return None, f"the reference's source tree is not at {src} and no built gi_serve_bench is under baseline/_ref/build"
    os.makedirs(REF_DIR, exist_ok=True)
    steps = (["cmake", "-S", src, "-B", os.path.join(REF_DIR, "build"), "-DCMAKE_BUILD_TYPE=Release", "-DGI_CUDA=ON",
              "-DCMAKE_CUDA_ARCHITECTURES=100"],
             ["cmake", "--build", os.path.join(REF_DIR, "build"), "--target", "gi_serve_bench", "-j", "8"])
    env = dict(os.environ)
    if os.path.isfile("/usr/local/cuda/bin/nvcc"):
        env.setdefault("CUDACXX", "/usr/local/cuda/bin/nvcc")
    for cmd in steps:
        try:
            p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=1200, env=env)
        except (OSError, subprocess.TimeoutExpired) as e:
            return None, f"building the reference failed: {e}"
        if p.returncode != 0:
            tail = [l for l in p.stdout.splitlines() if l.strip()][-3:]
            return None, "building the reference with its CMake files failed: " + " | ".join(tail)[:400]
    return (exe, None) if os.path.isfile(exe) else (None, "the reference's build produced no gi_serve_bench")


def run_reference(args):
    """The unmodified reference through its own serve bench and CUDA backend, on the random model
    folder this bench writes: 8 requests of 16 prompt + 64 generated tokens run together, the
    workload that finishes (at context 8192 its run printed nothing within 15 minutes and is not
    run again). Nothing of this repository's models, kernels or engine is on this path."""
    if args.gpus != 1:
        print(json.dumps({"impl": "reference", "unavailable": "the reference's device backend runs on one GPU"}), flush=True)
        return 0
    exe, why = reference_binary()
    if exe is None:
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
        return 0
    shape_name, shape = SHAPES["1b"]
    cfg = dict(shape)
    folder = model_folder(cfg)
    batch = 8
    cmd = [exe, "--model", folder, "--device", "cuda", "--concurrency", str(batch), "--prompt-tokens", str(SHORT_PROMPT),
           "--decode-tokens", str(SHORT_NEW), "--runs", str(REF_RUNS), "--max-seq-len", "256"]
    clocks = ClockSampler()
    clocks.start()
    try:
        p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=1500)
    except (OSError, subprocess.TimeoutExpired) as e:
        clocks.stop()
        print(json.dumps({"impl": "reference", "unavailable": f"gi_serve_bench did not finish: {e}"}), flush=True)
        return 0
    clock_record = clocks.stop()
    row = None
    for l in p.stdout.splitlines():
        f = l.split()
        if len(f) >= 8 and f[0] == str(batch):
            try:
                row = (float(f[1]), float(f[2]), float(f[4]), " ".join(f[7:]))
            except ValueError:
                pass
    if row is None:
        tail = " | ".join([l for l in p.stdout.splitlines() if l.strip()][-3:])[:400]
        print(json.dumps({"impl": "reference", "unavailable": f"gi_serve_bench gave no result line (exit {p.returncode}): {tail}"}),
              flush=True)
        return 0
    wall, tps, rows_per_pass, outputs = row
    line = {
        "metric": f"generated tok/s, {batch} concurrent requests of {SHORT_PROMPT} prompt + {SHORT_NEW} generated tokens "
                  f"({shape_name} shape, random bf16 weights), wall time with the prompts",
        "value": tps, "unit": "tok/s", "n_gpus": 1, "impl": "reference", "same_config": False,
        "steps": REF_RUNS * SHORT_NEW, "warmup": SHORT_NEW, "ms_per_step": round(wall / SHORT_NEW * 1e3, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 weights; 32-bit activations and cache (the reference's device backend)",
        "data": "synthetic: the same random model folder as the other arm, the tool's own random token ids",
        "config": {"model": f"{shape_name} shape", "global_batch": batch, "seq_len": SHORT_PROMPT + SHORT_NEW,
                   "parallelism": "single GPU", "tool": "gi_serve_bench --device cuda", "runs": REF_RUNS,
                   "rows_per_pass": rows_per_pass, "outputs": outputs,
                   "compare_with": "points.short_requests_b8 of the other arm (the same workload through Engine.generate)",
                   "why_not_context_8192": "the reference's run at context 8192 printed no result within 15 minutes"},
        "e2e": {"value": tps, "unit": "tok/s", "note": "the tool's own wall clock: token ids from the host in, generated ids out"},
        "clocks": clock_record,
    }
    print(json.dumps(line), flush=True)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the named configuration (0 = all)")
    ap.add_argument("--shape", choices=sorted(SHAPES), default="1b", help="layer sizes (the default is the baseline's third configuration)")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16",
                    help="precision of a --scenario run (float32: the requests run alone must give identical tokens)")
    ap.add_argument("--scenario", choices=["mixed", "prefix", "sizes"], default="",
                    help="a workload through the scheduler (mixed, prefix) or decode steps at a grid of sizes, instead of the default run")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(3, args.warmup)
    if args.scenario == "sizes":
        return run_sizes(args)
    if args.scenario:
        return run_scenario(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
