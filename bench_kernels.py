"""Small workloads of single kernels and of whole steps, for timing and for profiler captures.

    python bench_kernels.py <case> [--shape 1b|3b|8b] [--batch B] [--context C] [--tokens T] [--layers L] [--repeat R]

Cases at the layer sizes of one of bench.py's shapes (random data, sizes larger than L2 where bandwidth matters):
  gemm_prefill       the four products of a layer for T tokens (tensor cores, persistent kernel)
  gemm_decode        the same products for B tokens (weights on the 128-row side, read tile by tile, split over K)
  attention_decode   B single tokens, each over a context of C cached positions
  attention_prefill  one prompt of T tokens, with the mma.sync kernel and with the tcgen05 kernel
  decode_step        R whole decode steps of B requests at context C through the step function
  prefill_step       R whole prefills of T tokens through the step function
  prefill_timeline   the same for a prompt portion of T tokens on top of C cached positions
  decode_timeline    one graph-replayed decode step of B requests at context C, seen from inside: the kernels of a library
                     built with time stamps (it is compiled at the first call) record when their blocks enter, wait, compute
                     and leave; prints one line per launch of the layers --from-launch .. --to-launch
Each case prints the time per launch measured with CUDA events. Under a profiler, give --repeat a
small value and select the kernel by name.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import bench  # noqa: E402  (the shapes and the model folder are bench.py's)

PAGE = bench.PAGE
D = H = HKV = HD = I = V = 0          # layer sizes of the chosen shape, set by main()


def _set_shape(name: str) -> dict:
    global D, H, HKV, HD, I, V
    cfg = dict(bench.SHAPES[name][1])
    D, H, HKV, HD = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    I, V = cfg["intermediate_size"], cfg["vocab_size"]
    return cfg


def _time(name, fn, repeat, nbytes=0, flops=0):
    fn(0)
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for i in range(repeat):
        fn(i + 1)
    e.record()
    torch.cuda.synchronize()
    us = s.elapsed_time(e) / repeat * 1e3
    extra = ""
    if nbytes:
        extra += f"  {nbytes / us / 1e6:6.2f} TB/s"
    if flops:
        extra += f"  {flops / us / 1e6:7.1f} TFLOP/s"
    print(f"{name:40s} {us:9.1f} us{extra}", flush=True)


def _weights(n, k, dev):
    copies = max(2, int(3e8 // (n * k * 2)))          # rotate through more than L2 holds
    return [torch.randn(n, k, device=dev).bfloat16() for _ in range(copies)]


def gemm_case(tokens, repeat, dev, kernels):
    for name, n, k, acc in (("qkv", (H + 2 * HKV) * HD, D, False), ("o", D, H * HD, True), ("gate_up", 2 * I, D, False),
                            ("down", D, I, True), ("head", V, D, False)):
        if name == "head" and tokens > 128:
            continue
        ws = _weights(n, k, dev)
        # few tokens: the engine's Linear reads the tile-by-tile copy of the weights
        tiles = [kernels.tile_weight(w) if tokens <= 128 else None for w in ws]
        a = torch.randn(tokens, k, device=dev).bfloat16()
        out = torch.zeros(tokens, n, device=dev)
        _time(f"gemm {name} [{tokens}x{k}] x [{n}x{k}]^T",
              lambda i: kernels.gemm_tc(a, ws[i % len(ws)], out, acc, w_tiles=tiles[i % len(ws)]), repeat,
              nbytes=n * k * 2, flops=2 * tokens * n * k)
    if tokens > 128:
        ws = _weights(2 * I, D, dev)
        a = torch.randn(tokens, D, device=dev).bfloat16()
        h = torch.empty(tokens, I, device=dev, dtype=torch.bfloat16)
        _time("gemm gate_up with SwiGLU epilogue", lambda i: kernels.gemm_swiglu(a, ws[i % len(ws)], h), repeat,
              flops=2 * tokens * 2 * I * D)


def attention_decode_case(batch, context, repeat, dev, kernels):
    pages_per = context // PAGE
    n_pages = batch * pages_per
    caches = [(torch.randn(n_pages, HKV, PAGE, HD, device=dev).bfloat16(), torch.randn(n_pages, HKV, PAGE, HD, device=dev).bfloat16())
              for _ in range(max(1, int(3e8 // (n_pages * HKV * PAGE * HD * 4))))]
    tables = torch.arange(n_pages, dtype=torch.int32, device=dev).view(batch, pages_per)
    pos = torch.full((batch,), context - 1, dtype=torch.int32, device=dev)
    rows = torch.arange(batch, dtype=torch.int32, device=dev)
    q = torch.randn(batch, H * HD, device=dev).bfloat16()
    out = torch.empty_like(q)
    chunk = kernels.attention_chunk_keys()
    mc = (context + chunk - 1) // chunk
    po = torch.empty(batch * H * mc * HD, device=dev)
    pml = torch.empty(batch * H * mc * 2, device=dev)

    def run(i):
        k, v = caches[i % len(caches)]
        kernels.attention_decode(q, k, v, out, rows, rows, pos, tables, H, HKV, HD, PAGE, HD ** -0.5, None, po, pml, mc, mc)

    _time(f"attention decode B={batch} context={context}", run, repeat, nbytes=batch * context * HKV * HD * 2 * 2)


def attention_prefill_case(tokens, repeat, dev, kernels):
    n_pages = (tokens + PAGE - 1) // PAGE
    kc = torch.randn(n_pages, HKV, PAGE, HD, device=dev).bfloat16()
    vc = torch.randn_like(kc)
    tables = torch.arange(n_pages, dtype=torch.int32, device=dev).view(1, n_pages)
    pos = torch.arange(tokens, dtype=torch.int32, device=dev)
    q = torch.randn(tokens, H * HD, device=dev).bfloat16()
    out = torch.empty_like(q)
    variants = [("mma.sync", kernels.attention_prefill, kernels.attention_prefill_rows(PAGE, HD))]
    if kernels.attention_prefill_tc_supported(HD, H, HKV, PAGE):
        variants.append(("tcgen05", kernels.attention_prefill_tc, 128))
    for name, fn, rows in variants:
        per = rows // (H // HKV)
        work = torch.tensor([[t, min(per, tokens - t), 0] for t in reversed(range(0, tokens, per))], dtype=torch.int32,
                            device=dev)
        _time(f"attention prefill T={tokens} ({name})",
              lambda i: fn(q, kc, vc, out, work, pos, tables, H, HKV, HD, PAGE, HD ** -0.5, None),
              repeat, flops=2 * tokens * tokens * HD * H)


def step_case(kind, shape_cfg, batch, context, tokens, layers, repeat):
    from geneinfer_b200 import Engine
    from geneinfer_b200.engine.step import StepEntry
    from geneinfer_b200.ops import kernels
    cfg = dict(shape_cfg, num_hidden_layers=layers or shape_cfg["num_hidden_layers"])
    folder = bench.model_folder(cfg)
    llm = Engine(folder, dtype="bfloat16", max_seq_len=max(context, tokens), page_size=PAGE,
                 kv_pages=batch * ((max(context, tokens) + PAGE - 1) // PAGE), max_running=batch, step_tokens=max(tokens, batch),
                 prefix_cache=False)
    eng = llm.steps
    eng.use_graphs = False                       # every kernel is launched directly, so a profiler sees each one
    if kind == "decode_step":
        keys = [f"b{i}" for i in range(batch)]
        bench.fill_cache(eng, keys, context - repeat - 2)
        ids = torch.zeros(batch, dtype=torch.int32, device="cuda:0")

        def run(i):
            logits = eng.step([StepEntry(k, [17 + i], [0]) for k in keys])
            kernels.argmax(logits, ids)
        _time(f"decode step B={batch} context={context} layers={cfg['num_hidden_layers']} (direct launches)", run, repeat)
    else:
        toks = torch.randint(0, V, (tokens,)).tolist()

        def run(i):
            eng.open("p")
            eng.step([StepEntry("p", toks, [tokens - 1])])
            eng.close("p")
        _time(f"prefill step T={tokens} layers={cfg['num_hidden_layers']}", run, repeat)


def timeline_case(shape_cfg, batch, context, layers, first, last, tokens=0):
    from geneinfer_b200.ops import library
    library.use_timeline_build()
    from geneinfer_b200 import Engine
    from geneinfer_b200.engine.step import StepEntry
    from geneinfer_b200.ops import kernels, timeline
    cfg = dict(shape_cfg, num_hidden_layers=layers or shape_cfg["num_hidden_layers"])
    folder = bench.model_folder(cfg)
    if tokens:
        batch = 1
        context = context + 10 * tokens
    llm = Engine(folder, dtype="bfloat16", max_seq_len=context, page_size=PAGE, kv_pages=batch * ((context + PAGE - 1) // PAGE),
                 max_running=batch, step_tokens=max(batch, 16, tokens), prefix_cache=False)
    eng = llm.steps
    keys = [f"b{i}" for i in range(batch)]
    bench.fill_cache(eng, keys, context - (10 * tokens if tokens else 12))
    ids = torch.zeros(batch, dtype=torch.int32, device="cuda:0")
    portion = torch.randint(0, V, (max(tokens, 1),)).tolist()

    def run(i):
        if tokens:                               # a portion of a prompt on top of the cached positions
            logits = eng.step([StepEntry(keys[0], portion, [tokens - 1])])
        else:
            logits = eng.step([StepEntry(k, [17 + i], [0]) for k in keys])
        kernels.argmax(logits, ids)
    for i in range(6):                           # the step's graph (or launch programs) are made and repeated a few times
        run(i)
    rec = timeline.Recorder(eng.device)
    run(6)
    rec.start()
    run(7)
    records = rec.records()
    found = timeline.launches(records)
    span = records[:, 3].max() / 1000 if len(records) else 0.0
    what = f"portion of {tokens} tokens after {context - 10 * tokens + 7 * tokens} cached ones" if tokens else f"decode step B={batch} context={context}"
    print(f"{what}, layers={cfg['num_hidden_layers']}: {len(records)} records of {len(found)} "
          f"launches over {span:.1f} us (the time stamps themselves cost a few per cent)")
    print(timeline.table(found, first, min(last, len(found))))


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("case", choices=["gemm_prefill", "gemm_decode", "attention_decode", "attention_prefill", "decode_step",
                                     "prefill_step", "decode_timeline", "prefill_timeline"])
    ap.add_argument("--shape", choices=sorted(bench.SHAPES), default="1b")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=0, help="layers of the step cases (0 = all of the shape)")
    ap.add_argument("--repeat", type=int, default=10)
    ap.add_argument("--from-launch", type=int, default=0, help="decode_timeline: the first launch to print")
    ap.add_argument("--to-launch", type=int, default=40, help="decode_timeline: the launch after the last one to print")
    ap.add_argument("--no-pairs", action="store_true", help="many-token products on single CTAs instead of pairs (cta_group::2)")
    a = ap.parse_args()
    if a.case in ("decode_timeline", "prefill_timeline"):              # before anything loads the ordinary library
        from geneinfer_b200.ops import library
        library.use_timeline_build()
    from geneinfer_b200.ops import kernels
    shape_cfg = _set_shape(a.shape)
    if a.no_pairs:
        kernels.PAIRED_PRODUCTS = False
    dev = torch.device("cuda:0")
    if a.case == "gemm_prefill":
        gemm_case(a.tokens, a.repeat, dev, kernels)
    elif a.case == "gemm_decode":
        gemm_case(a.batch, a.repeat, dev, kernels)
    elif a.case == "attention_decode":
        attention_decode_case(a.batch, a.context, a.repeat, dev, kernels)
    elif a.case == "attention_prefill":
        attention_prefill_case(a.tokens, a.repeat, dev, kernels)
    elif a.case == "decode_timeline":
        timeline_case(shape_cfg, a.batch, a.context, a.layers, a.from_launch, a.to_launch)
    elif a.case == "prefill_timeline":
        timeline_case(shape_cfg, 1, a.context, a.layers, a.from_launch, a.to_launch, tokens=a.tokens)
    else:
        step_case(a.case, shape_cfg, a.batch, a.context, a.tokens, a.layers, a.repeat)
    status = kernels.gemm_tc_status(dev)
    print(f"status word: {status}")
    return 0 if status == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
