"""Per-operation timing of one decode step, for ``gi_generate --profile``, in the manner of the
reference's device profile (src/gpu/gpu_transformer.cpp:178-222): one line per kind of operation
with its time, its share of the step and, for matrix products, the rate at which the weights were
read. Every kernel wrapper is timed with a pair of CUDA events; the timed step runs outside CUDA
graphs (events inside a captured graph measure nothing), so the kernels do not overlap their
neighbours as they do in serving and the sum is an upper bound of the step's time.
"""
from __future__ import annotations

from collections import defaultdict

import torch

from ..ops import kernels

# wrapper in ops.kernels -> (operation as the report names it, index of its weight argument or None)
OPERATIONS = {
    "embed": ("embedding lookup", None),
    "rmsnorm": ("rmsnorm", None),
    "gemm_rope_store": ("q/k/v projections + rope + store", 1),
    "rope_store": ("rope + store", None),
    "attention_generic": ("attention", None),
    "attention_decode": ("attention", None),
    "attention_prefill": ("attention", None),
    "attention_prefill_tc": ("attention", None),
    "gemm_tc": ("matrix products (tensor cores)", 1),
    "gemm_simt": ("matrix products (32-bit)", 1),
    "gemm_swiglu": ("ffn gate+up with silu * up", 1),
    "swiglu": ("silu * up", None),
    "copy_pages": ("page copies", None),
    "argmax": ("sampling", None),
    "sample": ("sampling", None),
}


def profile_report(engine, prompt) -> str:
    """Feeds ``prompt`` (all but its last token untimed), then times one decode step at that context."""
    from ..sampling.params import SamplingParams
    from .step import StepEntry
    records = defaultdict(list)
    saved = {name: getattr(kernels, name) for name in OPERATIONS}

    def timed(name, fn):
        label, weight_arg = OPERATIONS[name]

        def wrapper(*a, **k):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            out = fn(*a, **k)
            e.record()
            w = a[weight_arg] if weight_arg is not None and len(a) > weight_arg else None
            records[label].append((s, e, w.numel() * w.element_size() if w is not None else 0))
            return out
        return wrapper

    steps = engine.steps
    n = max(1, min(len(prompt), steps.model.max_position) - 1)
    graphs, programs = steps.use_graphs, steps.use_programs
    steps.open("profile")
    try:
        if n > 1 or len(prompt) > 1:
            steps.step([StepEntry("profile", list(prompt[:n]), [])])
        steps.use_graphs = steps.use_programs = False      # every launch goes through its (timed) wrapper
        for name in OPERATIONS:
            setattr(kernels, name, timed(name, saved[name]))
        logits = steps.step([StepEntry("profile", [int(prompt[min(n, len(prompt) - 1)])], [0])])
        engine.sampler.sample(logits, [SamplingParams(0.0)], [0.0])      # the step's greedy pick belongs to it
        torch.cuda.synchronize()
    finally:
        for name in OPERATIONS:
            setattr(kernels, name, saved[name])
        steps.use_graphs, steps.use_programs = graphs, programs
        steps.close("profile")
    per = {label: (len(v), sum(s.elapsed_time(e) for s, e, _ in v), sum(b for _, _, b in v)) for label, v in records.items()}
    total = sum(ms for _, ms, _ in per.values()) or 1e-9
    lines = [f"device profile: one decode step at context {n}, "
             f"{total:.3f} ms in {sum(c for c, _, _ in per.values())} timed operations (outside CUDA graphs, nothing overlaps)",
             f"  {'operation':<36} {'calls':>5} {'ms':>9} {'share':>7} {'weights GB/s':>13}"]
    for label, (count, ms, nbytes) in sorted(per.items(), key=lambda kv: -kv[1][1]):
        rate = f"{nbytes / (ms * 1e-3) / 1e9:.1f}" if nbytes and ms > 0 else ""
        lines.append(f"  {label:<36} {count:>5} {ms:>9.3f} {100 * ms / total:>6.1f}% {rate:>13}")
    return "\n".join(lines) + "\n"
