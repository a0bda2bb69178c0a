"""Per-kernel timing of one decode step, for ``gi_generate --profile``: every kernel wrapper is
timed with CUDA events around one more step of the finished request's context (the idea of the
reference's per-section report, src/gpu/gpu_transformer.cpp:178-222)."""
from __future__ import annotations

from collections import defaultdict

import torch

from ..ops import kernels


def profile_report(engine, prompt) -> str:
    from .step import StepEntry
    names = ["embed", "rmsnorm", "swiglu", "rope_store", "attention_generic", "gemm_simt", "argmax"]
    names += [n for n in ("gemm_bf16", "attention_decode", "attention_prefill") if hasattr(kernels, n)]
    records = defaultdict(list)
    saved = {n: getattr(kernels, n) for n in names}

    def timed(name, fn):
        def wrapper(*a, **k):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            out = fn(*a, **k)
            e.record()
            records[name].append((s, e))
            return out
        return wrapper

    steps = engine.steps
    n = min(len(prompt), steps.model.max_position - 1)
    steps.open("profile")
    try:
        steps.step([StepEntry("profile", list(prompt[:n]), [])])
        for name in names:
            setattr(kernels, name, timed(name, saved[name]))
        steps.step([StepEntry("profile", [int(prompt[0])], [0])])
        torch.cuda.synchronize()
    finally:
        for name in names:
            setattr(kernels, name, saved[name])
        steps.close("profile")
    total = sum(s.elapsed_time(e) for v in records.values() for s, e in v) or 1e-9
    lines = [f"[profile] one decode step at context {n}: {total:.3f} ms in kernels"]
    for name, v in sorted(records.items(), key=lambda kv: -sum(s.elapsed_time(e) for s, e in kv[1])):
        ms = sum(s.elapsed_time(e) for s, e in v)
        lines.append(f"[profile]   {name:<20} {len(v):4d} launches {ms:9.3f} ms {100 * ms / total:5.1f} %")
    return "\n".join(lines) + "\n"
