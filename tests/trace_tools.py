"""Traces (lists of steps in the format bin/trace_run reads) that cut the same requests in
different ways, a runner that plays a trace through an engine in this process, and the comparison
with the plain implementation."""
from __future__ import annotations

import json
import os
import subprocess
import sys
from typing import Dict, List, Sequence, Tuple

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def round_up(n: int, unit: int = 64) -> int:
    return (n + unit - 1) // unit * unit


# ------------------------------------------------------------------------------------------ traces
def trace_whole(requests: Dict[str, List[int]]) -> List[dict]:
    """Each request alone and whole: one step, logits at every position."""
    steps = []
    for i, (rid, toks) in enumerate(requests.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}],
                      "end": [rid]})
    return steps


def trace_tail_decode(requests: Dict[str, List[int]], tail: int = 32) -> List[dict]:
    """Most of a request in one step, then its last ``tail`` tokens one by one."""
    steps, n = [], 0
    for rid, toks in requests.items():
        head = max(0, len(toks) - tail)
        if head:
            steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[:head], "want": [head - 1]}], "end": []})
            n += 1
        for p in range(head, len(toks)):
            steps.append({"step": n, "entries": [{"id": rid, "tokens": [toks[p]], "want": [0]}],
                          "end": [rid] if p == len(toks) - 1 else []})
            n += 1
    return steps


def trace_portions(requests: Dict[str, List[int]], sizes: Sequence[int] = (2, 3, 5, 8, 13, 2, 7, 21, 4, 34, 2)) -> List[dict]:
    """Portions of changing size, down to two tokens; logits at every position."""
    steps, n = [], 0
    for rid, toks in requests.items():
        p, k = 0, 0
        while p < len(toks):
            take = min(sizes[k % len(sizes)], len(toks) - p)
            k += 1
            steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[p:p + take], "want": list(range(take))}],
                          "end": [rid] if p + take == len(toks) else []})
            p += take
            n += 1
    return steps


def trace_mixed(requests: Dict[str, List[int]], seed: int, max_live: int = 4, tail: int = 32) -> List[dict]:
    """Up to ``max_live`` requests live at a time: portions of some beside single decoded tokens of
    others, some left out of a step; a request is ended as soon as it is through, so that the next
    one starts on the pages it gave back."""
    rng = np.random.default_rng(seed)
    waiting = list(requests.items())
    live: List[Tuple[str, List[int], int]] = []       # id, tokens, fed
    steps, n = [], 0
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rng.random() < 0.7):
            rid, toks = waiting.pop(0)
            live.append((rid, toks, 0))
        entries, end, nxt = [], [], []
        for rid, toks, fed in live:
            left = len(toks) - fed
            if rng.random() < 0.25 and len(live) > 1:            # left out of this step
                nxt.append((rid, toks, fed))
                continue
            if left <= tail:
                take = 1                                          # decoding
            else:
                take = int(min(left - tail, rng.choice([2, 3, 5, 9, 16, 17, 31, 40])))
            want = list(range(take)) if rng.random() < 0.7 else [take - 1]
            entries.append({"id": rid, "tokens": toks[fed:fed + take], "want": want})
            if fed + take == len(toks):
                end.append(rid)
            else:
                nxt.append((rid, toks, fed + take))
        live = nxt
        if entries:
            steps.append({"step": n, "entries": entries, "end": end})
            n += 1
    return steps


def max_tokens_of(steps: List[dict], requests: Dict[str, List[int]], unit: int = 64) -> int:
    """The most tokens live requests hold at any time, each rounded up to ``unit``."""
    held: Dict[str, int] = {}
    worst = 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        worst = max(worst, sum(round_up(v, unit) for v in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return worst


def wanted_positions(steps: List[dict]) -> Dict[int, List[Tuple[str, int]]]:
    """For every step with wanted logits: the (request, position) of each row, in file order."""
    fed: Dict[str, int] = {}
    out: Dict[int, List[Tuple[str, int]]] = {}
    for s in steps:
        rows = []
        for e in s["entries"]:
            base = fed.get(e["id"], 0)
            rows += [(e["id"], base + w) for w in e.get("want", [])]
            fed[e["id"]] = base + len(e["tokens"])
        for rid in s["end"]:
            fed.pop(rid, None)
        if rows:
            out[s["step"]] = rows
    return out


# ------------------------------------------------------------------------------------------ running
def run_in_process(engine, steps: List[dict]) -> Dict[Tuple[str, int], np.ndarray]:
    """Plays a trace through a StepEngine; returns logits by (request, position)."""
    from geneinfer_b200.engine.step import StepEntry
    where = wanted_positions(steps)
    out: Dict[Tuple[str, int], np.ndarray] = {}
    for s in steps:
        entries = []
        for e in s["entries"]:
            if e["id"] not in engine.cache.requests:
                engine.open(e["id"])
            entries.append(StepEntry(e["id"], e["tokens"], e.get("want", [])))
        logits = engine.step(entries)
        if s["step"] in where:
            rows = logits.float().cpu().numpy()
            assert rows.shape[0] == len(where[s["step"]])
            for key, row in zip(where[s["step"]], rows):
                out[key] = row.copy()
        for rid in s["end"]:
            engine.close(rid)
    return out


def run_trace_tool(model_dir: str, dtype: str, steps: List[dict], max_tokens: int, out_dir: str, vocab: int,
                   timeout: int = 600) -> Dict[Tuple[str, int], np.ndarray]:
    """Plays a trace through bin/trace_run as a child process; returns logits by (request, position)."""
    text = "".join(json.dumps(s) + "\n" for s in steps)
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens)]
    p = subprocess.run(cmd, input=text, capture_output=True, text=True, timeout=timeout)
    assert p.returncode == 0, p.stderr[-3000:]
    done = [l for l in p.stdout.splitlines() if l.startswith("done ")]
    assert [int(l.split()[1]) for l in done] == [s["step"] for s in steps]
    out: Dict[Tuple[str, int], np.ndarray] = {}
    for step, rows in wanted_positions(steps).items():
        data = np.fromfile(os.path.join(out_dir, f"{step}.f32"), dtype="<f4").reshape(len(rows), vocab)
        for key, row in zip(rows, data):
            out[key] = row
    return out


# ------------------------------------------------------------------------------------------ comparing
def rel_err(a: np.ndarray, b: np.ndarray) -> float:
    """max|a-b| / max(1, max|b|): the reference's own measure (tests/verify_forward.py:72-77)."""
    return float(np.abs(a - b).max() / max(1.0, np.abs(b).max()))


def compare(got: Dict[Tuple[str, int], np.ndarray], plain: Dict[str, np.ndarray], tol, what: str) -> float:
    """Every returned row against the plain logits of its request; names the first wrong place.
    ``tol`` is a number (no position may reach it) or a bound with ``worst``, ``median`` and
    ``noise`` (gpu_fixtures.Bound): then the median position is held to its own limit too, and the
    messages give the errors as shares of the model's bfloat16 noise. ``plain[rid]`` is [T, vocab]
    or a dictionary from position to its row."""
    limit = float(tol)
    median_limit = getattr(tol, "median", None)
    noise = getattr(tol, "noise", 0.0)
    share = (lambda e: f" = {e / noise:.2f} of the bfloat16 noise") if noise else (lambda e: "")
    errs = []
    assert got, f"{what}: no logits came back"
    for (rid, pos) in sorted(got):
        row = got[(rid, pos)]
        assert np.isfinite(row).all(), f"{what}: request {rid} position {pos}: logits are not finite"
        err = rel_err(row, plain[rid][pos])
        assert err < limit, (f"{what}: request {rid} position {pos} (first wrong place): error {err:.3e}{share(err)} "
                             f">= {limit:.1e}; page offset {pos % 16}, page {pos // 16}")
        errs.append(err)
    worst, median = max(errs), float(np.median(errs))
    if median_limit is not None:
        assert median < median_limit, (f"{what}: the median position is off by {median:.3e}{share(median)} "
                                       f">= {median_limit:.1e} (worst {worst:.3e}{share(worst)})")
    log = os.environ.get("GENEINFER_TEST_SHARES")
    if log:
        with open(log, "a") as f:
            f.write(f"{what}\t{len(errs)}\tworst {worst:.3e}\tmedian {median:.3e}\tnoise {noise:.3e}\t"
                    f"shares {worst / noise if noise else 0:.3f} {median / noise if noise else 0:.3f}\n")
    return worst
