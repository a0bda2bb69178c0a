"""A step's timeline from time stamps that the kernels take themselves.

Built with ``-DGI_TIMELINE`` (``library.use_timeline_build()``, a library of its own beside the ordinary one), the
kernels of a step record (kernel, event, block, %globaltimer) at a few places: a block enters, its wait for the
kernel ahead is over, its first operands have arrived, its last MMA is issued, the accumulator is complete, (the first block of a cluster:) the
other blocks' partial tiles have arrived, the sums are complete, its results are stored, it leaves. This shows what no per-kernel profile shows: how the kernels of a step overlap (programmatic
dependent launch lets a block enter, and fetch weights, long before it may read what the kernel ahead writes), what
the hand-over from one kernel to the next costs, and which blocks of a kernel are late. 32 ns resolution on a B200.
"""
from __future__ import annotations

from typing import Dict, List

import numpy as np
import torch

from .library import lib

KERNELS = {1: "rmsnorm", 2: "swiglu", 3: "attention_decode", 4: "add ranges", 5: "rope_store", 6: "attention_prefill",
           101: "product qkv+rope", 102: "product add", 103: "product store",
           111: "product qkv+rope (general)", 112: "product add (general)", 113: "product store (general)",
           200: "products store", 201: "products store (pairs)", 202: "products add", 203: "products add (pairs)",
           204: "products swiglu", 205: "products swiglu (pairs)", 206: "products rope", 207: "products rope (pairs)"}
EVENTS = {"rmsnorm": {0: "enter", 1: "waited", 6: "leave"}, "swiglu": {0: "enter", 1: "waited", 6: "leave"},
          "attention_decode": {0: "enter", 1: "waited", 2: "queries loaded", 3: "first tile done", 4: "last tile done", 6: "leave"},
          "add ranges": {0: "enter", 1: "waited", 6: "leave"}, "rope_store": {0: "enter", 1: "waited"},
          "attention_prefill": {0: "enter", 1: "waited", 6: "leave"},
          "product": {0: "enter", 1: "waited", 2: "first operands", 3: "last MMA issued", 4: "accumulator ready",
                      7: "partial tiles arrived", 8: "sums complete", 5: "results stored", 6: "leave"},
          "products": {0: "enter", 1: "waited", 2: "first operands", 3: "last MMA issued", 4: "first accumulator ready",
                       5: "results stored", 6: "leave"}}


class Recorder:
    """Holds the device buffer the kernels record into: ``start()`` empties it, ``records()`` reads it."""

    def __init__(self, device: torch.device, capacity: int = 1 << 19):
        self.buffer = torch.zeros(2 + 2 * capacity, dtype=torch.int64, device=device)
        self.buffer[1] = capacity
        for setter in ("gi_timeline_set_gemm", "gi_timeline_set_elementwise", "gi_timeline_set_attention",
                       "gi_timeline_set_attention_tc"):
            code = getattr(lib(), setter)(self.buffer.data_ptr())
            if code == 2:
                raise RuntimeError("this library was built without time stamps: call library.use_timeline_build() first")
            if code != 0:
                raise RuntimeError(f"{setter} failed")

    def start(self) -> None:
        torch.cuda.synchronize(self.buffer.device)
        self.buffer[0] = 0
        torch.cuda.synchronize(self.buffer.device)

    def records(self) -> np.ndarray:
        """[n, 4] int64: kernel id, event, block, time in ns since the first record."""
        torch.cuda.synchronize(self.buffer.device)
        n = min(int(self.buffer[0].item()), int(self.buffer[1].item()))
        raw = self.buffer[2:2 + 2 * n].cpu().numpy().reshape(n, 2)
        meta, t = raw[:, 0], raw[:, 1]
        out = np.stack([meta >> 40, (meta >> 32) & 0xff, meta & 0xffffffff, t - (t.min() if n else 0)], axis=1)
        return out[np.argsort(out[:, 3], kind="stable")]


def launches(records: np.ndarray) -> List[Dict]:
    """Groups time-ordered records into launches: a kernel's launch ends where one of its blocks enters a second
    time. Each launch: {"kernel": id, "blocks": {block: {event: ns}}} (for event 6 the last warp's stamp)."""
    out: List[Dict] = []
    current: Dict[int, Dict] = {}
    for kernel, event, block, t in records.tolist():
        launch = current.get(kernel)
        if event == 0:
            if launch is None or block in launch["blocks"]:
                launch = {"kernel": kernel, "blocks": {}}
                current[kernel] = launch
                out.append(launch)
            launch["blocks"][block] = {0: t}
        elif launch is not None and block in launch["blocks"]:
            events = launch["blocks"][block]
            events[event] = max(t, events.get(event, 0)) if event == 6 else events.get(event, t)
    return out


def table(all_launches: List[Dict], first: int, last: int) -> str:
    """One line per launch ``first <= n < last``: for each event the earliest and the latest block, in microseconds."""
    lines = []
    for n, launch in enumerate(all_launches[first:last], first):
        name = KERNELS.get(launch["kernel"], str(launch["kernel"]))
        events = EVENTS["products" if name.startswith("products") else "product" if name.startswith("product") else name]
        cells = []
        for event, label in events.items():
            stamps = [b[event] / 1000 for b in launch["blocks"].values() if event in b]
            if stamps:
                cells.append(f"{label} {min(stamps):.2f}..{max(stamps):.2f}")
        lines.append(f"{n:4d} {name:24s} {len(launch['blocks']):4d} blocks | " + " | ".join(cells))
    return "\n".join(lines)
