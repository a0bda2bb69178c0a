"""Sampling of a step's logits rows on the device; only token ids come back to the host.

The ids are written to a device buffer that the caller may name (the step engine's feedback buffer,
from which the next step can read its tokens without waiting for the host) and copied to pinned host
memory behind the kernels; ``PendingSample.result()`` waits for that copy.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..ops import kernels
from .params import SamplingParams

_RING = 4          # samples that may be in flight before the oldest must have been read


class PendingSample:
    """The token ids of one sampling call, on their way to the host."""

    def __init__(self, host: torch.Tensor, rows: int, event, status: Optional[torch.Tensor] = None, on_failure=None):
        """``status``: the host copy [1] of the kernels' status word, taken behind the ids; a value
        other than 0 says that a kernel of the steps before gave up a bounded wait, so the ids are
        not to be trusted. ``on_failure`` is called (to clear the device's word) before the error."""
        self._host, self._rows, self._event, self._status, self._on_failure = host, rows, event, status, on_failure

    def result(self) -> List[int]:
        self._event.synchronize()
        if self._status is not None and int(self._status[0]) != 0:
            code = int(self._status[0])
            self._status[0] = 0
            if self._on_failure is not None:
                self._on_failure()
            raise kernels.KernelError(f"a kernel gave up a bounded wait (status {code:#x}): the sampled tokens are not valid")
        return self._host[:self._rows].tolist()


class DeviceSampler:
    def __init__(self, vocab_size: int, device: torch.device, ids: Optional[torch.Tensor] = None):
        """``ids``: the device buffer (int32) that receives the sampled ids, row r at place r."""
        self.vocab_size = vocab_size
        self.device = device
        self._ids = ids
        self._probs = None          # scratch [rows, vocab] for the probabilities of sampled rows
        self._rows = 0
        self._slot = 0

    def _ensure(self, rows: int) -> None:
        if self._ids is None or self._ids.numel() < rows:
            self._ids = torch.empty(max(rows, 8), dtype=torch.int32, device=self.device)
        if rows > self._rows:
            self._rows = max(rows, 2 * self._rows, 8, self._ids.numel())
            self._host_ids = [torch.empty(self._rows, dtype=torch.int32).pin_memory() for _ in range(_RING)]
            self._host_status = [torch.zeros(1, dtype=torch.int32).pin_memory() for _ in range(_RING)]
            self._host = [torch.empty((4, self._rows), dtype=torch.float32).pin_memory() for _ in range(_RING)]
            self._dev = torch.empty((4, self._rows), dtype=torch.float32, device=self.device)
            self._top_k = torch.empty(self._rows, dtype=torch.int32, device=self.device)
            self._events = [None] * _RING

    def sample_async(self, logits: torch.Tensor, params: Sequence[SamplingParams],
                     uniforms: Sequence[float]) -> PendingSample:
        """One token per row of ``logits`` [rows, vocab]; ``uniforms[r]`` is the row's number from
        its request's stream (ignored for greedy rows). Returns at once."""
        rows = logits.shape[0]
        self._ensure(rows)
        slot = self._slot
        self._slot = (slot + 1) % _RING
        if self._events[slot] is not None:
            self._events[slot].synchronize()       # the slot's host buffers are free again
        ids = self._ids[:rows]
        greedy = [p.greedy for p in params]
        if any(greedy) or rows == 0:
            kernels.argmax(logits, ids)
        if not all(greedy):
            host = self._host[slot]
            for r, (p, u) in enumerate(zip(params, uniforms)):
                host[0, r] = p.temperature           # <= 0: the kernel leaves the row's argmax in place
                host[1, r] = float(p.top_k)
                host[2, r] = p.top_p
                host[3, r] = u
            self._dev[:, :rows].copy_(host[:, :rows], non_blocking=True)
            top_k = self._top_k[:rows]
            top_k.copy_(self._dev[1, :rows])
            if self._probs is None or self._probs.numel() < rows * self.vocab_size:
                self._probs = torch.empty(max(rows, 8) * self.vocab_size, dtype=torch.float32, device=self.device)
            kernels.sample(logits, self._probs, self._dev[0, :rows], top_k, self._dev[2, :rows], self._dev[3, :rows], ids)
        host_ids = self._host_ids[slot]
        host_ids[:rows].copy_(ids, non_blocking=True)
        word = kernels.status_word(self.device)
        status = self._host_status[slot]
        status.copy_(word, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        self._events[slot] = event
        return PendingSample(host_ids, rows, event, status, word.zero_)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], uniforms: Sequence[float]) -> List[int]:
        if logits.shape[0] == 0:
            return []
        return self.sample_async(logits, params, uniforms).result()
