"""Sampling of a step's logits rows on the device; only token ids come back to the host."""
from __future__ import annotations

from typing import List, Sequence

import torch

from ..ops import kernels
from .params import SamplingParams


class DeviceSampler:
    def __init__(self, vocab_size: int, device: torch.device):
        self.vocab_size = vocab_size
        self.device = device
        self._probs = None          # scratch [rows, vocab] for the probabilities of sampled rows
        self._rows = 0

    def _ensure(self, rows: int) -> None:
        if rows > self._rows:
            self._rows = max(rows, 2 * self._rows, 8)
            self._probs = torch.empty(self._rows * self.vocab_size, dtype=torch.float32, device=self.device)
            self._ids = torch.empty(self._rows, dtype=torch.int32, device=self.device)
            self._host = torch.empty((4, self._rows), dtype=torch.float32).pin_memory()
            self._dev = torch.empty((4, self._rows), dtype=torch.float32, device=self.device)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], uniforms: Sequence[float]) -> List[int]:
        """One token per row of ``logits`` [rows, vocab]; ``uniforms[r]`` is the row's number from
        its request's stream (ignored for greedy rows)."""
        rows = logits.shape[0]
        if rows == 0:
            return []
        self._ensure(rows)
        ids = self._ids[:rows]
        if all(p.greedy for p in params):
            kernels.argmax(logits, ids)
            return ids.cpu().tolist()
        host = self._host
        for r, (p, u) in enumerate(zip(params, uniforms)):
            host[0, r] = p.temperature if not p.greedy else 1.0
            host[1, r] = float(p.top_k)
            host[2, r] = p.top_p
            host[3, r] = u
        self._dev[:, :rows].copy_(host[:, :rows], non_blocking=True)
        temperature = self._dev[0, :rows].contiguous()
        top_k = self._dev[1, :rows].to(torch.int32)
        top_p = self._dev[2, :rows].contiguous()
        uniform = self._dev[3, :rows].contiguous()
        kernels.sample(logits, self._probs, temperature, top_k, top_p, uniform, ids)
        out = ids.cpu().tolist()
        if any(p.greedy for p in params):
            greedy = torch.empty(rows, dtype=torch.int32, device=self.device)
            kernels.argmax(logits, greedy)
            g = greedy.cpu().tolist()
            out = [g[r] if params[r].greedy else out[r] for r in range(rows)]
        return out
