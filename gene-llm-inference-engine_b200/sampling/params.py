"""Sampling parameters and the per-request random stream.

Names, defaults and rules are the reference sampler's (src/sampler/sampler.h:22-27,
src/sampler/sampler.cpp:25-52): temperature <= 0 is greedy and consumes no randomness; top_k 0 and
top_p 1 switch the filters off; the stream is splitmix64(seed) (0 becomes 1) driving xorshift64*,
of which the high 32 bits give u = (bits >> 8) / 2^24 in [0, 1).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

_MASK = (1 << 64) - 1


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.8
    top_k: int = 0
    top_p: float = 1.0
    seed: int = 1

    def __post_init__(self):
        if not (isinstance(self.temperature, (int, float)) and self.temperature >= 0.0) or math.isnan(self.temperature):
            raise ValueError("sampler: temperature must be >= 0")
        if not isinstance(self.top_k, int) or self.top_k < 0:
            raise ValueError("sampler: top_k must be >= 0")
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError("sampler: top_p must be in (0, 1]")
        if not isinstance(self.seed, int) or self.seed < 0:
            raise ValueError("sampler: seed must be a non-negative integer")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0


class RandomStream:
    """xorshift64* seeded through splitmix64; one per request, advanced once per sampled token."""

    def __init__(self, seed: int):
        x = (seed + 0x9E3779B97F4A7C15) & _MASK
        x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
        x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
        x ^= x >> 31
        self.state = x if x else 1

    def next_u32(self) -> int:
        s = self.state
        s ^= s >> 12
        s ^= (s << 25) & _MASK
        s ^= s >> 27
        self.state = s
        return ((s * 0x2545F4914F6CDD1D) & _MASK) >> 32

    def next_uniform(self) -> float:
        return (self.next_u32() >> 8) / 16777216.0
