"""Position encodings."""
from __future__ import annotations

import math

import numpy as np
import torch

from .registry import register_position_encoding


def rope_frequencies(head_dim: int, theta: float, scaling, rotary_dim=None) -> np.ndarray:
    """Rotation frequency of each pair in double precision: 1/theta^(2k/rotary_dim), with the
    "llama3" scaling when given (src/kernels/kernels.cpp:142-163). theta is rounded to 32-bit
    first, as the reference stores it so (src/loader/hf_checkpoint.cpp:125)."""
    rd = rotary_dim or head_dim
    theta = float(np.float32(theta))
    k = np.arange(rd // 2, dtype=np.float64)
    freq = 1.0 / np.power(theta, 2.0 * k / rd)
    if scaling:
        factor = float(scaling["factor"])
        low, high = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
        original = float(scaling["original_max_position"])
        wavelength = 6.283185307179586476925 / freq
        out = freq.copy()
        slow = wavelength > original / low
        out[slow] = freq[slow] / factor
        mid = ~slow & ~(wavelength < original / high)
        smooth = (original / wavelength - low) / (high - low)
        out[mid] = ((1.0 - smooth) * freq / factor + smooth * freq)[mid]
        freq = out
    return freq


@register_position_encoding("rope")
class RotaryPosition:
    """Rotary position encoding applied to queries and keys before the key is stored. Owns the
    cos/sin table [max_position, rotary_dim/2], computed on the host in double precision and
    rounded to 32-bit once (src/kernels/kernels.cpp:159-161). Params: ``head_dim``, ``theta``,
    ``pairing`` ("half_split": pair k is (v[k], v[k+rd/2]); "interleaved": (v[2k], v[2k+1])),
    ``scaling`` (None or the four llama3 numbers), optional ``rotary_dim`` (< head_dim rotates only
    the first dims)."""

    applies = "qk_before_store"
    not_weights = ("cos", "sin")        # tables computed from constants: not counted among a model's weight bytes

    def __init__(self, params, weights, build):
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim") or self.head_dim)
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError(f"rope: rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        pairing = params.get("pairing", "half_split")
        if pairing not in ("half_split", "interleaved"):
            raise ValueError(f"rope: unknown pairing '{pairing}'")
        self.interleaved = pairing == "interleaved"
        freq = rope_frequencies(self.head_dim, params["theta"], params.get("scaling"), self.rotary_dim)
        pos = np.arange(build.max_position, dtype=np.float64)[:, None]
        angle = pos * freq[None, :]
        self.cos = torch.from_numpy(np.cos(angle).astype(np.float32)).to(build.device).contiguous()
        self.sin = torch.from_numpy(np.sin(angle).astype(np.float32)).to(build.device).contiguous()


@register_position_encoding("none")
class NoPosition:
    """No position encoding: queries and keys are stored as they are."""

    applies = "none"
    interleaved = False
    cos = None
    sin = None

    def __init__(self, params, weights, build):
        pass
