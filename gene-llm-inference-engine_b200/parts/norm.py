"""Normalisation parts."""
from __future__ import annotations

from typing import Optional

import torch

from ..ops import kernels
from .registry import register_norm


@register_norm("rmsnorm")
class RMSNorm:
    """out = weight * (x / sqrt(mean(x^2) + eps)), computed in 32-bit from the 32-bit residual
    stream (src/kernels/kernels.cpp:72-83); the weight is used as is (no ``1 + w``) and is kept in
    32-bit whatever the checkpoint stores. Params: ``size``, ``eps``. Weights: ``weight`` [size]."""

    def __init__(self, params, weights, build):
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        w = weights["weight"]
        if tuple(w.shape) != (self.size,):
            raise ValueError(f"rmsnorm: weight has shape {tuple(w.shape)}, expected ({self.size},)")
        self.weight = w.to(device=build.device, dtype=torch.float32).contiguous()

    def launch_key(self, ctx):
        """Its one launch depends on the number of rows only (which the caller's key holds)."""
        return ()

    def forward(self, x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        kernels.rmsnorm(x, self.weight, out, self.eps, rows)
        return out
