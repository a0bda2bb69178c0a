"""A weight matrix with the matrix products the engine needs: ``out (+)= a @ weight^T``.

The weight is [N, K] row-major, as checkpoints store it (``y = W x``). On the 32-bit path weight
and activations are 32-bit and the product runs on the CUDA cores with fused multiply-adds. On the
bfloat16 path the weight is bfloat16 and the product runs on the tensor cores (tcgen05) with 32-bit
accumulation; the output may be 32-bit (and may accumulate into the 32-bit residual stream) or
bfloat16. A width that TMA cannot address (not a multiple of 8) falls back to the CUDA cores.

With ``tiles`` a bfloat16 weight is also kept tile by tile (``kernels.tile_weight``): products of
few tokens (decoding) stream the weights once per step and are bound by how fast an SM can fetch
them; a bulk copy of 32 KB of consecutive tiles is fetched 1.5 times faster than TMA boxes over the
row-major matrix (whose 128-byte rows lie 2 K bytes apart), with half as many barrier round trips.
Products of many tokens keep reading the row-major matrix. The copy doubles the memory of the
matrices (2.5 GB more for Llama-3.2-1B, where it buys about 5 % of decoding speed).
"""
from __future__ import annotations

import torch

from . import kernels


class Linear:
    not_weights = ("weight_tiles",)      # a second layout of the same weights, not counted among a model's weight bytes

    def __init__(self, weight: torch.Tensor, compute_dtype: torch.dtype, device: torch.device, tiles: bool = True):
        if weight.dim() != 2:
            raise ValueError("Linear: the weight must be a matrix")
        self.out_features, self.in_features = weight.shape
        self.compute_dtype = compute_dtype
        self.weight = weight.to(device=device, dtype=compute_dtype).contiguous()
        self.weight_tiles = None
        if tiles and compute_dtype is torch.bfloat16 and self.in_features % 8 == 0:
            self.weight_tiles = kernels.tile_weight(self.weight)

    @classmethod
    def sharing(cls, other: "Linear") -> "Linear":
        """A second Linear over the same device tensor (a tied head)."""
        new = cls.__new__(cls)
        new.__dict__.update(other.__dict__)
        return new

    @classmethod
    def over(cls, weight: torch.Tensor, tiles: bool = True) -> "Linear":
        """A Linear over a matrix that is on the device already (the embedding table as a tied head)."""
        new = cls.__new__(cls)
        new.out_features, new.in_features = weight.shape
        new.compute_dtype = weight.dtype
        new.weight = weight
        new.weight_tiles = None
        if tiles and weight.dtype is torch.bfloat16 and new.in_features % 8 == 0:
            new.weight_tiles = kernels.tile_weight(weight)
        return new

    def forward(self, a: torch.Tensor, out: torch.Tensor, accumulate: bool = False, then: "Linear" = None) -> torch.Tensor:
        """``then``: the Linear whose product runs next but one (after a small kernel); a product of few tokens
        asks the start of its weights into L2 meanwhile (``kernels.gemm_tc``: ``ahead``)."""
        if a.dtype != self.compute_dtype:
            raise kernels.KernelError(f"Linear: activations are {a.dtype}, the weight is {self.compute_dtype}")
        if self.compute_dtype is torch.bfloat16 and self.in_features % 8 == 0:
            kernels.gemm_tc(a, self.weight, out, accumulate, w_tiles=self.weight_tiles,   # tensor cores (TMA needs 16-byte rows)
                            ahead=then.weight_tiles if then is not None else None)
        else:
            kernels.gemm_simt(a, self.weight, out, accumulate)
        return out
