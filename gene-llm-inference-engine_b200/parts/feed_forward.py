"""Feed-forward parts."""
from __future__ import annotations

import torch

from ..ops import kernels
from ..ops.linear import Linear
from .registry import register_feed_forward


@register_feed_forward("swiglu")
class SwiGLUFeedForward:
    """x += W_down (silu(W_gate xn) * (W_up xn)) (src/model/transformer.cpp:437-450).

    Params: ``hidden_size``, ``intermediate_size``. Weights: ``w_gate_up`` [2I, hidden] (gate rows
    first, then up rows) and ``w_down`` [hidden, I]."""

    graph_safe = True      # launches depend only on the step's shape: decode steps may be captured in a CUDA graph


    def __init__(self, params, weights, build):
        self.hidden_size = int(params["hidden_size"])
        self.intermediate_size = int(params["intermediate_size"])
        I, D = self.intermediate_size, self.hidden_size
        if tuple(weights["w_gate_up"].shape) != (2 * I, D):
            raise ValueError(f"swiglu: w_gate_up has shape {tuple(weights['w_gate_up'].shape)}, expected ({2 * I}, {D})")
        if tuple(weights["w_down"].shape) != (D, I):
            raise ValueError(f"swiglu: w_down has shape {tuple(weights['w_down'].shape)}, expected ({D}, {I})")
        self.w_gate_up = Linear(weights["w_gate_up"], build.compute_dtype, build.device, tiles=build.weight_tiles)
        self.w_down = Linear(weights["w_down"], build.compute_dtype, build.device, tiles=build.weight_tiles)
        self.dtype = build.compute_dtype

    @property
    def first_product(self):
        """The Linear of the first product (a block hands it to the mixer that runs before, see AttentionMixer.forward)."""
        return self.w_gate_up

    def launch_key(self, ctx):
        """Its launches depend on the token count only (which the caller's key holds)."""
        return ()

    def forward(self, ctx, xn: torch.Tensor, x: torch.Tensor) -> None:
        T = xn.shape[0]
        h = ctx.scratch("ffn_hidden", (T, self.intermediate_size), self.dtype)
        if self.dtype is torch.bfloat16 and kernels.gemm_swiglu_supported(T, self.intermediate_size, self.hidden_size):
            kernels.gemm_swiglu(xn, self.w_gate_up.weight, h)      # activation in the product's epilogue
        else:
            gu = ctx.scratch("gate_up", (T, 2 * self.intermediate_size), torch.float32)
            self.w_gate_up.forward(xn, gu)
            kernels.swiglu(gu, h)
        self.w_down.forward(h, x, accumulate=True)
