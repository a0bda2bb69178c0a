"""Arrangements of the parts of one layer."""
from __future__ import annotations

import torch

from .registry import FEED_FORWARDS, MIXERS, NORMS, build_part, register_block, sub_weights


@register_block("pre_norm")
class PreNormBlock:
    """x += mixer(norm(x)); x += feed_forward(norm(x)), the residual stream x kept in 32-bit
    (src/model/transformer.cpp:379-451)."""

    def __init__(self, layer_spec, weights, build):
        self.mixer_norm = build_part(NORMS, "norm", layer_spec.mixer_norm, sub_weights(weights, "mixer_norm."), build)
        self.mixer = build_part(MIXERS, "mixer", layer_spec.mixer, sub_weights(weights, "mixer."), build)
        self.feed_forward_norm = build_part(NORMS, "norm", layer_spec.feed_forward_norm,
                                            sub_weights(weights, "feed_forward_norm."), build)
        self.feed_forward = build_part(FEED_FORWARDS, "feed-forward", layer_spec.feed_forward,
                                       sub_weights(weights, "feed_forward."), build)
        self.dtype = build.compute_dtype

    def forward(self, ctx, run, x: torch.Tensor) -> None:
        xn = ctx.scratch("normed", tuple(x.shape), self.dtype)
        self.mixer_norm.forward(x, xn)
        self.mixer.forward(ctx, run, xn, x)
        ctx.tap("attn_out", run.layer, x)
        self.feed_forward_norm.forward(x, xn)
        self.feed_forward.forward(ctx, xn, x)
        ctx.tap("ffn_out", run.layer, x)
