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
        T = x.shape[0]
        # each half of the layer is one launch program when its parts say what their launches depend on
        # (``launch_key``); a part without that method (one that computes with other libraries) runs as it is
        key = _launch_key(ctx, (self.mixer_norm, None), (self.mixer, run))
        if key is not None:
            ctx.recorded(self, ("mixer", run, T) + key, lambda: self._mixer_half(ctx, run, xn, x))
        else:
            self._mixer_half(ctx, run, xn, x)
        ctx.tap("attn_out", run.layer, x)
        key = _launch_key(ctx, (self.feed_forward_norm, None), (self.feed_forward, None))
        if key is not None:
            ctx.recorded(self, ("feed_forward", T) + key, lambda: self._feed_forward_half(ctx, xn, x))
        else:
            self._feed_forward_half(ctx, xn, x)
        ctx.tap("ffn_out", run.layer, x)

    def _mixer_half(self, ctx, run, xn, x) -> None:
        self.mixer_norm.forward(x, xn)
        then = getattr(self.feed_forward, "first_product", None)
        if then is not None and getattr(self.mixer, "takes_then", False):
            self.mixer.forward(ctx, run, xn, x, then=then)      # the mixer's last product asks for the weights that follow
        else:
            self.mixer.forward(ctx, run, xn, x)

    def _feed_forward_half(self, ctx, xn, x) -> None:
        self.feed_forward_norm.forward(x, xn)
        self.feed_forward.forward(ctx, xn, x)


def build_extra(layer_spec, key: str, table, what: str, weights, build):
    """Builds the part that a layer's ``extra`` names ``key`` (for arrangements with more parts than
    the usual four), with the weights under ``<key>.``."""
    if key not in layer_spec.extra:
        raise KeyError(f"block arrangement '{layer_spec.block}' needs a part '{key}' that the layer's specification lacks")
    return build_part(table, what, layer_spec.extra[key], sub_weights(weights, key + "."), build)


def _launch_key(ctx, *parts):
    """The joint key of some parts' launches for this step, or None when one of them has none (or the
    context records nothing)."""
    if not hasattr(ctx, "recorded"):
        return None
    key = ()
    for part, run in parts:
        fn = getattr(part, "launch_key", None)
        if fn is None:
            return None
        k = fn(ctx) if run is None else fn(ctx, run)
        if k is None:
            return None
        key += tuple(k)
    return key
