"""Shared pieces of the GPU tests: model folders made in a temporary place, plain logits of the
test requests, tolerances."""
import functools
import os
import tempfile

import numpy as np
import torch

import plain_model as pm
import tiny_configs as tc

# 32-bit: both sides compute in 32-bit, only summation orders differ.
TOL_F32 = 2e-5
# bfloat16: the plain implementation rounds to bfloat16 where the engine does, but two bfloat16
# computations that round in a slightly different order (the running maximum of an online softmax
# over tiles of keys, the order of a sum) differ by a fraction of the model's own bfloat16 noise,
# which depends on how much the weights amplify it and on how many tiles a sequence has. The
# bound is therefore tied to that noise, measured per model with the measure the comparison
# itself uses (per position, max|a-b| / max(1, max|b|), worst position of all requests) as the
# distance between the rounding and the exact plain implementation. Two conditions, set from what
# the engine shows on B200 over all comparisons of the suite. The median position of a comparison
# is a stable figure (0.05 to 0.24 of the noise, the largest at the full widths of the 1B and 3B
# shapes) and is held to MEDIAN_SHARE: a slightly wrong scale or a lost low-order contribution
# shifts it before anything shows at the worst place. The worst position of a comparison is the
# maximum of about a thousand rounding patterns and moves with any change of a summation order
# (0.25 to 0.57 with 128-key tiles in the prefill attention at head size 128, up to 0.66 with
# 64-key tiles, the same arithmetic in another order), so it keeps the bound it has always had,
# MAX_SHARE of the noise. A wrong key, position or page in the sharp models moves logits by about
# their own size, an order of magnitude more than the noise.
BF16_MAX_SHARE = 0.75
BF16_MEDIAN_SHARE = 0.30


class Bound:
    """What a comparison with the plain implementation must keep: every position below ``worst``,
    the median position below ``median`` (None: not checked). ``noise`` is the model's own
    bfloat16 noise, for the message (0 in 32-bit)."""

    def __init__(self, worst: float, median=None, noise: float = 0.0):
        self.worst, self.median, self.noise = worst, median, noise

    def __float__(self) -> float:
        return self.worst


_TMP = tempfile.TemporaryDirectory(prefix="geneinfer_tests_")

CASES = {
    "a": (tc.TINY_A, tc.SHARP_A), "b": (tc.TINY_B, tc.SHARP_B),
    "a_named": (tc.TINY_A, tc.WEIGHTS_A), "b_named": (tc.TINY_B, tc.WEIGHTS_B),
    "c": (tc.TINY_C, tc.SHARP_C), "d": (tc.TINY_D, tc.SHARP_D), "w": (tc.WIDE_W, tc.SHARP_W),
    "w3": (tc.WIDE_W3, tc.SHARP_W3),
}

REQUEST_LENGTHS = {"a": [40, 75, 128, 100, 64, 33, 90], "b": [1, 5, 24, 64, 100, 200, 256],
                   "a_named": [7, 16, 33], "b_named": [1, 5, 24, 64, 100], "c": [300, 140, 512, 129, 2, 260],
                   "d": [200, 384, 131, 66, 3], "w": [150, 37], "w3": [140, 35]}


@functools.lru_cache(maxsize=None)
def model_dir(case: str) -> str:
    config, weights = CASES[case]
    return tc.make_model_dir(config, weights, os.path.join(_TMP.name, case))


@functools.lru_cache(maxsize=None)
def requests(case: str):
    vocab = CASES[case][0]["vocab_size"]
    return {f"r{i}": tc.random_tokens(n, vocab, 100 + i) for i, n in enumerate(REQUEST_LENGTHS[case])}


@functools.lru_cache(maxsize=None)
def plain_logits(case: str, dtype: str):
    """Plain logits [T, vocab] of every test request; for bfloat16 the plain implementation rounds
    weights and stored activations to bfloat16 where the engine does."""
    w, cfg = pm.load_plain(model_dir(case))
    rnd = pm.no_rounding
    if dtype == "bfloat16":
        w, rnd = pm.round_weights_bf16(w), pm.bf16_rounding
    return {rid: pm.plain_forward(w, cfg, toks, rnd).numpy() for rid, toks in requests(case).items()}


@functools.lru_cache(maxsize=None)
def bf16_noise(case: str) -> float:
    """Worst position's max|a-b| / max(1, max|b|) between the bfloat16-rounding and the exact plain implementation."""
    exact, rounded = plain_logits(case, "float32"), plain_logits(case, "bfloat16")
    per_row = [np.abs(rounded[r] - exact[r]).max(axis=-1) / np.maximum(1.0, np.abs(exact[r]).max(axis=-1)) for r in exact]
    return float(max(rows.max() for rows in per_row))


def tolerance(dtype: str, case: str, noise: float = None) -> Bound:
    """The bound of a comparison; ``noise``: the bfloat16 noise measured on the comparison's own rows
    (default: on the case's standard requests)."""
    if dtype == "float32":
        return Bound(TOL_F32)
    noise = bf16_noise(case) if noise is None else noise
    return Bound(BF16_MAX_SHARE * noise, BF16_MEDIAN_SHARE * noise, noise)


def make_engine(case: str, dtype: str, n_pages: int, max_requests: int = 4, page_size: int = 16,
                max_step_tokens: int = 512):
    from geneinfer_b200.engine.loading import load_model
    from geneinfer_b200.engine.step import StepEngine
    model = load_model(model_dir(case), dtype=dtype)
    return StepEngine(model, page_size=page_size, n_pages=n_pages, max_requests=max_requests,
                      max_step_tokens=max_step_tokens, debug_checks=True)
