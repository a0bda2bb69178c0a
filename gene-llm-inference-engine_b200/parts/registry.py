"""Registries of parts: a name in a ``PartSpec`` selects the class that is built.

A part class is constructed as ``cls(params: dict, weights: dict, build: BuildContext)`` where
``params`` are the constants of its ``PartSpec``, ``weights`` the tensors whose names start with
the part's path (path stripped) and ``build`` gives device, compute dtype and limits. New parts
are added with the ``register_*`` functions; nothing else in the framework changes.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict

import torch

MIXERS: Dict[str, Callable] = {}
FEED_FORWARDS: Dict[str, Callable] = {}
NORMS: Dict[str, Callable] = {}
POSITION_ENCODINGS: Dict[str, Callable] = {}
BLOCKS: Dict[str, Callable] = {}
LOGIT_TRANSFORMS: Dict[str, Callable] = {}     # what an architecture does to its logits after the head; none is built in


@dataclass
class BuildContext:
    device: torch.device
    compute_dtype: torch.dtype       # torch.float32 (true 32-bit path) or torch.bfloat16
    max_position: int                # context length the engine is built for
    weight_tiles: bool = True        # bfloat16: keep a second, tile-by-tile copy of each matrix for few-token products


def _register(table: Dict[str, Callable], kind: str):
    def deco(cls):
        table[kind] = cls
        return cls
    return deco


def register_mixer(kind: str):
    return _register(MIXERS, kind)


def register_feed_forward(kind: str):
    return _register(FEED_FORWARDS, kind)


def register_norm(kind: str):
    return _register(NORMS, kind)


def register_position_encoding(kind: str):
    return _register(POSITION_ENCODINGS, kind)


def register_block(kind: str):
    return _register(BLOCKS, kind)


def register_logit_transform(kind: str):
    return _register(LOGIT_TRANSFORMS, kind)


def build_part(table: Dict[str, Callable], what: str, spec, weights, build: BuildContext):
    if spec.kind not in table:
        raise KeyError(f"unknown {what} '{spec.kind}' (known: {', '.join(sorted(table))})")
    return table[spec.kind](dict(spec.params), weights, build)


def sub_weights(weights: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}
