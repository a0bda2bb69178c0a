"""Typed descriptions that every architecture is translated into.

An architecture's own configuration (its ``config.json`` keys) is turned into a ``ModelSpec``:
a list of ``LayerSpec`` (which mixer, feed-forward, norm and position encoding a layer has, with
all their sizes and constants) plus a ``schedule`` that says in which order layers run and whose
cache each run reads. Nothing below this level knows an architecture's name.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


class ConfigError(ValueError):
    """A config.json that is missing a key, has a bad value or asks for something unsupported."""


@dataclass(frozen=True)
class PartSpec:
    """One part chosen by name, with the constants it is built with."""
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)

    def __hash__(self):
        return hash((self.kind, repr(sorted(self.params.items()))))


@dataclass(frozen=True)
class LayerSpec:
    """The parts of one layer. ``block`` names the arrangement (see parts/block.py); ``extra`` holds
    further parts that an arrangement may name beyond the usual four (norms after the mixer or the
    feed-forward of a sandwich arrangement, a second feed-forward run in parallel, ...): the block
    builds them by their key, with the weights under ``layers.<i>.<key>.``."""
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec
    block: str = "pre_norm"
    extra: Dict[str, PartSpec] = field(default_factory=dict)

    def __hash__(self):
        return hash((self.mixer, self.feed_forward, self.mixer_norm, self.feed_forward_norm, self.block,
                     tuple(sorted((k, hash(v)) for k, v in self.extra.items()))))


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer. ``cache_of`` names the layer whose cache (pages or state) this run
    reads and writes; ``None`` means the layer's own. ``writes_cache`` False makes the run a
    reader only (the keys and values of the owner are used as they are)."""
    layer: int
    cache_of: Optional[int] = None
    writes_cache: bool = True


@dataclass
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_position: int
    layers: List[LayerSpec]
    schedule: List[ScheduleEntry]
    final_norm: PartSpec
    tie_word_embeddings: bool
    embedding_scale: float = 1.0   # multiplier on embedding rows (1 = none)
    logit_transform: Optional[PartSpec] = None   # applied to the logits after the head (a scale, a soft cap); None = none

    def validate(self) -> None:
        n = len(self.layers)
        if n == 0:
            raise ConfigError("a model needs at least one layer")
        for e in self.schedule:
            if not (0 <= e.layer < n):
                raise ConfigError(f"schedule names layer {e.layer}, the model has {n}")
            if e.cache_of is not None and not (0 <= e.cache_of < n):
                raise ConfigError(f"schedule entry reads the cache of layer {e.cache_of}, the model has {n}")
