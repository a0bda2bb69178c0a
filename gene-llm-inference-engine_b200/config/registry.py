"""One registry from an architecture's name to what builds it.

``config.json``'s ``architectures[0]`` selects the entry; when that key is absent the entry whose
``model_types`` holds ``model_type`` is taken. An entry gives the typed configuration class (with
``from_json``, ``to_json`` and ``model_spec``) and the weight plan (weights/plan.py) that maps tensor
names of the checkpoint onto the parameters of the parts.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Tuple

from .base import ConfigError


@dataclass(frozen=True)
class Architecture:
    name: str                                  # e.g. "LlamaForCausalLM"
    model_types: Tuple[str, ...]               # accepted ``model_type`` values
    config_class: Any                          # has from_json(dict), to_json(), model_spec()
    weight_plan: Callable[[Any], Any]          # config -> weights.plan.WeightPlan


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture) -> None:
    _ARCHITECTURES[arch.name] = arch


def known_architectures() -> Tuple[str, ...]:
    return tuple(sorted(_ARCHITECTURES))


def resolve_architecture(config_json: Dict[str, Any]) -> Architecture:
    if not isinstance(config_json, dict):
        raise ConfigError("config.json is not a JSON object")
    names = config_json.get("architectures")
    if isinstance(names, list) and names:
        name = names[0]
        if name in _ARCHITECTURES:
            return _ARCHITECTURES[name]
        raise ConfigError(f"unknown architecture '{name}' (known: {', '.join(known_architectures())})")
    mt = config_json.get("model_type")
    for arch in _ARCHITECTURES.values():
        if mt in arch.model_types:
            return arch
    raise ConfigError(
        f"config.json names no known architecture (model_type {mt!r}; known: {', '.join(known_architectures())})")


def parse_config(config_json: Dict[str, Any]):
    """Returns (architecture entry, typed configuration)."""
    arch = resolve_architecture(config_json)
    return arch, arch.config_class.from_json(config_json)
