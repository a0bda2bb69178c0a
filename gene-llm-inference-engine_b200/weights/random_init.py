"""Random-weights mode: writes a model folder (config.json, model.safetensors) from a
configuration and a seed.

Every tensor has its own generator seeded from (seed, tensor name), so the values do not depend on
the order in which tensors are drawn or on the dtype they are stored in: values are drawn in
32-bit and rounded to bfloat16 (nearest even) only when stored so. Matrices are N(0, std); norm
weights are ``norm_mean + N(0, norm_std)``.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Any, Dict

import torch

from ..config import parse_config
from .safetensors_io import write_safetensors

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           "f32": torch.float32}


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def write_random_model(config_json: Dict[str, Any], seed: int, out_dir: str, dtype: str = "bfloat16",
                       std: float = 0.02, norm_mean: float = 1.0, norm_std: float = 0.02) -> str:
    """Writes ``out_dir/config.json`` and ``out_dir/model.safetensors``; returns ``out_dir``."""
    if dtype not in _DTYPES:
        raise ValueError(f"dtype must be one of {sorted(_DTYPES)}")
    store = _DTYPES[dtype]
    arch, cfg = parse_config(config_json)
    plan = arch.weight_plan(cfg)
    os.makedirs(out_dir, exist_ok=True)

    def tensors():
        for rule in plan.rules:
            g = torch.Generator(device="cpu")
            g.manual_seed(_tensor_seed(seed, rule.name))
            if rule.kind == "table":
                yield rule.name, torch.zeros(rule.shape, dtype=torch.int32)
                continue
            t = torch.randn(rule.shape, generator=g, dtype=torch.float32)
            if rule.kind == "vector":
                t = t.mul_(norm_std).add_(norm_mean)
            else:
                t = t.mul_(std)
            yield rule.name, t.to(store)

    out_json = dict(config_json)
    out_json.setdefault("architectures", [arch.name])
    out_json["torch_dtype"] = "bfloat16" if store is torch.bfloat16 else "float32"
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(out_json, f, indent=2)
    write_safetensors(os.path.join(out_dir, "model.safetensors"), tensors(), metadata={"format": "pt"})
    return out_dir
