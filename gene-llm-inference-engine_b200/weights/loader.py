"""Loading a model folder: config.json through the registry, model.safetensors (or the files that
model.safetensors.index.json names) by tensor name.

Tensors keep the precision they are stored in: bfloat16 stays bfloat16 and 32-bit floats stay
32-bit; float16 is widened to 32-bit (exact); integer tables become int32. One ``WeightsError``
lists every missing tensor, every unexpected one and every wrong shape or dtype at once.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Tuple

import torch

from ..config import ConfigError, parse_config
from .plan import WeightPlan
from .safetensors_io import SafetensorsError, SafetensorsFile, ShardedSafetensors

_FLOATS = {"F32", "F16", "BF16"}
_INTS = {"I64", "I32", "I16", "I8", "U8"}


class WeightsError(ValueError):
    """The checkpoint does not hold what the configuration asks for."""

    def __init__(self, path: str, missing, unexpected, wrong):
        self.missing, self.unexpected, self.wrong = list(missing), list(unexpected), list(wrong)
        lines = [f"weights: {path} does not match the configuration:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong:
            lines.append(f"  wrong shape or dtype ({len(self.wrong)}): " + "; ".join(self.wrong))
        super().__init__("\n".join(lines))


def read_config(model_dir: str):
    """Returns (architecture entry, typed configuration, raw dict) of a model folder."""
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in {model_dir}")
    try:
        with open(path, "r", encoding="utf-8") as f:
            raw = json.load(f)
    except (UnicodeDecodeError, json.JSONDecodeError) as e:
        raise ConfigError(f"config.json: {e}") from None
    arch, cfg = parse_config(raw)
    return arch, cfg, raw


def read_tensors(path: str, plan: WeightPlan) -> Dict[str, torch.Tensor]:
    """Reads every tensor the plan names; raises one WeightsError for all mismatches."""
    st = ShardedSafetensors(path) if path.endswith(".index.json") else SafetensorsFile(path)
    try:
        missing, wrong = [], []
        wanted = {r.name for r in plan.rules}
        unexpected = [n for n in st.names() if n not in wanted and not plan.is_ignorable(n)]
        for r in plan.rules:
            e = st.entries.get(r.name)
            if e is None:
                missing.append(r.name)
                continue
            if tuple(e.shape) != tuple(r.shape):
                wrong.append(f"'{r.name}' has shape {list(e.shape)}, expected {list(r.shape)}")
            elif r.kind == "table" and e.dtype_name not in _INTS:
                wrong.append(f"'{r.name}' has dtype {e.dtype_name}, expected an integer type")
            elif r.kind != "table" and e.dtype_name not in _FLOATS:
                wrong.append(f"'{r.name}' has unsupported dtype {e.dtype_name} (supported: F32, F16, BF16)")
        if missing or unexpected or wrong:
            raise WeightsError(path, missing, unexpected, wrong)
        out: Dict[str, torch.Tensor] = {}
        for r in plan.rules:
            t = st.tensor(r.name)
            if r.kind == "table":
                t = t.to(torch.int32)
            elif t.dtype == torch.float16:
                t = t.float()
            out[r.name] = t
        return out
    finally:
        st.close()


def load_model_folder(model_dir: str) -> Tuple[object, object, Dict[str, torch.Tensor]]:
    """Returns (architecture entry, typed configuration, parameters by part path), on the host."""
    arch, cfg, _ = read_config(model_dir)
    weights_path = os.path.join(model_dir, "model.safetensors")
    if not os.path.isfile(weights_path):
        weights_path = os.path.join(model_dir, "model.safetensors.index.json")     # a checkpoint in several files
        if not os.path.isfile(weights_path):
            raise SafetensorsError(f"no model.safetensors (nor model.safetensors.index.json) in {model_dir}")
    plan = arch.weight_plan(cfg)
    tensors = read_tensors(weights_path, plan)
    return arch, cfg, plan.assemble(tensors)
