"""From a model folder to a model on the device."""
from __future__ import annotations

from typing import Optional

import torch

from ..parts import DecoderModel
from ..weights import load_model_folder

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           "f32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.float32, torch.bfloat16):
            raise ValueError("dtype must be float32 or bfloat16")
        return name
    try:
        return _DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"unknown dtype '{name}' (bfloat16 or float32)") from None


def load_model(model_dir: str, dtype="bfloat16", device="cuda:0", max_position: Optional[int] = None,
               weight_tiles: bool = True) -> DecoderModel:
    """Reads config.json (the registry picks the architecture) and model.safetensors, and builds
    the model on the device. ``dtype`` float32 runs everything in true 32-bit; bfloat16 weights of
    the file are then widened exactly. ``max_position`` may lower the context length.
    ``weight_tiles`` (bfloat16 only): keep a second, tile-by-tile copy of each matrix, from which
    decode steps stream the weights faster (it doubles the memory of the matrices)."""
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device: this engine runs on the GPU only")
    arch, cfg, params = load_model_folder(model_dir)
    model = DecoderModel(cfg.model_spec(), params, parse_dtype(dtype), torch.device(device), max_position, weight_tiles)
    model.config = cfg
    return model
