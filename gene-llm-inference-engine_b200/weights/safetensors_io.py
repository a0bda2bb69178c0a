"""Reading and writing the safetensors container, without the safetensors package.

Format: 8-byte little-endian header length, a JSON header ``{name: {dtype, shape, data_offsets}}``
(plus an optional ``__metadata__``), then the raw little-endian data. The checks are those of the
reference reader (src/loader/safetensors.cpp:25-93): header size within the file and at most
100 MiB, entries are objects, no negative dimension, offsets inside the data region, and the
number of bytes equal to shape x dtype size.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Tuple

import torch

MAX_HEADER_BYTES = 100 * 1024 * 1024

_DTYPES = {
    "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype_name: str
    shape: Tuple[int, ...]
    begin: int   # absolute byte offsets in the file
    end: int

    @property
    def numel(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n


class SafetensorsFile:
    """A memory-mapped safetensors file; tensors are read by name."""

    def __init__(self, path: str):
        self.path = path
        if not os.path.isfile(path):
            raise SafetensorsError(f"safetensors: cannot open {path}")
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"safetensors: {path}: file is too small to contain a header")
        self._fh = open(path, "rb")
        self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        (header_size,) = struct.unpack("<Q", self._mm[:8])
        if header_size > MAX_HEADER_BYTES or header_size > size - 8:
            raise SafetensorsError(f"safetensors: {path}: header size {header_size} does not fit in the file")
        data_start = 8 + header_size
        data_len = size - data_start
        try:
            header = json.loads(self._mm[8:data_start].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"safetensors: {path}: invalid header JSON: {e}") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"safetensors: {path}: the header is not a JSON object")
        self.metadata = header.get("__metadata__")
        self.entries: Dict[str, TensorEntry] = {}
        for name, info in header.items():
            if name == "__metadata__":
                continue
            if not isinstance(info, dict):
                raise SafetensorsError(f"safetensors: {path}: entry '{name}' is not an object")
            try:
                dtype_name = info["dtype"]
                shape = info["shape"]
                offsets = info["data_offsets"]
                if not isinstance(dtype_name, str) or not isinstance(shape, list) or not isinstance(offsets, list):
                    raise TypeError("wrong field types")
                if not all(isinstance(d, int) and not isinstance(d, bool) for d in shape):
                    raise TypeError("shape must hold integers")
                if len(offsets) != 2 or not all(isinstance(o, int) and not isinstance(o, bool) for o in offsets):
                    raise TypeError("data_offsets must have 2 integers")
            except (KeyError, TypeError) as e:
                raise SafetensorsError(f"safetensors: {path}: malformed entry '{name}': {e}") from None
            if any(d < 0 for d in shape):
                raise SafetensorsError(f"safetensors: {path}: negative dimension in '{name}'")
            b, e = offsets
            if b < 0 or e < b or e > data_len:
                raise SafetensorsError(f"safetensors: {path}: data_offsets of '{name}' lie outside the data region")
            entry = TensorEntry(name, dtype_name, tuple(shape), data_start + b, data_start + e)
            if dtype_name in _DTYPES and entry.numel * _DTYPES[dtype_name][1] != e - b:
                raise SafetensorsError(
                    f"safetensors: {path}: tensor '{name}': {e - b} bytes of data do not match shape x {dtype_name}")
            self.entries[name] = entry

    def names(self) -> List[str]:
        return list(self.entries)

    def __contains__(self, name: str) -> bool:
        return name in self.entries

    def tensor(self, name: str) -> torch.Tensor:
        """The tensor in its stored dtype, as a copy that owns its memory."""
        e = self.entries[name]
        if e.dtype_name not in _DTYPES:
            raise SafetensorsError(f"safetensors: tensor '{name}' has unsupported dtype {e.dtype_name}")
        dtype, _ = _DTYPES[e.dtype_name]
        if e.numel == 0:
            return torch.empty(e.shape, dtype=dtype)
        raw = bytearray(self._mm[e.begin:e.end])   # a copy: alignment of the file does not matter
        return torch.frombuffer(raw, dtype=dtype).reshape(e.shape)

    def close(self) -> None:
        self._mm.close()
        self._fh.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class ShardedSafetensors:
    """A checkpoint in several safetensors files named by ``model.safetensors.index.json``
    (``{"weight_map": {tensor name: file name}}``): read by tensor name like a single file. The
    reference refuses such folders (src/loader/hf_checkpoint.cpp:146-151); the larger published
    checkpoints of this architecture come in this form, so they are read here. Every file the index
    names must exist and hold the tensors the index says it holds; tensors that a file holds but the
    index does not name are reported like any other unexpected tensor."""

    def __init__(self, index_path: str):
        self.path = index_path
        folder = os.path.dirname(os.path.abspath(index_path))
        try:
            with open(index_path, "r", encoding="utf-8") as f:
                index = json.load(f)
        except OSError as e:
            raise SafetensorsError(f"safetensors: cannot open {index_path}: {e}") from None
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"safetensors: {index_path}: invalid JSON: {e}") from None
        weight_map = index.get("weight_map") if isinstance(index, dict) else None
        if not isinstance(weight_map, dict) or not weight_map or not all(
                isinstance(k, str) and isinstance(v, str) for k, v in weight_map.items()):
            raise SafetensorsError(f"safetensors: {index_path}: no \"weight_map\" from tensor names to file names")
        self._files: Dict[str, SafetensorsFile] = {}
        self.entries: Dict[str, TensorEntry] = {}
        self._owner: Dict[str, SafetensorsFile] = {}
        try:
            for file_name in sorted(set(weight_map.values())):
                if os.path.basename(file_name) != file_name:
                    raise SafetensorsError(f"safetensors: {index_path}: file name '{file_name}' leaves the model folder")
                self._files[file_name] = SafetensorsFile(os.path.join(folder, file_name))
            for name, file_name in weight_map.items():
                shard = self._files[file_name]
                if name not in shard.entries:
                    raise SafetensorsError(f"safetensors: {index_path}: tensor '{name}' is not in {file_name}, where the index puts it")
                self.entries[name] = shard.entries[name]
                self._owner[name] = shard
            for file_name, shard in self._files.items():      # tensors the index does not know: reported by the loader
                for name, entry in shard.entries.items():
                    if name not in self.entries:
                        self.entries[name] = entry
                        self._owner[name] = shard
        except SafetensorsError:
            self.close()
            raise

    def names(self) -> List[str]:
        return list(self.entries)

    def __contains__(self, name: str) -> bool:
        return name in self.entries

    def tensor(self, name: str) -> torch.Tensor:
        return self._owner[name].tensor(name)

    def close(self) -> None:
        for shard in self._files.values():
            shard.close()
        self._files = {}

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]],
                      metadata: Optional[Dict[str, str]] = None) -> None:
    """Writes tensors in the given order (header padded with spaces to 8 bytes)."""
    header: Dict[str, object] = {}
    if metadata is not None:
        header["__metadata__"] = metadata
    blobs: List[bytes] = []
    offset = 0
    for name, t in tensors:
        t = t.detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"safetensors: cannot store dtype {t.dtype} ('{name}')")
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * ((8 - len(text) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for raw in blobs:
            f.write(raw)
