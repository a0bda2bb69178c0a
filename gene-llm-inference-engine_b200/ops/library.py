"""Loads the kernel library and declares the C signatures of its entry points.

There is no CPU fallback: if the library cannot be built or loaded, or no CUDA device is present,
``lib()`` raises and nothing of the product path runs.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_longlong, c_void_p
from typing import Optional

from .build import library_path

_lib: Optional[ctypes.CDLL] = None


class KernelError(RuntimeError):
    """A kernel entry point refused its arguments or a launch failed."""


_SIGNATURES = {
    "gi_embed": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p],
    "gi_rmsnorm": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p],
    "gi_swiglu": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "gi_rope_store": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                      c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "gi_copy_pages": [c_void_p, c_longlong, c_int, c_longlong, c_void_p, c_void_p, c_int, c_void_p],
    "gi_attention_generic": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                             c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
    "gi_gemm_simt": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                     c_int, c_void_p],
    "gi_gemm_tc": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong,
                   c_int, c_int, c_int, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_longlong,
                   c_void_p],
    "gi_gemm_tc_persistent": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong,
                              c_int, c_void_p, c_int, c_void_p, c_longlong, c_int, c_void_p],
    "gi_gemm_tc_persistent_rope": [c_void_p, c_void_p, c_int, c_int, c_longlong, c_longlong, c_void_p, c_void_p, c_void_p,
                                   c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                   c_int, c_int, c_int, c_void_p, c_int, c_void_p],
    "gi_gemm_tc_rope": [c_void_p, c_void_p, c_int, c_int, c_longlong, c_longlong, c_int, c_int, c_void_p, c_longlong,
                        c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                        c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "gi_gemm_tc_status": [c_void_p, c_void_p, c_void_p],
    "gi_attention_decode": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                            c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_int, c_int, c_longlong,
                            c_void_p, c_void_p],
    "gi_attention_prefill": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                             c_int, c_int, c_int, c_float, c_int, c_longlong, c_void_p, c_void_p],
    "gi_attention_prefill_rows": [c_int, c_int],
    "gi_gemm_tc_set_cluster": [c_int],
    "gi_gemm_tc_set_stream_weights": [c_int],
    "gi_gemm_tc_set_specialised": [c_int],
    "gi_timeline_set_gemm": [c_void_p], "gi_timeline_set_elementwise": [c_void_p], "gi_timeline_set_attention": [c_void_p],
    "gi_timeline_set_attention_tc": [c_void_p],
    "gi_attention_set_stream_kv": [c_int],
    "gi_gemm_tc_cluster_capacity": [c_int, c_int, c_int],
    "gi_attention_prefill_tc": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                                c_int, c_int, c_int, c_float, c_int, c_longlong, c_void_p, c_void_p],
    "gi_attention_prefill_tc_supported": [c_int, c_int, c_int, c_int],
    "gi_attention_fast_supported": [c_int, c_int, c_int],
    "gi_attention_generic_supported": [c_int],
    "gi_attention_chunk_keys": [],
    "gi_program_begin": [],
    "gi_program_size": [c_void_p],
    "gi_program_run": [c_void_p, c_void_p],
    "gi_program_free": [c_void_p],
    "gi_argmax": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
    "gi_sample": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
}


_timeline_build = False


def use_timeline_build() -> None:
    """Makes this process load the library variant whose kernels record time stamps of their phases
    (``ops/timeline.py``); to be called before the first kernel call."""
    global _timeline_build
    if _lib is not None and not _timeline_build:
        raise RuntimeError("the kernel library is loaded already: ask for the timeline build before the first kernel call")
    _timeline_build = True


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = library_path(timeline=_timeline_build)
        loaded = ctypes.CDLL(path)
        loaded.gi_last_error.restype = c_char_p
        loaded.gi_last_error.argtypes = []
        loaded.gi_program_end.restype = c_void_p
        loaded.gi_program_end.argtypes = []
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(loaded, name, None)
            if fn is None:
                continue            # optional entry points are declared by the modules that use them
            fn.restype = c_int
            fn.argtypes = argtypes
        _lib = loaded
    return _lib


def declare(name: str, argtypes) -> None:
    """Declares the signature of a further entry point (used by modules with kernels of their own)."""
    _SIGNATURES[name] = list(argtypes)
    if _lib is not None:
        fn = getattr(_lib, name)
        fn.restype = c_int
        fn.argtypes = list(argtypes)


def check(code: int, what: str) -> None:
    if code != 0:
        msg = lib().gi_last_error().decode("utf-8", "replace")
        raise KernelError(f"{what}: {msg}")
