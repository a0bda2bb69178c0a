"""Compiles the CUDA sources under ``csrc/`` into one shared library for sm_100a.

The library is built in-tree (``csrc/_build/libgeneinfer_b200.so``) with nvcc at the first call
that needs it and rebuilt when a source file or a flag changes. When the source tree cannot be
written, a per-user folder under the system's temporary directory is used instead. While nvcc
runs, a progress line is printed every few seconds so that a first call does not look hung.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from typing import List

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
LIB_NAME = "libgeneinfer_b200.so"
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


class BuildError(RuntimeError):
    pass


def sources() -> List[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise BuildError("nvcc was not found (looked at $NVCC, PATH and /usr/local/cuda/bin): "
                     "the CUDA kernels of this engine cannot be built")


def _flags(timeline: bool) -> List[str]:
    """nvcc flags; ``timeline``: the kernels also record time stamps of their phases (csrc/common.cuh: GI_TIMELINE)."""
    return NVCC_FLAGS + (["-DGI_TIMELINE"] if timeline else [])


def _digest(timeline: bool = False) -> str:
    h = hashlib.sha256()
    h.update(" ".join(_flags(timeline)).encode())
    for name in sorted(os.listdir(CSRC)):
        if name.endswith((".cu", ".cuh", ".h")):
            h.update(name.encode())
            with open(os.path.join(CSRC, name), "rb") as f:
                h.update(f.read())
    return h.hexdigest()


def _build_dir(timeline: bool = False) -> str:
    in_tree = os.path.join(CSRC, "_build", "timeline") if timeline else os.path.join(CSRC, "_build")
    try:
        os.makedirs(in_tree, exist_ok=True)
        probe = os.path.join(in_tree, f".write_probe_{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return in_tree
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"geneinfer_b200_build_{os.getuid()}" + ("_timeline" if timeline else ""))
        os.makedirs(d, exist_ok=True)
        return d


def library_path(build_if_needed: bool = True, verbose: bool = True, timeline: bool = False) -> str:
    """Path of the built library, compiling it first when missing or stale. ``timeline``: the variant whose
    kernels record time stamps (a library of its own beside the ordinary one)."""
    digest = _digest(timeline)
    in_tree = os.path.join(CSRC, "_build", "timeline") if timeline else os.path.join(CSRC, "_build")
    for d in (in_tree, os.path.join(tempfile.gettempdir(), f"geneinfer_b200_build_{os.getuid()}" + ("_timeline" if timeline else ""))):
        lib, stamp = os.path.join(d, LIB_NAME), os.path.join(d, "stamp.txt")
        if os.path.isfile(lib) and os.path.isfile(stamp):
            with open(stamp) as f:
                if f.read().strip() == digest:
                    return lib
    if not build_if_needed:
        raise BuildError("the kernel library is not built")
    return build(verbose=verbose, timeline=timeline)


def build(verbose: bool = True, timeline: bool = False) -> str:
    nvcc = _nvcc()
    out_dir = _build_dir(timeline)
    digest = _digest(timeline)
    srcs = sources()
    log = (lambda m: print(f"[geneinfer_b200 build] {m}", file=sys.stderr, flush=True)) if verbose else (lambda m: None)
    log(f"compiling {len(srcs)} CUDA files for sm_100a into {out_dir}")
    results = {}

    def compile_one(name: str) -> None:
        obj = os.path.join(out_dir, name[:-3] + ".o")
        cmd = [nvcc, *_flags(timeline), "-I", CSRC, "-c", os.path.join(CSRC, name), "-o", obj]
        p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        results[name] = (p.returncode, p.stdout, obj)

    threads = [threading.Thread(target=compile_one, args=(s,)) for s in srcs]
    t0 = time.time()
    for t in threads:
        t.start()
    last = t0
    while any(t.is_alive() for t in threads):
        for t in threads:
            t.join(timeout=0.2)
        if any(t.is_alive() for t in threads) and time.time() - last >= 5.0:
            last = time.time()
            done = sum(1 for s in srcs if s in results)
            log(f"nvcc is running: {done}/{len(srcs)} files done after {last - t0:.0f} s")
    with open(os.path.join(out_dir, "ptxas.log"), "w") as f:
        for name in srcs:
            f.write(f"==== {name}\n{results[name][1]}\n")
    failed = [n for n in srcs if results[n][0] != 0]
    if failed:
        raise BuildError("nvcc failed for " + ", ".join(failed) + ":\n" + "\n".join(results[n][1] for n in failed))
    lib = os.path.join(out_dir, LIB_NAME)
    tmp = lib + f".tmp{os.getpid()}"
    cmd = [nvcc, "-shared", "-o", tmp, *[results[n][2] for n in srcs]]
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise BuildError("linking the kernel library failed:\n" + p.stdout)
    os.replace(tmp, lib)
    with open(os.path.join(out_dir, "stamp.txt"), "w") as f:
        f.write(digest)
    log(f"built {lib} in {time.time() - t0:.0f} s")
    return lib
