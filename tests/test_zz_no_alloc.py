"""The allocation-free sampling entry point (csrc/no_alloc.h), called through its exported C
symbol, against the ordinary entry point that takes a scratch buffer from the caller.

Some embedders of the library cannot call cudaMalloc once they are running (a host that gave the
device heap to its own pool, a real-time loop, a service with an audited memory budget); for them
the library carries the sampling work area inside itself. This file is collected last on purpose:
the entry point keeps a work area for the life of the process, and a failure here must not hide
the other tests from a run that stops at the first failure.
"""
import ctypes
from ctypes import c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
MAX_FLOATS = 2 * 1024 * 1024


def _entry():
    from geneinfer_b200.ops import lib
    fn = lib().gi_sample_no_alloc
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]
    return fn


def _case(rows, vocab, seed, top_k, top_p):
    g = torch.Generator().manual_seed(seed)
    dev = "cuda:0"
    return {
        "logits": (torch.randn(rows, vocab, generator=g) * 3).to(dev),
        "temperature": torch.full((rows,), 0.9, device=dev),
        "top_k": torch.full((rows,), top_k, dtype=torch.int32, device=dev),
        "top_p": torch.full((rows,), top_p, device=dev),
        "uniform": torch.rand(rows, generator=g).to(dev),
    }


def _ordinary(c):
    from geneinfer_b200.ops import kernels
    rows, vocab = c["logits"].shape
    out = torch.full((rows,), -1, dtype=torch.int32, device="cuda:0")
    scratch = torch.empty(rows * vocab, device="cuda:0")
    kernels.sample(c["logits"], scratch, c["temperature"], c["top_k"], c["top_p"], c["uniform"], out)
    return out.cpu().tolist()


def _no_alloc(c):
    rows, vocab = c["logits"].shape
    out = torch.full((rows,), -1, dtype=torch.int32, device="cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    rc = _entry()(c["logits"].data_ptr(), rows, vocab, c["temperature"].data_ptr(), c["top_k"].data_ptr(),
                  c["top_p"].data_ptr(), c["uniform"].data_ptr(), out.data_ptr(), stream)
    return rc, out.cpu().tolist()


def test_two_calls_in_a_row_match_the_ordinary_entry_point():
    # the second call is smaller and of another shape: what the first left in the work area must not matter
    first = _case(12, 50257, seed=1, top_k=0, top_p=1.0)
    second = _case(5, 1000, seed=2, top_k=40, top_p=0.9)
    want_first, want_second = _ordinary(first), _ordinary(second)
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    rc1, got_first = _no_alloc(first)
    rc2, got_second = _no_alloc(second)
    assert rc1 == 0 and rc2 == 0
    assert got_first == want_first
    assert got_second == want_second
    assert all(0 <= t < 50257 for t in got_first) and all(0 <= t < 1000 for t in got_second)
    # the only allocations in between are this test's own small output tensors
    assert torch.cuda.memory_allocated() - before < 4096


def test_a_greedy_row_among_sampled_rows_keeps_the_callers_value():
    """Rows with temperature <= 0 are skipped by the kernel (the header says so): the id that the
    caller wrote there before the call (its argmax) is still there afterwards."""
    c = _case(6, 3000, seed=4, top_k=0, top_p=1.0)
    c["temperature"][2] = 0.0
    want = _ordinary(c)                              # the ordinary entry point leaves its -1 in row 2 as well
    assert want[2] == -1
    rc, got = _no_alloc(c)
    assert rc == 0 and got == want
    assert got[2] == -1 and all(0 <= t < 3000 for i, t in enumerate(got) if i != 2)


def test_sizes_beyond_the_work_area_are_refused_with_a_clear_error():
    from geneinfer_b200.ops import lib
    rows, vocab = 17, 128256                         # 17 x 128256 > 2 Mi floats; nothing is launched
    assert rows * vocab > MAX_FLOATS
    dummy = torch.zeros(8, device="cuda:0")
    out = torch.full((rows,), -1, dtype=torch.int32, device="cuda:0")
    rc = _entry()(dummy.data_ptr(), rows, vocab, dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
                  dummy.data_ptr(), out.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc != 0
    msg = lib().gi_last_error().decode()
    assert "exceed the built-in work area" in msg and "17 rows" in msg
    torch.cuda.synchronize()
    assert out.cpu().tolist() == [-1] * rows
    rc, got = _no_alloc(_case(16, 128256, seed=3, top_k=0, top_p=1.0))      # exactly at the limit is served
    assert rc == 0 and all(0 <= t < 128256 for t in got)
