"""The allocation-free sum-of-squares entry point, called through its exported C symbol.

It exists for callers that must not allocate device memory: the memory-scaling sweeps and the
out-of-memory health checks run with the GPU (almost) full, where cudaMalloc or torch.empty would fail.
The check: on two calls in a row (different inputs, same stream) it returns what the regular entry
point -- fed with caller-allocated scratch -- returns.  The file name sorts last so a run that stops at
the first failure has already run every other test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_sumsq_noalloc_matches_regular_entry_point():
    from context_parallelism_b200 import _native as nv
    L = nv.lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    L.cpb_sumsq_noalloc.restype = ctypes.c_int
    L.cpb_sumsq_noalloc.argtypes = [ctypes.c_void_p, ctypes.c_long, ctypes.c_void_p, ctypes.c_void_p]
    L.cpb_sumsq.restype = ctypes.c_int
    L.cpb_sumsq.argtypes = [ctypes.c_void_p, ctypes.c_long, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    torch.manual_seed(0)
    # everything the two entry points need is allocated up front; the calls themselves allocate nothing
    inputs = [torch.randn(3_000_001, device=dev), torch.randn(70_003, device=dev) * 3.0]
    partial = torch.zeros(1024, dtype=torch.float32, device=dev)
    ticket = torch.zeros(1, dtype=torch.int32, device=dev)
    want = torch.zeros(1, dtype=torch.float32, device=dev)
    got = torch.zeros(1, dtype=torch.float32, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    for g in inputs:                                   # two calls in a row share the built-in scratch area
        assert L.cpb_sumsq(g.data_ptr(), g.numel(), partial.data_ptr(), ticket.data_ptr(), want.data_ptr(), stream) == 0
        rc = L.cpb_sumsq_noalloc(g.data_ptr(), g.numel(), got.data_ptr(), stream)
        assert rc == 0, L.cpb_last_error().decode()
        torch.cuda.synchronize(dev)
        ref = float((g.double() ** 2).sum())
        assert abs(float(got) - float(want)) <= 1e-5 * abs(float(want))
        assert abs(float(got) - ref) <= 1e-4 * ref
    # sizes beyond the stated maximum are rejected with a clear message and nothing is launched
    rc = L.cpb_sumsq_noalloc(inputs[0].data_ptr(), 2 ** 31, got.data_ptr(), stream)
    assert rc != 0 and b"2147483647" in L.cpb_last_error()
