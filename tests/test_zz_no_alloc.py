"""The allocation-free fp32 GEMM entry point (docc_b200_gemm_f32_noalloc).

It serves embedders that cannot allocate device memory while running (the application owns all
of the GPU's memory through its own allocator, or cannot afford the device-wide synchronisation
of cudaMalloc): its bf16 hi/lo planes live in a fixed 16 MiB array inside the library. The test
calls it through the C ABI twice in a row and checks both results against docc_b200_gemm, which
runs the same kernels out of a pooled workspace. This file sorts last so that a run that stops
at the first failure has already executed every other test."""
import ctypes

import numpy as np
import pytest
import torch

from conftest import relerr
from docc_b200 import _lib, ops

pytestmark = pytest.mark.gpu

NO_TRANS, TRANS = 111, 112


def noalloc_gemm(rt, a, b, c, transa=False, transb=False, alpha=1.0, beta=0.0):
    m, n = c.shape
    k = a.shape[0] if transa else a.shape[1]
    stream = torch.cuda.current_stream().cuda_stream or 1  # 0 is the legacy default stream: pass cudaStreamLegacy
    return rt.docc_b200_gemm_f32_noalloc(TRANS if transa else NO_TRANS, TRANS if transb else NO_TRANS, m, n, k, alpha,
                                         a.data_ptr(), a.shape[1], b.data_ptr(), b.shape[1], beta, c.data_ptr(), c.shape[1],
                                         stream)


def test_two_calls_in_a_row_match_the_pooled_entry_point(rt):
    torch.manual_seed(21)
    # second problem is smaller: it must not be disturbed by what the first left in the shared array
    for (m, n, k, ta, tb) in ((384, 320, 200, False, False), (130, 72, 96, True, True)):
        a = torch.randn((k, m) if ta else (m, k), device="cuda")
        b = torch.randn((n, k) if tb else (k, n), device="cuda")
        c0 = torch.randn(m, n, device="cuda")
        got = c0.clone()
        # A warm-up call first: the first call on a device loads the kernels and resolves the array's address.
        # After it, the driver's own count of free device memory (cudaMemGetInfo, which sees every cudaMalloc,
        # not only torch's allocator) must not move across a call.
        assert noalloc_gemm(rt, a, b, got.clone(), ta, tb) == 0, rt.docc_b200_last_error()
        torch.cuda.synchronize()
        before, free_before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
        assert noalloc_gemm(rt, a, b, got, ta, tb, alpha=0.5, beta=2.0) == 0, rt.docc_b200_last_error()
        assert torch.cuda.memory_allocated() == before
        assert torch.cuda.mem_get_info()[0] == free_before
        want = c0.clone()
        ops.gemm(a, b, want, alpha=0.5, beta=2.0, transa=ta, transb=tb)
        ops.sync()
        torch.cuda.synchronize()
        assert relerr(got.cpu().numpy(), want.cpu().numpy()) <= 1e-4  # the fp32 tolerance of the other GEMM tests
        ref = 0.5 * ((a.t() if ta else a).double() @ (b.t() if tb else b).double()) + 2.0 * c0.double()
        assert relerr(got.cpu().numpy(), ref.cpu().numpy()) <= 1e-4


def test_call_from_a_fresh_host_thread_needs_no_library_context(rt):
    # a new host thread has no per-thread context in the library (no stream, no workspace, no pinned status word);
    # the entry point must work from it without creating one, and without moving the free-memory count
    import threading

    torch.manual_seed(23)
    a, b = torch.randn(96, 64, device="cuda"), torch.randn(64, 80, device="cuda")
    c = torch.empty(96, 80, device="cuda")
    assert noalloc_gemm(rt, a, b, c.clone()) == 0
    torch.cuda.synchronize()
    stream = torch.cuda.current_stream().cuda_stream or 1
    out = {}

    def worker():
        torch.cuda.set_device(0)
        free_before = torch.cuda.mem_get_info()[0]
        out["status"] = rt.docc_b200_gemm_f32_noalloc(NO_TRANS, NO_TRANS, 96, 80, 64, 1.0, a.data_ptr(), 64, b.data_ptr(), 80,
                                                      0.0, c.data_ptr(), 80, stream)
        out["moved"] = free_before - torch.cuda.mem_get_info()[0]

    t = threading.Thread(target=worker)
    t.start()
    t.join()
    assert out["status"] == 0 and out["moved"] == 0
    torch.cuda.synchronize()
    assert relerr(c.cpu().numpy(), (a.double() @ b.double()).cpu().numpy()) <= 1e-4


def test_rejects_problems_beyond_the_built_in_array(rt):
    a = torch.zeros(8, 8, device="cuda")
    # 4 * (m + n) * k bytes = 4 * 8192 * 1024 = 32 MiB > 16 MiB; rejected before any pointer is touched
    st = rt.docc_b200_gemm_f32_noalloc(NO_TRANS, NO_TRANS, 4096, 4096, 1024, 1.0, a.data_ptr(), 1024, a.data_ptr(), 4096, 0.0,
                                       a.data_ptr(), 4096, 1)
    assert st == 1
    msg = rt.docc_b200_last_error().decode()
    assert "scratch" in msg and "16777216" in msg
    # extents whose size product would wrap a 64-bit integer are rejected, not mis-sized
    big = (1 << 31) - 16
    assert rt.docc_b200_gemm_f32_noalloc(NO_TRANS, NO_TRANS, big, big, big, 1.0, a.data_ptr(), big, a.data_ptr(), big, 0.0,
                                         a.data_ptr(), big, 1) == 1
    assert rt.docc_b200_gemm_f32_noalloc(NO_TRANS, NO_TRANS, 1 << 40, 4, 8, 1.0, a.data_ptr(), 8, a.data_ptr(), 8, 0.0,
                                         a.data_ptr(), 8, 1) == 1
    assert rt.docc_b200_gemm_f32_noalloc(NO_TRANS, NO_TRANS, 4, 4, 0, 1.0, a.data_ptr(), 8, a.data_ptr(), 8, 0.0,
                                         a.data_ptr(), 8, 1) == 1
