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
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        assert noalloc_gemm(rt, a, b, got, ta, tb, alpha=0.5, beta=2.0) == 0, rt.docc_b200_last_error()
        assert torch.cuda.memory_allocated() == before
        want = c0.clone()
        ops.gemm(a, b, want, alpha=0.5, beta=2.0, transa=ta, transb=tb)
        ops.sync()
        torch.cuda.synchronize()
        assert relerr(got.cpu().numpy(), want.cpu().numpy()) <= 1e-4  # the fp32 tolerance of the other GEMM tests
        ref = 0.5 * ((a.t() if ta else a).double() @ (b.t() if tb else b).double()) + 2.0 * c0.double()
        assert relerr(got.cpu().numpy(), ref.cpu().numpy()) <= 1e-4


def test_rejects_problems_beyond_the_built_in_array(rt):
    a = torch.zeros(8, 8, device="cuda")
    # 4 * (m + n) * k bytes = 4 * 8192 * 1024 = 32 MiB > 16 MiB; rejected before any pointer is touched
    st = rt.docc_b200_gemm_f32_noalloc(NO_TRANS, NO_TRANS, 4096, 4096, 1024, 1.0, a.data_ptr(), 1024, a.data_ptr(), 4096, 0.0,
                                       a.data_ptr(), 4096, 1)
    assert st == 1
    msg = rt.docc_b200_last_error().decode()
    assert "scratch" in msg and "16777216" in msg
    assert rt.docc_b200_gemm_f32_noalloc(NO_TRANS, NO_TRANS, 4, 4, 0, 1.0, a.data_ptr(), 8, a.data_ptr(), 8, 0.0,
                                         a.data_ptr(), 8, 1) == 1
