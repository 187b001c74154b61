"""Generic element-wise maps: the sm_100a kernels and launches the B200 map dispatcher writes (b200_map_emit.h).

CPU tests: the emitted text against the golden file, and that nvcc compiles it for sm_100a and links it against the
runtime library. GPU tests: the compiled kernels against the same loop bodies run as sequential C loops on the host,
bit for bit, over sizes that exercise the vector form, the scalar tail and the scalar fallback for misaligned operands."""
import ctypes
import os
import shutil
import subprocess

import numpy as np
import pytest

from conftest import ROOT
from docc_b200 import build

PLUGIN = os.path.join(ROOT, "docc_b200", "plugin")
GOLDEN = os.path.join(ROOT, "tests", "golden", "emitted_maps.cu")
NVCC = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


@pytest.fixture(scope="module")
def map_driver(tmp_path_factory):
    exe = str(tmp_path_factory.mktemp("map_emit") / "map_emit_driver")
    subprocess.run(["g++", "-std=c++17", "-I" + PLUGIN, os.path.join(ROOT, "tests", "map_emit_driver.cpp"), "-o", exe], check=True)
    return exe


@pytest.fixture(scope="module")
def map_libs(map_driver, tmp_path_factory):
    """(CUDA library built from the emitted text, host library built from the same loop bodies)."""
    d = tmp_path_factory.mktemp("map_libs")
    cu = d / "maps.cu"
    cu.write_text(subprocess.run([map_driver], check=True, capture_output=True, text=True).stdout)
    gpu_lib = str(d / "libmaps.so")
    subprocess.run([NVCC, "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-Xcompiler", "-fPIC", "-shared",
                    "-I" + os.path.join(ROOT, "include"), str(cu), "-o", gpu_lib, "-L" + build.LIB_DIR, "-Xlinker", "-rpath," + build.LIB_DIR, "-ldocc_b200_rt"], check=True)
    cpp = d / "maps_cpu.cpp"
    cpp.write_text(subprocess.run([map_driver, "cpu"], check=True, capture_output=True, text=True).stdout)
    cpu_lib = str(d / "libmaps_cpu.so")
    # no contraction on the host: the loop bodies hold their fused operations explicitly (fmaf)
    subprocess.run(["g++", "-O2", "-ffp-contract=off", "-shared", "-fPIC", str(cpp), "-o", cpu_lib], check=True)
    return gpu_lib, cpu_lib


def test_emitted_map_kernels_match_golden_text(map_driver):
    out = subprocess.run([map_driver], check=True, capture_output=True, text=True).stdout
    assert out == open(GOLDEN).read()


def test_emitted_map_kernels_have_the_b200_shape(map_driver):
    text = subprocess.run([map_driver], check=True, capture_output=True, text=True).stdout
    # vector width from the widest operand: 4 x fp32, 2 x (fp32 -> fp64), 8 x 16-bit
    assert "kernel_axpby_3<4><<<" in text and "kernel_widen_7<2><<<" in text and "kernel_sumdiff_9<8><<<" in text
    # scalar fallback, grid-stride walk, launch on the runtime's stream, grid bounded by the SM count
    for needle in ("kernel_axpby_3<1><<<", "__g += __stride", "docc_b200_get_stream", "cudaDevAttrMultiProcessorCount", "__launch_bounds__(256)"):
        assert needle in text
    # a body in docc's own form (container[indvar]) is wrapped, not rewritten: the names are bound to the thread's vectors
    assert "float* const __daisy_cuda_acc = __daisy_cuda_acc_out.v;" in text and "const int i = __e;" in text
    # an in-place map loads the vector it updates
    assert "__daisy_cuda_acc_out = *reinterpret_cast<const docc_b200_vec<float, V>*>(__daisy_cuda_acc_ptr + __g * V);" in text
    # kernel and launcher share a translation unit; the generated host code only sees the launcher
    assert 'extern "C" void kernel_scale_12_launch(const float* __daisy_cuda_w_ptr, float* __daisy_cuda_acc_ptr, float lr, int N)' in text
    # the widening map checks each operand for its own access width: 8 bytes of fp32, 16 bytes of fp64
    assert "(x_ptr) % 8 == 0" in text and "(y_ptr) % 16 == 0" in text


def test_emitted_map_kernels_compile_for_sm100a_and_link(map_libs):
    gpu_lib, cpu_lib = map_libs
    assert os.path.getsize(gpu_lib) > 0
    host = ctypes.CDLL(cpu_lib)
    for fn in ("axpby_op", "widen_op", "sumdiff_op", "scale_op"):
        assert hasattr(host, fn)
    # the host loops are the checker of the GPU tests: pin them against numpy here
    rng = np.random.RandomState(0)
    a, b = rng.randn(1001).astype(np.float32), rng.randn(1001).astype(np.float32)
    out = np.empty_like(a)
    vp = ctypes.c_void_p
    host.axpby_op(vp(a.ctypes.data), vp(b.ctypes.data), vp(out.ctypes.data), ctypes.c_float(0.75), ctypes.c_longlong(a.size))
    want = (np.float64(np.float32(0.75)) * a.astype(np.float64) + b.astype(np.float64)).astype(np.float32)  # one rounding, like fmaf
    assert np.array_equal(out, want)
    p, q = rng.randint(0, 65536, 999).astype(np.uint16), rng.randint(0, 65536, 999).astype(np.uint16)
    s, d = np.empty_like(p), np.empty_like(p)
    host.sumdiff_op(vp(p.ctypes.data), vp(q.ctypes.data), vp(s.ctypes.data), vp(d.ctypes.data), ctypes.c_longlong(p.size))
    assert np.array_equal(s, p + q) and np.array_equal(d, p - q)


SIZES = [0, 1, 3, 7, 8, 255, 256, 1000, 4099, 65536, 1 << 20, (1 << 22) + 5, 50_000_003]


@pytest.mark.gpu
@pytest.mark.parametrize("offset", [0, 1, 3])
def test_map_kernels_match_the_host_loops_bit_for_bit(rt, map_libs, offset):
    """offset > 0 shifts every operand off its vector alignment, so the launch takes the scalar form."""
    import torch

    gpu = ctypes.CDLL(map_libs[0], mode=ctypes.RTLD_GLOBAL)
    host = ctypes.CDLL(map_libs[1])
    vp, ll = ctypes.c_void_p, ctypes.c_longlong
    rng = np.random.RandomState(11 + offset)
    for n in SIZES:
        if offset and n > (1 << 22) + 5:
            continue
        # axpby (fp32, fused multiply-add)
        a, b = rng.randn(n).astype(np.float32), rng.randn(n).astype(np.float32)
        want = np.empty_like(a)
        host.axpby_op(vp(a.ctypes.data), vp(b.ctypes.data), vp(want.ctypes.data), ctypes.c_float(1.25), ll(n))
        da, db = (torch.zeros(n + offset, dtype=torch.float32, device="cuda") for _ in range(2))
        da[offset:].copy_(torch.from_numpy(a))
        db[offset:].copy_(torch.from_numpy(b))
        dout = torch.full((n + offset + 8,), -7.0, dtype=torch.float32, device="cuda")
        es = 4
        gpu.axpby_op(vp(da.data_ptr() + offset * es), vp(db.data_ptr() + offset * es), vp(dout.data_ptr() + offset * es), ctypes.c_float(1.25), ll(n))
        got = dout.cpu().numpy()
        assert np.array_equal(got[offset:offset + n].view(np.uint32), want.view(np.uint32)), f"axpby n={n}"
        assert np.all(got[:offset] == -7.0) and np.all(got[offset + n:] == -7.0), f"axpby wrote outside its range, n={n}"

        # widen (fp32 -> fp64, two shape symbols)
        rows = 3 if n % 3 == 0 and n else 1
        x = (rng.randn(n) * 100).astype(np.float32)
        want64 = np.empty(n, dtype=np.float64)
        host.widen_op(vp(x.ctypes.data), vp(want64.ctypes.data), ll(rows), ll(n // rows))
        dx = torch.zeros(n + offset, dtype=torch.float32, device="cuda")
        dx[offset:].copy_(torch.from_numpy(x))
        dy = torch.full((n + offset + 4,), -7.0, dtype=torch.float64, device="cuda")
        gpu.widen_op(vp(dx.data_ptr() + offset * 4), vp(dy.data_ptr() + offset * 8), ll(rows), ll(n // rows))
        got64 = dy.cpu().numpy()
        assert np.array_equal(got64[offset:offset + n].view(np.uint64), want64.view(np.uint64)), f"widen n={n}"
        assert np.all(got64[:offset] == -7.0) and np.all(got64[offset + n:] == -7.0)

        # in-place update written in docc's container[indvar] form, int shape symbol
        if n < 2**31:
            w, acc = rng.randn(n).astype(np.float32), rng.randn(n).astype(np.float32)
            want_acc = acc.copy()
            host.scale_op(vp(w.ctypes.data), vp(want_acc.ctypes.data), ctypes.c_float(0.01), ctypes.c_int(n))
            dw = torch.zeros(n + offset, dtype=torch.float32, device="cuda")
            dw[offset:].copy_(torch.from_numpy(w))
            dacc = torch.full((n + offset + 8,), -7.0, dtype=torch.float32, device="cuda")
            dacc[offset:offset + n].copy_(torch.from_numpy(acc))
            gpu.scale_op(vp(dw.data_ptr() + offset * 4), vp(dacc.data_ptr() + offset * 4), ctypes.c_float(0.01), ctypes.c_int(n))
            got = dacc.cpu().numpy()
            assert np.array_equal(got[offset:offset + n].view(np.uint32), want_acc.view(np.uint32)), f"scale n={n}"
            assert np.all(got[:offset] == -7.0) and np.all(got[offset + n:] == -7.0)

        # two 16-bit outputs
        p, q = rng.randint(0, 65536, n).astype(np.uint16), rng.randint(0, 65536, n).astype(np.uint16)
        ws, wd = np.empty_like(p), np.empty_like(p)
        host.sumdiff_op(vp(p.ctypes.data), vp(q.ctypes.data), vp(ws.ctypes.data), vp(wd.ctypes.data), ll(n))
        dp, dq = (torch.zeros(n + offset, dtype=torch.int16, device="cuda") for _ in range(2))
        dp[offset:].copy_(torch.from_numpy(p.view(np.int16)))
        dq[offset:].copy_(torch.from_numpy(q.view(np.int16)))
        ds, dd = (torch.full((n + offset + 16,), 77, dtype=torch.int16, device="cuda") for _ in range(2))
        gpu.sumdiff_op(vp(dp.data_ptr() + offset * 2), vp(dq.data_ptr() + offset * 2), vp(ds.data_ptr() + offset * 2), vp(dd.data_ptr() + offset * 2), ll(n))
        gs, gd = ds.cpu().numpy().view(np.uint16), dd.cpu().numpy().view(np.uint16)
        assert np.array_equal(gs[offset:offset + n], ws) and np.array_equal(gd[offset:offset + n], wd), f"sumdiff n={n}"
        assert np.all(gs[offset + n:] == 77) and np.all(gd[:offset] == 77)


@pytest.mark.gpu
def test_map_kernel_bandwidth_is_in_the_hbm_range(rt, map_libs):
    """A sanity bound, not a benchmark: the vector form of the fp32 axpby map (12 B per element) moves a 600 MB working
    set well above what one-element-per-thread kernels of 32-thread blocks reach."""
    import torch

    gpu = ctypes.CDLL(map_libs[0], mode=ctypes.RTLD_GLOBAL)
    vp, ll = ctypes.c_void_p, ctypes.c_longlong
    n = 50_000_000
    a, b, out = (torch.randn(n, device="cuda") for _ in range(3))
    for _ in range(3):
        gpu.axpby_op(vp(a.data_ptr()), vp(b.data_ptr()), vp(out.data_ptr()), ctypes.c_float(0.5), ll(n))
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(10):
        gpu.axpby_op(vp(a.data_ptr()), vp(b.data_ptr()), vp(out.data_ptr()), ctypes.c_float(0.5), ll(n))
    stop.record()
    torch.cuda.synchronize()
    gbs = 12.0 * n * 10 / (start.elapsed_time(stop) * 1e-3) / 1e9
    print(f"axpby map: {gbs:.0f} GB/s")
    assert gbs > 3000
