"""The docc-side plugin: golden text of the emitted host calls (b200_emit.h), and generated host code
in the shape docc's CPPCodeGenerator produces (extern "C" entry, connector locals declared by
LibraryNodeDispatcher::dispatch, one call into the runtime) compiled, linked against
libdocc_b200_rt.so and loaded with ctypes the way CompiledSDFG does."""
import ctypes
import os
import subprocess

import numpy as np
import pytest

from conftest import ROOT, relerr
from docc_b200 import build

PLUGIN = os.path.join(ROOT, "docc_b200", "plugin")
GOLDEN = os.path.join(ROOT, "tests", "golden")


@pytest.fixture(scope="module")
def emit_driver(tmp_path_factory):
    exe = str(tmp_path_factory.mktemp("emit") / "emit_driver")
    subprocess.run(["g++", "-std=c++17", "-I" + PLUGIN, os.path.join(ROOT, "tests", "emit_driver.cpp"), "-o", exe], check=True)
    return exe


def test_emitted_calls_match_golden_text(emit_driver):
    out = subprocess.run([emit_driver], check=True, capture_output=True, text=True).stdout
    assert out == open(os.path.join(GOLDEN, "emitted_calls.txt")).read()
    out = subprocess.run([emit_driver, "checked"], check=True, capture_output=True, text=True).stdout
    assert out == open(os.path.join(GOLDEN, "emitted_calls_checked.txt")).read()


def test_debug_switch_is_read_from_the_environment(tmp_path):
    src = tmp_path / "dbg.cpp"
    src.write_text('#include <iostream>\n#include "b200_emit.h"\nint main() { std::cout << docc_b200_plugin::debug_checks_enabled(); }\n')
    exe = str(tmp_path / "dbg")
    subprocess.run(["g++", "-std=c++17", "-I" + PLUGIN, str(src), "-o", exe], check=True)
    env = dict(os.environ)
    env.pop("DOCC_CUDA_DEBUG", None)
    assert subprocess.run([exe], capture_output=True, text=True, env=env).stdout == "0"
    for val in ("1", "true"):
        assert subprocess.run([exe], capture_output=True, text=True, env=dict(env, DOCC_CUDA_DEBUG=val)).stdout == "1"


def compile_program(emit_driver, tmp_path, checked):
    """The translation unit `emit_driver program` prints: every node call comes from the dispatchers' emitters."""
    text = subprocess.run([emit_driver, "program"] + (["checked"] if checked else []), check=True, capture_output=True, text=True).stdout
    src = tmp_path / "program.cpp"
    src.write_text(text)
    lib = str(tmp_path / "libprogram.so")
    subprocess.run(["g++", "-std=c++17", "-shared", "-fPIC", "-I" + os.path.join(ROOT, "include"), str(src), "-o", lib,
                    "-L" + build.LIB_DIR, "-Wl,-rpath," + build.LIB_DIR, "-ldocc_b200_rt"], check=True)
    return ctypes.CDLL(lib), text


@pytest.mark.parametrize("checked", [False, True])
def test_generated_program_with_every_new_node_compiles_and_links(emit_driver, tmp_path, checked):
    handle, text = compile_program(emit_driver, tmp_path, checked)
    for fn in ("matmul_op", "softmax_op", "conv_op", "attn_op", "ln_erf_div_op", "offload_op"):
        assert hasattr(handle, fn)
    for call in ("docc_b200_gemm", "docc_b200_softmax", "docc_b200_conv", "docc_b200_attention", "docc_b200_layernorm", "docc_b200_bias_act", "docc_b200_binary", "docc_b200_cast",
                 "docc_b200_reduce", "docc_b200_malloc", "docc_b200_h2d", "docc_b200_d2h", "docc_b200_free"):
        assert call in text


@pytest.mark.gpu
def test_generated_program_runs_on_the_gpu(rt, emit_driver, tmp_path):
    import scipy.special

    handle, _ = compile_program(emit_driver, tmp_path, checked=True)
    vp, i64 = ctypes.c_void_p, ctypes.c_int64
    rng = np.random.RandomState(3)
    # attention, causal, default scale, host pointers
    B, H, S, D = 2, 3, 40, 32
    q, k, v = (rng.randn(B, H, S, D).astype(np.float32) for _ in range(3))
    o = np.zeros_like(q)
    handle.attn_op(vp(q.ctypes.data), vp(k.ctypes.data), vp(v.ctypes.data), vp(o.ctypes.data), i64(B), i64(H), i64(S), i64(S))
    sc = np.einsum("bhid,bhjd->bhij", q.astype(np.float64), k.astype(np.float64)) / np.sqrt(D)
    sc = np.where(np.tril(np.ones((S, S), dtype=bool)), sc, -np.inf)
    ref = np.einsum("bhij,bhjd->bhid", scipy.special.softmax(sc, axis=-1), v.astype(np.float64))
    assert relerr(o, ref) <= 1e-4
    # LayerNorm -> erf -> divide by the input
    x = (rng.randn(37, 96) + 2.0).astype(np.float32)
    g, b = (rng.rand(96) + 0.5).astype(np.float32), rng.randn(96).astype(np.float32)
    y = np.zeros_like(x)
    handle.ln_erf_div_op(vp(x.ctypes.data), vp(g.ctypes.data), vp(b.ctypes.data), vp(y.ctypes.data), i64(37), i64(96))
    x64 = x.astype(np.float64)
    ln = (x64 - x64.mean(-1, keepdims=True)) / np.sqrt(x64.var(-1, keepdims=True) + 1e-5) * g + b
    assert relerr(y, scipy.special.erf(ln) / x64) <= 1e-4
    # offloaded region: device-resident cast and mean between the transfers
    a = rng.randn(50, 70).astype(np.float32)
    c, m = np.zeros((50, 70)), np.zeros(50)
    handle.offload_op(vp(a.ctypes.data), vp(c.ctypes.data), vp(m.ctypes.data), i64(50), i64(70))
    assert np.array_equal(c, a.astype(np.float64))
    assert relerr(m, a.astype(np.float64).mean(axis=1)) <= 1e-12


@pytest.mark.gpu
def test_generated_config1_config2_and_conv_run_on_the_gpu(rt, emit_driver, tmp_path):
    handle, _ = compile_program(emit_driver, tmp_path, checked=True)
    vp, i64 = ctypes.c_void_p, ctypes.c_int64
    rng = np.random.RandomState(0)
    a, b = rng.rand(10, 12), rng.rand(12, 7)
    c = np.zeros((10, 7))
    handle.matmul_op(vp(a.ctypes.data), vp(b.ctypes.data), vp(c.ctypes.data), i64(10), i64(12), i64(7))
    assert np.allclose(c, a @ b)
    x = (rng.randn(8192, 4096) * 3).astype(np.float32)
    y = np.empty_like(x)
    handle.softmax_op(vp(x.ctypes.data), vp(y.ctypes.data), i64(8192), i64(4096))
    e = np.exp(x - x.max(axis=1, keepdims=True))
    assert relerr(y, e / e.sum(axis=1, keepdims=True)) <= 1e-4
    import oracle

    xc, wc, bc = rng.randn(3, 8, 12, 12).astype(np.float32), rng.randn(16, 8, 3, 3).astype(np.float32), rng.randn(16).astype(np.float32)
    yc = np.zeros((3, 16, 12, 12), dtype=np.float32)
    handle.conv_op(vp(xc.ctypes.data), vp(wc.ctypes.data), vp(bc.ctypes.data), vp(yc.ctypes.data), i64(3))
    assert relerr(yc, oracle.conv(xc, wc, bc, pads=[1, 1, 1, 1])) <= 1e-4
