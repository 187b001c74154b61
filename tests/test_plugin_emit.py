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


def generated_source(checked: bool) -> str:
    lines = open(os.path.join(GOLDEN, "emitted_calls_checked.txt" if checked else "emitted_calls.txt")).read().splitlines()
    if checked:
        gemm_call = "\n".join(lines[1:8])
        softmax_start = next(i for i, l in enumerate(lines) if "docc_b200_softmax" in l) - 1
        softmax_call = "\n".join(lines[softmax_start:softmax_start + 7])
    else:
        gemm_call = lines[1]
        softmax_call = next(l for l in lines if l.startswith("docc_b200_softmax"))
    return f"""
#include <docc_b200/rt.h>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
// entry in the shape of CPPCodeGenerator (cpp_code_generator.cpp:8-24): arrays, _s<i> shape symbols, _docc_ret_<i>
extern "C" void matmul_op(double* a, double* b, double* _docc_ret_0, int64_t _s0, int64_t _s1, int64_t _s2) {{
    {{
        double* __A = a; double* __B = b; double* __C = _docc_ret_0; double __alpha = 1.0; double __beta = 0.0;
        {gemm_call}
    }}
}}
extern "C" void softmax_op(float* x, float* _docc_ret_0) {{
    {{
        float* X = x; float* Y = _docc_ret_0;
        {softmax_call}
    }}
}}
"""


def compile_generated(tmp_path, checked):
    src = tmp_path / "generated.cpp"
    src.write_text(generated_source(checked))
    lib = str(tmp_path / "libgenerated.so")
    subprocess.run(["g++", "-std=c++17", "-shared", "-fPIC", "-I" + os.path.join(ROOT, "include"), str(src), "-o", lib,
                    "-L" + build.LIB_DIR, "-Wl,-rpath," + build.LIB_DIR, "-ldocc_b200_rt"], check=True)
    return ctypes.CDLL(lib)


@pytest.mark.parametrize("checked", [False, True])
def test_generated_host_code_compiles_and_links(tmp_path, checked):
    handle = compile_generated(tmp_path, checked)
    assert hasattr(handle, "matmul_op") and hasattr(handle, "softmax_op")


@pytest.mark.gpu
def test_generated_host_code_runs_on_the_gpu(rt, tmp_path):
    handle = compile_generated(tmp_path, checked=True)
    rng = np.random.RandomState(0)
    a, b = rng.rand(10, 12), rng.rand(12, 7)
    c = np.zeros((10, 7))
    handle.matmul_op(ctypes.c_void_p(a.ctypes.data), ctypes.c_void_p(b.ctypes.data), ctypes.c_void_p(c.ctypes.data),
                     ctypes.c_int64(10), ctypes.c_int64(12), ctypes.c_int64(7))
    assert np.allclose(c, a @ b)
    x = (rng.randn(8192, 4096) * 3).astype(np.float32)
    y = np.empty_like(x)
    handle.softmax_op(ctypes.c_void_p(x.ctypes.data), ctypes.c_void_p(y.ctypes.data))
    e = np.exp(x - x.max(axis=1, keepdims=True))
    assert relerr(y, e / e.sum(axis=1, keepdims=True)) <= 1e-4
