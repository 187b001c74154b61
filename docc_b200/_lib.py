"""ctypes binding of ``libdocc_b200_rt.so`` (declarations mirror ``include/docc_b200/rt.h``).

There is no fallback: if the shared library has not been built, loading raises.
"""
from __future__ import annotations

import ctypes
import os

from .build import LIB_PATH

_i64 = ctypes.c_int64
_vp = ctypes.c_void_p
_int = ctypes.c_int
_f32 = ctypes.c_float
_f64 = ctypes.c_double
_sz = ctypes.c_size_t
_pi64 = ctypes.POINTER(ctypes.c_int64)


class BlockParams(ctypes.Structure):
    """``docc_b200_block_params``."""

    _fields_ = [
        ("batch", _i64), ("seq", _i64), ("d_model", _i64), ("n_heads", _i64), ("d_ff", _i64),
        ("eps", _f64),
        ("ln1_g", _vp), ("ln1_b", _vp), ("w_qkv", _vp), ("b_qkv", _vp), ("w_o", _vp), ("b_o", _vp),
        ("ln2_g", _vp), ("ln2_b", _vp), ("w_1", _vp), ("b_1", _vp), ("w_2", _vp), ("b_2", _vp),
    ]


# name -> (restype, argtypes); every symbol declared in rt.h
SIGNATURES = {
    "docc_b200_init": (_int, [_int]),
    "docc_b200_shutdown": (_int, []),
    "docc_b200_device_count": (_int, []),
    "docc_b200_malloc": (_int, [ctypes.POINTER(_vp), _sz]),
    "docc_b200_free": (_int, [_vp]),
    "docc_b200_h2d": (_int, [_vp, _vp, _sz]),
    "docc_b200_d2h": (_int, [_vp, _vp, _sz]),
    "docc_b200_host_alloc": (_int, [ctypes.POINTER(_vp), _sz]),
    "docc_b200_host_free": (_int, [_vp]),
    "docc_b200_set_alloc_limit": (_int, [_sz]),
    "docc_b200_set_stream": (_int, [_vp]),
    "docc_b200_get_stream": (_int, [ctypes.POINTER(_vp)]),
    "docc_b200_sync": (_int, []),
    "docc_b200_strerror": (ctypes.c_char_p, [_int]),
    "docc_b200_last_error": (ctypes.c_char_p, []),
    "docc_b200_launch_count": (_i64, [_int]),
    "docc_b200_selftest_wait_timeout": (_int, [_i64]),
    "docc_b200_gemm": (_int, [_int, _int, _int, _int, _i64, _i64, _i64, _vp, _vp, _i64, _vp, _i64, _vp, _vp, _i64, _int]),
    "docc_b200_gemm_f32_noalloc": (_int, [_int, _int, _i64, _i64, _i64, _f32, _vp, _i64, _vp, _i64, _f32, _vp, _i64, _vp]),
    "docc_b200_matmul": (_int, [_int, _i64, _i64, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _i64, _int]),
    "docc_b200_gemm_epilogue": (_int, [_int, _int, _i64, _i64, _i64, _f32, _vp, _i64, _vp, _i64, _vp, _int, _vp, _i64, _vp, _i64, _int]),
    "docc_b200_softmax": (_int, [_int, _int, _pi64, _int, _pi64, _vp, _vp, _int]),
    "docc_b200_reduce": (_int, [_int, _int, _int, _pi64, _int, _pi64, _vp, _vp, _int]),
    "docc_b200_conv": (_int, [_int, _int, _int, _pi64, _pi64, _pi64, _pi64, _pi64, _i64, _i64, _vp, _vp, _vp, _vp, _int]),
    "docc_b200_attention": (_int, [_int, _i64, _i64, _i64, _i64, _i64, _f32, _int, _vp, _pi64, _vp, _pi64, _vp, _pi64, _vp, _pi64, _int]),
    "docc_b200_layernorm": (_int, [_int, _i64, _i64, _vp, _vp, _vp, _f64, _vp, _int]),
    "docc_b200_bias_act": (_int, [_int, _i64, _i64, _vp, _f32, _vp, _int, _vp, _vp, _int]),
    "docc_b200_binary": (_int, [_int, _int, _i64, _vp, _vp, _vp, _int]),
    "docc_b200_cast": (_int, [_int, _int, _i64, _vp, _vp, _int]),
    "docc_b200_transformer_block": (_int, [_int, ctypes.POINTER(BlockParams), _vp, _vp, _int]),
}

_lib = None


class DoccB200Error(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, status: int, name: str, detail: str):
        self.status = status
        super().__init__(f"{name} failed with status {status}: {detail}")


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = os.environ.get("DOCC_B200_RT_LIB", LIB_PATH)  # a differently built runtime may be substituted
        if not os.path.exists(path):
            raise RuntimeError(
                f"{path} is missing: the CUDA runtime library has not been built. "
                "Run `python -m docc_b200.build` (needs nvcc); there is no CPU fallback."
            )
        handle = ctypes.CDLL(path)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def check(status: int, name: str) -> None:
    if status != 0:
        handle = lib()
        detail = handle.docc_b200_last_error().decode() or handle.docc_b200_strerror(status).decode()
        raise DoccB200Error(status, name, detail)


def call(name: str, *args) -> None:
    check(getattr(lib(), name)(*args), name)
