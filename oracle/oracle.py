"""ctypes front end of the CPU oracle (``oracle.cpp``).

TEST INFRASTRUCTURE — not part of the product. Only the test-suite, the smoke
check and the CPU-baseline / reference arm of the benchmark import this module.
Each function mirrors one entry of the runtime's C ABI on numpy arrays.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_lib = None

ROW_MAJOR, COL_MAJOR = 101, 102
NO_TRANS, TRANS = 111, 112
RED_SUM, RED_MAX, RED_MIN, RED_MEAN, RED_STD = range(5)
ACT_NONE, ACT_GELU_ERF, ACT_RELU, ACT_TANH, ACT_SIGMOID, ACT_EXP, ACT_ERF, ACT_SQRT, ACT_ABS = range(9)

_i64 = ctypes.c_int64
_vp = ctypes.c_void_p


def build(force: bool = False) -> str:
    """Compile ``liboracle.so`` with the Makefile beside this file."""
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(
        os.path.join(_HERE, "oracle.cpp")
    ):
        subprocess.run(["make", "-B", "-C", _HERE], check=True, capture_output=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.oracle_num_threads.restype = ctypes.c_int
    return _lib


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def set_num_threads(n: int) -> None:
    """OpenMP team size for the following calls (launchers like torchrun export OMP_NUM_THREADS=1)."""
    lib().oracle_set_num_threads(int(n))


def _prec(dtype) -> int:
    dt = np.dtype(dtype)
    if dt == np.float64:
        return ord("d")
    if dt == np.float32:
        return ord("s")
    if dt == np.float16:
        return ord("h")
    if dt.name == "bfloat16":
        return ord("b")
    raise TypeError(f"unsupported dtype {dt}")


def _ptr(a):
    return _vp(a.ctypes.data) if a is not None else _vp(0)


def _i64arr(seq):
    seq = [int(v) for v in seq]
    return (_i64 * max(len(seq), 1))(*seq)


def gemm(A, B, C=None, alpha=1.0, beta=0.0, transa=False, transb=False, layout=ROW_MAJOR, m=None, n=None, k=None,
         lda=None, ldb=None, ldc=None):
    """C = alpha*op(A)*op(B) + beta*C with the GEMMNode loop order. Arrays are
    interpreted as flat buffers with the given leading dimensions."""
    A = np.ascontiguousarray(A)
    B = np.ascontiguousarray(B)
    if m is None:
        if layout == ROW_MAJOR:
            m, k = (A.shape[1], A.shape[0]) if transa else A.shape
            n = B.shape[0] if transb else B.shape[1]
        else:  # numpy arrays hold the column-major matrix transposed
            m, k = (A.shape[0], A.shape[1]) if transa else (A.shape[1], A.shape[0])
            n = B.shape[1] if transb else B.shape[0]
    lda = lda or A.shape[-1]
    ldb = ldb or B.shape[-1]
    if C is None:
        C = np.zeros((m, n) if layout == ROW_MAJOR else (n, m), dtype=A.dtype)
    ldc = ldc or C.shape[-1]
    rc = lib().oracle_gemm(_prec(A.dtype), layout, TRANS if transa else NO_TRANS, TRANS if transb else NO_TRANS,
                           _i64(m), _i64(n), _i64(k), ctypes.c_double(alpha), _ptr(A), _i64(lda), _ptr(B), _i64(ldb),
                           ctypes.c_double(beta), _ptr(C), _i64(ldc))
    assert rc == 0
    return C


def matmul(A, B):
    """Batched row-major matmul (MatMulNode)."""
    A = np.ascontiguousarray(A)
    B = np.ascontiguousarray(B)
    batch_shape = np.broadcast_shapes(A.shape[:-2], B.shape[:-2])
    m, k = A.shape[-2:]
    n = B.shape[-1]
    Ab = np.ascontiguousarray(np.broadcast_to(A, batch_shape + (m, k)))
    Bb = np.ascontiguousarray(np.broadcast_to(B, batch_shape + (k, n)))
    Y = np.zeros(batch_shape + (m, n), dtype=A.dtype)
    batch = int(np.prod(batch_shape)) if batch_shape else 1
    rc = lib().oracle_matmul(_prec(A.dtype), _i64(batch), _i64(m), _i64(n), _i64(k), _ptr(Ab), _i64(k), _i64(m * k),
                             _ptr(Bb), _i64(n), _i64(k * n), _ptr(Y), _i64(n), _i64(m * n))
    assert rc == 0
    return Y


def softmax(X, axes=None):
    X = np.ascontiguousarray(X)
    if axes is None:
        axes = list(range(X.ndim))
    if np.isscalar(axes):
        axes = [axes]
    Y = np.empty_like(X)
    rc = lib().oracle_softmax(_prec(X.dtype), X.ndim, _i64arr(X.shape), len(axes), _i64arr(axes), _ptr(X), _ptr(Y))
    assert rc == 0
    return Y


def reduce(op, X, axes):
    X = np.ascontiguousarray(X)
    if np.isscalar(axes):
        axes = [axes]
    norm = sorted(a % X.ndim for a in axes)
    out_shape = tuple(s for d, s in enumerate(X.shape) if d not in norm)
    Y = np.empty(out_shape, dtype=X.dtype)
    rc = lib().oracle_reduce(op, _prec(X.dtype), X.ndim, _i64arr(X.shape), len(axes), _i64arr(axes), _ptr(X), _ptr(Y))
    assert rc == 0
    return Y


def conv_out_shape(x_shape, k_shape, strides, pads, dilations, c_out):
    sr = len(k_shape)
    out = [x_shape[0], c_out]
    for i in range(sr):
        out.append((x_shape[2 + i] + pads[i] + pads[sr + i] - dilations[i] * (k_shape[i] - 1) - 1) // strides[i] + 1)
    return tuple(out)


def conv(X, W, bias=None, strides=None, pads=None, dilations=None, group=1, out_dtype=None):
    """N-D cross-correlation (ConvNode). ``pads`` = [begin..., end...]."""
    X = np.ascontiguousarray(X)
    W = np.ascontiguousarray(W)
    sr = X.ndim - 2
    strides = list(strides or [1] * sr)
    pads = list(pads or [0] * (2 * sr))
    dilations = list(dilations or [1] * sr)
    k_shape = W.shape[2:]
    c_out = W.shape[0]
    out_dtype = np.dtype(out_dtype or (np.float32 if X.dtype.itemsize == 2 else X.dtype))
    Y = np.empty(conv_out_shape(X.shape, k_shape, strides, pads, dilations, c_out), dtype=out_dtype)
    if bias is not None:
        bias = np.ascontiguousarray(bias, dtype=out_dtype)
    rc = lib().oracle_conv(_prec(X.dtype), _prec(out_dtype), sr, _i64arr(X.shape), _i64arr(k_shape), _i64arr(strides),
                           _i64arr(pads), _i64arr(dilations), _i64(c_out), _i64(group), _ptr(X), _ptr(W), _ptr(bias),
                           _ptr(Y))
    assert rc == 0
    return Y


def attention(Q, K, V, scale=None, causal=False):
    """softmax(scale*Q K^T [+causal]) V on contiguous [B,H,S,D] arrays."""
    Q, K, V = (np.ascontiguousarray(t) for t in (Q, K, V))
    B, H, Sq, D = Q.shape
    Skv = K.shape[2]
    if scale is None:
        scale = 1.0 / np.sqrt(D)
    O = np.empty_like(Q)
    rc = lib().oracle_attention(_prec(Q.dtype), _i64(B), _i64(H), _i64(Sq), _i64(Skv), _i64(D), ctypes.c_float(scale),
                                int(bool(causal)), _ptr(Q), _vp(0), _ptr(K), _vp(0), _ptr(V), _vp(0), _ptr(O), _vp(0))
    assert rc == 0
    return O


def layernorm(X, gamma=None, beta=None, eps=1e-5):
    X = np.ascontiguousarray(X)
    cols = X.shape[-1]
    rows = X.size // cols
    g = None if gamma is None else np.ascontiguousarray(gamma, dtype=np.float32)
    b = None if beta is None else np.ascontiguousarray(beta, dtype=np.float32)
    Y = np.empty_like(X)
    rc = lib().oracle_layernorm(_prec(X.dtype), _i64(rows), _i64(cols), _ptr(X), _ptr(g), _ptr(b), ctypes.c_double(eps),
                                _ptr(Y))
    assert rc == 0
    return Y


def bias_act(X, scale=1.0, bias=None, act=ACT_NONE, residual=None):
    X = np.ascontiguousarray(X)
    cols = X.shape[-1]
    rows = X.size // cols
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    r = None if residual is None else np.ascontiguousarray(residual, dtype=X.dtype)
    Y = np.empty_like(X)
    rc = lib().oracle_bias_act(_prec(X.dtype), _i64(rows), _i64(cols), _ptr(X), ctypes.c_float(scale), _ptr(b), int(act),
                               _ptr(r), _ptr(Y))
    assert rc == 0
    return Y


def binary(op, A, B):
    A = np.ascontiguousarray(A)
    B = np.ascontiguousarray(B, dtype=A.dtype)
    Y = np.empty_like(A)
    rc = lib().oracle_binary(int(op), _prec(A.dtype), _i64(A.size), _ptr(A), _ptr(B), _ptr(Y))
    assert rc == 0
    return Y


def linear(X, W, bias=None, act=ACT_NONE, residual=None):
    """Y = act(X W^T + bias) + residual — GEMM (transb) followed by the element-wise chain."""
    X2 = np.ascontiguousarray(X).reshape(-1, X.shape[-1])
    Y = gemm(X2, np.ascontiguousarray(W), transb=True)
    res2 = None if residual is None else np.ascontiguousarray(residual).reshape(Y.shape)
    if bias is not None or act != ACT_NONE or residual is not None:
        Y = bias_act(Y, 1.0, bias, act, res2)
    return Y.reshape(X.shape[:-1] + (W.shape[0],))


def transformer_block(x, p, n_heads, eps=1e-5):
    """Pre-LN encoder block composed from the restated nodes. ``p`` maps the
    docc_b200_block_params field names to arrays (weights [out, in])."""
    Bn, S, d = x.shape
    dh = d // n_heads
    h1 = layernorm(x, p["ln1_g"], p["ln1_b"], eps)
    qkv = linear(h1, p["w_qkv"], p["b_qkv"]).reshape(Bn, S, 3, n_heads, dh)
    q, k, v = (np.ascontiguousarray(qkv[:, :, i].transpose(0, 2, 1, 3)) for i in range(3))
    a = attention(q, k, v, 1.0 / np.sqrt(dh), False)
    a = np.ascontiguousarray(a.transpose(0, 2, 1, 3)).reshape(Bn, S, d)
    h = linear(a, p["w_o"], p["b_o"], ACT_NONE, x)
    h2 = layernorm(h, p["ln2_g"], p["ln2_b"], eps)
    f = linear(h2, p["w_1"], p["b_1"], ACT_GELU_ERF)
    return linear(f, p["w_2"], p["b_2"], ACT_NONE, h)


def to_bf16_bits(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    out = np.empty(a.shape, dtype=np.uint16)
    lib().oracle_f32_to_bf16(_ptr(a), _ptr(out), _i64(a.size))
    return out


def from_bf16_bits(a):
    a = np.ascontiguousarray(a, dtype=np.uint16)
    out = np.empty(a.shape, dtype=np.float32)
    lib().oracle_bf16_to_f32(_ptr(a), _ptr(out), _i64(a.size))
    return out
