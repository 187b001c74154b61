"""Array-level host API over the C ABI.

Each function accepts either numpy arrays (host memory: the call stages the data
through the device, docc's "WithTransfers" flavour) or torch CUDA tensors (device
pointers, asynchronous on the library's current stream). Mixed inputs are an error.
Outputs have the kind of the inputs.

Stream ordering of device calls: the library's current stream is, by default, a private
non-blocking stream of the calling thread that is NOT ordered after torch's streams. Code that
mixes torch operations and these calls on the same tensors must either route the library to
torch's stream first (``set_stream(torch.cuda.current_stream().cuda_stream)``, which the front
ends in ``docc_b200.torch`` / ``docc_b200.python`` do on every call) or synchronise around the
calls (``torch.cuda.synchronize()`` before, ``sync()`` after).
"""
from __future__ import annotations

import ctypes
import math

import numpy as np

from . import _lib
from ._lib import BlockParams, call

ROW_MAJOR, COL_MAJOR = 101, 102
NO_TRANS, TRANS = 111, 112
FLAG_HOST_PTRS, FLAG_FP32_EXACT = 1, 2
ACT_NONE, ACT_GELU_ERF, ACT_RELU, ACT_TANH, ACT_SIGMOID, ACT_EXP, ACT_ERF, ACT_SQRT, ACT_ABS = range(9)
EW_ADD, EW_SUB, EW_MUL, EW_DIV, EW_MAX, EW_MIN = range(6)
RED_SUM, RED_MAX, RED_MIN, RED_MEAN, RED_STD = range(5)

_i64 = ctypes.c_int64
_vp = ctypes.c_void_p


class DeviceArray:
    """A C-order array in device memory obtained from ``docc_b200_malloc`` (the runtime's pool).

    This is what a container of an offloaded SDFG is between its H2D and D2H transfer nodes: the
    front ends keep intermediates in DeviceArrays so that consecutive library nodes exchange no
    data with the host. Freed through ``docc_b200_free`` when the last reference goes away."""

    is_cuda = True

    def __init__(self, shape, dtype):
        self.shape = tuple(int(v) for v in shape)
        self.dtype = np.dtype(dtype)
        self.nbytes = int(np.prod(self.shape, dtype=np.int64)) * self.dtype.itemsize if self.shape else self.dtype.itemsize
        ptr = _vp()
        call("docc_b200_malloc", ctypes.byref(ptr), max(self.nbytes, 1))
        self._ptr = ptr.value
        self._owner = None

    @property
    def ndim(self):
        return len(self.shape)

    def data_ptr(self):
        return self._ptr

    def is_contiguous(self):
        return True

    @classmethod
    def from_numpy(cls, a):
        a = np.ascontiguousarray(a)
        out = cls(a.shape, a.dtype)
        if a.nbytes:
            call("docc_b200_h2d", _vp(out._ptr), _vp(a.ctypes.data), a.nbytes)
        return out

    def to_numpy(self):
        out = np.empty(self.shape, dtype=self.dtype)
        if out.nbytes:
            call("docc_b200_d2h", _vp(out.ctypes.data), _vp(self._ptr), out.nbytes)
        return out

    def reshape(self, *shape):
        shape = shape[0] if len(shape) == 1 and isinstance(shape[0], (tuple, list)) else shape
        shape = list(shape)
        n = int(np.prod(self.shape, dtype=np.int64)) if self.shape else 1
        if -1 in shape:
            known = int(np.prod([v for v in shape if v != -1], dtype=np.int64)) if len(shape) > 1 else 1
            shape[shape.index(-1)] = n // max(known, 1)
        if int(np.prod(shape, dtype=np.int64)) != n:
            raise ValueError("reshape changes the number of elements")
        view = object.__new__(DeviceArray)
        view.shape, view.dtype, view.nbytes, view._ptr = tuple(shape), self.dtype, self.nbytes, self._ptr
        view._owner = self._owner or self  # keeps the allocation alive
        return view

    def __del__(self):
        if getattr(self, "_owner", None) is None and getattr(self, "_ptr", None):
            try:
                _lib.lib().docc_b200_free(_vp(self._ptr))
            except Exception:
                pass
            self._ptr = None


def _is_torch(x) -> bool:
    return type(x).__module__.startswith("torch")


def _prec(x) -> int:
    if _is_torch(x):
        name = str(x.dtype).replace("torch.", "")
    else:
        name = np.dtype(x.dtype).name  # numpy arrays and DeviceArrays
    try:
        return {"float64": ord("d"), "float32": ord("s"), "float16": ord("h"), "bfloat16": ord("b")}[name]
    except KeyError:
        raise TypeError(f"unsupported element type {name}") from None


def _ptr(x):
    if x is None:
        return _vp(0)
    if _is_torch(x) or isinstance(x, DeviceArray):
        return _vp(x.data_ptr())
    return _vp(x.ctypes.data)


def _arr(seq):
    seq = [int(v) for v in seq]
    return (_i64 * max(len(seq), 1))(*seq)


def _kind(*xs):
    """Returns (flags, empty_like factory) after checking all arrays live on the same side."""
    xs = [x for x in xs if x is not None]
    torch_side = [_is_torch(x) or isinstance(x, DeviceArray) for x in xs]
    if any(torch_side) and not all(torch_side):
        raise TypeError("mix of host arrays and device tensors")
    if all(torch_side):
        for x in xs:
            if not x.is_cuda:
                raise TypeError("torch tensors must live on a CUDA device (pass numpy arrays for host data)")
            if not x.is_contiguous():
                raise ValueError("tensors must be contiguous")
        return 0
    for x in xs:
        if not x.flags["C_CONTIGUOUS"]:
            raise ValueError("arrays must be C-contiguous")
    return FLAG_HOST_PTRS


def _empty(like, shape, dtype=None):
    if isinstance(like, DeviceArray):
        return DeviceArray(shape, dtype or like.dtype)
    if _is_torch(like):
        import torch

        return torch.empty(tuple(shape), dtype=dtype or like.dtype, device=like.device)
    return np.empty(tuple(shape), dtype=dtype or like.dtype)


def _scalar(prec, value):
    return ctypes.c_double(value) if prec == ord("d") else ctypes.c_float(value)


def init(device: int = 0) -> None:
    call("docc_b200_init", int(device))


def sync() -> None:
    call("docc_b200_sync")


def set_stream(stream_handle) -> None:
    """Route launches of the calling thread to ``stream_handle`` (a cudaStream_t value, e.g.
    ``torch.cuda.current_stream().cuda_stream``). ``None`` restores the library's own stream; the
    value 0 names the legacy default stream and is passed on as CUDA's ``cudaStreamLegacy`` handle."""
    if stream_handle is None:
        call("docc_b200_set_stream", _vp(0))
    else:
        call("docc_b200_set_stream", _vp(int(stream_handle) or 1))


def launch_count(reset: bool = False) -> int:
    return int(_lib.lib().docc_b200_launch_count(1 if reset else 0))


def gemm(A, B, C=None, alpha=1.0, beta=0.0, transa=False, transb=False, layout=ROW_MAJOR, flags=0):
    """C = alpha*op(A)*op(B) + beta*C (GEMMNode). 2-D arrays; for COL_MAJOR the arrays hold the
    matrices transposed, as a Fortran caller would see them."""
    flags |= _kind(A, B, C)
    prec = _prec(A)
    if layout == ROW_MAJOR:
        m, k = (A.shape[1], A.shape[0]) if transa else A.shape
        n = B.shape[0] if transb else B.shape[1]
        c_shape = (m, n)
    else:
        k, m = (A.shape[1], A.shape[0]) if transa else A.shape
        n = B.shape[1] if transb else B.shape[0]
        c_shape = (n, m)
    if C is None:
        C = _empty(A, c_shape)
        beta = 0.0
    al, be = _scalar(prec, alpha), _scalar(prec, beta)
    call("docc_b200_gemm", prec, layout, TRANS if transa else NO_TRANS, TRANS if transb else NO_TRANS, m, n, k,
         ctypes.cast(ctypes.pointer(al), _vp), _ptr(A), A.shape[-1], _ptr(B), B.shape[-1],
         ctypes.cast(ctypes.pointer(be), _vp), _ptr(C), C.shape[-1], flags)
    return C


def gemm_strided(precision, layout, transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, flags=0):
    """GEMM on flat buffers with explicit leading dimensions, the form docc's generated code passes to BLAS
    (gemm_node.cpp:441-520): ``C`` is updated in place. ``precision`` is one of 'h', 's', 'd', 'b'."""
    flags |= _kind(A, B, C)
    prec = ord(precision)
    if prec != _prec(A) or prec != _prec(B) or prec != _prec(C):
        raise TypeError(f"gemm_strided: operands are not all of precision {precision!r}")
    al, be = _scalar(prec, float(alpha)), _scalar(prec, float(beta))
    call("docc_b200_gemm", prec, int(layout), TRANS if transa else NO_TRANS, TRANS if transb else NO_TRANS, int(m), int(n), int(k),
         ctypes.cast(ctypes.pointer(al), _vp), _ptr(A), int(lda), _ptr(B), int(ldb),
         ctypes.cast(ctypes.pointer(be), _vp), _ptr(C), int(ldc), flags)
    return C


def matmul(A, B, flags=0):
    """Batched row-major matmul with numpy broadcasting rules on the batch dims (MatMulNode)."""
    flags |= _kind(A, B)
    m, k = A.shape[-2:]
    n = B.shape[-1]
    batch_shape = tuple(np.broadcast_shapes(tuple(A.shape[:-2]), tuple(B.shape[:-2])))
    batch = int(np.prod(batch_shape)) if batch_shape else 1
    sa = 0 if A.ndim == 2 else m * k
    sb = 0 if B.ndim == 2 else k * n
    if A.ndim > 2 and tuple(A.shape[:-2]) != batch_shape or B.ndim > 2 and tuple(B.shape[:-2]) != batch_shape:
        raise ValueError("batch dims must match exactly or the operand must be 2-D")
    Y = _empty(A, batch_shape + (m, n))
    call("docc_b200_matmul", _prec(A), batch, m, n, k, _ptr(A), k, sa, _ptr(B), n, sb, _ptr(Y), n, m * n, flags)
    return Y


def linear(X, W, bias=None, act=ACT_NONE, residual=None, alpha=1.0, flags=0):
    """Y = act(alpha * X W^T + bias) + residual with the torch Linear weight layout [out, in]."""
    flags |= _kind(X, W, bias, residual)
    if bias is not None:
        # the ABI reads the bias as fp32 for 16-bit operands and in the operand type otherwise
        want = ord("s") if _prec(X) in (ord("h"), ord("b")) else _prec(X)
        if _prec(bias) != want:
            raise TypeError(f"linear: bias must be {'float32' if want == ord('s') else 'float64'} for {chr(_prec(X))!r} operands")
    k = X.shape[-1]
    m = int(np.prod(X.shape[:-1]))
    n = W.shape[0]
    # the ABI sees pointers and leading dimensions only: extents and types are checked here
    if W.ndim != 2 or W.shape[1] != k or _prec(W) != _prec(X):
        raise ValueError(f"linear: weight {tuple(W.shape)} does not match inputs of width {k} and type {chr(_prec(X))!r}")
    if bias is not None and int(np.prod(bias.shape)) != n:
        raise ValueError(f"linear: bias has {int(np.prod(bias.shape))} elements for {n} output features")
    if residual is not None and (tuple(residual.shape) != tuple(X.shape[:-1]) + (n,) or _prec(residual) != _prec(X)):
        raise ValueError("linear: the residual must have the shape and type of the output (broadcast it first)")
    Y = _empty(X, tuple(X.shape[:-1]) + (n,))
    call("docc_b200_gemm_epilogue", _prec(X), TRANS, m, n, k, float(alpha), _ptr(X), k, _ptr(W), k, _ptr(bias), int(act),
         _ptr(residual), n, _ptr(Y), n, flags)
    return Y


def softmax(X, axes=None, flags=0):
    flags |= _kind(X)
    if axes is None:
        axes = list(range(X.ndim))
    if np.isscalar(axes):
        axes = [axes]
    Y = _empty(X, X.shape)
    call("docc_b200_softmax", _prec(X), X.ndim, _arr(X.shape), len(axes), _arr(axes), _ptr(X), _ptr(Y), flags)
    return Y


def reduce(op, X, axes, flags=0):
    flags |= _kind(X)
    if np.isscalar(axes):
        axes = [axes]
    norm = sorted(a % X.ndim for a in axes)
    out_shape = tuple(s for d, s in enumerate(X.shape) if d not in norm)
    Y = _empty(X, out_shape)
    call("docc_b200_reduce", int(op), _prec(X), X.ndim, _arr(X.shape), len(axes), _arr(axes), _ptr(X), _ptr(Y), flags)
    return Y


def conv_out_shape(x_shape, k_shape, strides, pads, dilations, c_out):
    sr = len(k_shape)
    out = [x_shape[0], c_out]
    for i in range(sr):
        num = x_shape[2 + i] + pads[i] + pads[sr + i] - dilations[i] * (k_shape[i] - 1) - 1
        out.append(0 if num < 0 else num // strides[i] + 1)
    return tuple(out)


def conv(X, W, bias=None, strides=None, pads=None, dilations=None, group=1, out_dtype=None, flags=0):
    """N-D cross-correlation in NC(D..) layout (ConvNode). ``pads`` = [begin..., end...]."""
    flags |= _kind(X, W, bias)
    sr = X.ndim - 2
    strides = list(strides or [1] * sr)
    pads = list(pads or [0] * (2 * sr))
    dilations = list(dilations or [1] * sr)
    k_shape = tuple(W.shape[2:])
    c_out = W.shape[0]
    prec_in = _prec(X)
    if out_dtype is None:
        prec_out = ord("s") if prec_in in (ord("b"), ord("h")) else prec_in
    else:
        prec_out = _prec(np.empty(0, dtype=out_dtype)) if not _is_torch(X) else _prec(_empty(X, (0,), out_dtype))
    if _is_torch(X):
        import torch

        odt = {ord("s"): torch.float32, ord("d"): torch.float64, ord("b"): torch.bfloat16, ord("h"): torch.float16}[prec_out]
    else:
        odt = {ord("s"): np.float32, ord("d"): np.float64, ord("h"): np.float16}.get(prec_out, X.dtype)
    Y = _empty(X, conv_out_shape(tuple(X.shape), k_shape, strides, pads, dilations, c_out), odt)
    call("docc_b200_conv", prec_in, prec_out, sr, _arr(X.shape), _arr(k_shape), _arr(strides), _arr(pads), _arr(dilations),
         c_out, int(group), _ptr(X), _ptr(W), _ptr(bias), _ptr(Y), flags)
    return Y


def attention(Q, K, V, scale=None, causal=False, flags=0):
    """softmax(scale * Q K^T [+ causal mask]) V on contiguous [B,H,S,D] arrays."""
    flags |= _kind(Q, K, V)
    B, H, Sq, D = Q.shape
    Skv = K.shape[2]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    O = _empty(Q, Q.shape)
    null = ctypes.cast(None, ctypes.POINTER(_i64))
    call("docc_b200_attention", _prec(Q), B, H, Sq, Skv, D, float(scale), int(bool(causal)), _ptr(Q), null, _ptr(K), null,
         _ptr(V), null, _ptr(O), null, flags)
    return O


def layernorm(X, gamma=None, beta=None, eps=1e-5, flags=0):
    flags |= _kind(X, gamma, beta)
    cols = X.shape[-1]
    rows = int(np.prod(X.shape[:-1]))
    Y = _empty(X, X.shape)
    call("docc_b200_layernorm", _prec(X), rows, cols, _ptr(X), _ptr(gamma), _ptr(beta), float(eps), _ptr(Y), flags)
    return Y


def bias_act(X, scale=1.0, bias=None, act=ACT_NONE, residual=None, flags=0):
    flags |= _kind(X, bias, residual)
    cols = X.shape[-1] if X.ndim else 1
    rows = int(np.prod(X.shape[:-1])) if X.ndim else 1
    Y = _empty(X, X.shape)
    call("docc_b200_bias_act", _prec(X), rows, cols, _ptr(X), float(scale), _ptr(bias), int(act), _ptr(residual), _ptr(Y), flags)
    return Y


def binary(op, A, B, flags=0):
    flags |= _kind(A, B)
    if tuple(A.shape) != tuple(B.shape):
        raise ValueError("binary: shapes differ (broadcast with numpy/torch first)")
    Y = _empty(A, A.shape)
    n = int(np.prod(A.shape)) if A.ndim else 1
    call("docc_b200_binary", int(op), _prec(A), n, _ptr(A), _ptr(B), _ptr(Y), flags)
    return Y


def cast(X, dtype, flags=0):
    flags |= _kind(X)
    Y = _empty(X, X.shape, dtype)
    n = int(np.prod(X.shape)) if X.ndim else 1
    call("docc_b200_cast", _prec(X), _prec(Y), n, _ptr(X), _ptr(Y), flags)
    return Y


BLOCK_FIELDS = ("ln1_g", "ln1_b", "w_qkv", "b_qkv", "w_o", "b_o", "ln2_g", "ln2_b", "w_1", "b_1", "w_2", "b_2")


def transformer_block(x, params, n_heads, eps=1e-5, flags=0):
    """Pre-LN encoder block; ``params`` maps the ``docc_b200_block_params`` field names to arrays."""
    tensors = [params.get(f) for f in BLOCK_FIELDS]
    flags |= _kind(x, *tensors)
    Bn, S, d = x.shape
    bp = BlockParams()
    bp.batch, bp.seq, bp.d_model, bp.n_heads, bp.d_ff, bp.eps = Bn, S, d, int(n_heads), params["w_1"].shape[0], float(eps)
    for f, t in zip(BLOCK_FIELDS, tensors):
        setattr(bp, f, _ptr(t).value or 0)
    y = _empty(x, x.shape)
    call("docc_b200_transformer_block", _prec(x), ctypes.byref(bp), _ptr(x), _ptr(y), flags)
    return y
