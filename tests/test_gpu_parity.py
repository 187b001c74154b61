"""Parity of the CUDA path (through the C ABI) with the CPU oracle on seeded inputs, and with
the committed golden fixtures. Tolerances are the stated ones: <= 1e-12 relative for fp64,
<= 1e-4 relative for fp32 paths, <= 2e-2 relative against an fp32 reference for 16-bit inputs
with fp32 accumulation; relative error is norm-wise, max|d| / max|ref|."""
import numpy as np
import pytest
import torch

import oracle
from conftest import relerr
from docc_b200 import _lib, ops

pytestmark = pytest.mark.gpu

TOL_F64, TOL_F32, TOL_16 = 1e-12, 1e-4, 2e-2


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    ops.sync()
    torch.cuda.synchronize()
    return t.float().cpu().numpy() if t.dtype in (torch.bfloat16, torch.float16) else t.cpu().numpy()


# ---- golden fixtures through both pointer flavours ---------------------------------------------
@pytest.mark.parametrize("name,tol", [("gemm_f64", TOL_F64), ("gemm_f32", TOL_F32), ("gemm_f32_8", TOL_F32), ("gemm_rect", TOL_F64)])
def test_gemm_golden(rt, golden, name, tol):
    a, b, y = golden[f"{name}_a"], golden[f"{name}_b"], golden[f"{name}_y"]
    assert relerr(ops.gemm(a, b), y) <= tol  # host pointers
    assert relerr(host(ops.gemm(dev(a), dev(b))), y) <= tol  # device pointers


def test_matmul_batched_golden(rt, golden):
    y = ops.matmul(golden["matmul_batched_a"], golden["matmul_batched_b"])
    assert relerr(y, golden["matmul_batched_y"]) <= TOL_F64


def test_softmax_golden(rt, golden):
    x = golden["softmax_x"]
    assert relerr(ops.softmax(x, [0]), golden["softmax_axis0_y"]) <= TOL_F64
    assert relerr(ops.softmax(x), golden["softmax_all_y"]) <= TOL_F64
    assert relerr(ops.softmax(golden["softmax_f32_x"], [-1]), golden["softmax_f32_y"]) <= TOL_F32


@pytest.mark.parametrize("name", ["conv3x3", "conv1x1", "conv5x5", "conv_s2", "conv_b4"])
def test_conv_golden(rt, golden, name):
    s = int(golden[f"{name}_stride"])
    y = ops.conv(golden[f"{name}_x"], golden[f"{name}_w"], strides=[s, s])
    assert relerr(y, golden[f"{name}_y"]) <= TOL_F32


def test_unpinned_golden(rt, golden):
    g = golden
    y = ops.conv(g["unpinned_conv_pad_x"], g["unpinned_conv_pad_w"], g["unpinned_conv_pad_b"], pads=[1, 1, 1, 1])
    assert relerr(y, g["unpinned_conv_pad_y"]) <= TOL_F32
    q, k, v = g["unpinned_attn_q"], g["unpinned_attn_k"], g["unpinned_attn_v"]
    assert relerr(ops.attention(q, k, v), g["unpinned_attn_y"]) <= TOL_F32
    assert relerr(ops.attention(q, k, v, causal=True), g["unpinned_attn_causal_y"]) <= TOL_F32
    assert relerr(ops.layernorm(g["unpinned_ln_x"], g["unpinned_ln_g"], g["unpinned_ln_b"]), g["unpinned_ln_y"]) <= TOL_F32
    assert relerr(ops.bias_act(g["unpinned_ln_x"], act=ops.ACT_GELU_ERF), g["unpinned_gelu_y"]) <= TOL_F32


# ---- GEMM ------------------------------------------------------------------------------------------
def test_gemm_fp64_config1(rt):
    rng = np.random.RandomState(0)
    a, b = rng.rand(1000, 1000), rng.rand(1000, 1000)
    got = host(ops.gemm(dev(a), dev(b)))
    assert relerr(got, a @ b) <= TOL_F64  # OpenBLAS stands in for the reference's -lblas
    sub = oracle.gemm(a[:64], b)  # oracle loop order on a slab the triple loop finishes quickly
    assert relerr(got[:64], sub) <= TOL_F64


@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (3, 5, 7), (64, 64, 64), (65, 63, 17), (129, 130, 131), (200, 100, 300)])
@pytest.mark.parametrize("dtype,tol", [(np.float64, TOL_F64), (np.float32, TOL_F32)])
def test_gemm_shapes(rt, m, n, k, dtype, tol):
    rng = np.random.RandomState(m * 1000 + n * 10 + k)
    a, b = rng.randn(m, k).astype(dtype), rng.randn(k, n).astype(dtype)
    c0 = rng.randn(m, n).astype(dtype)
    c = dev(c0.copy())
    ops.gemm(dev(a), dev(b), c, alpha=0.75, beta=-1.5)
    ref = c0.copy()
    oracle.gemm(a, b, ref, alpha=0.75, beta=-1.5)
    assert relerr(host(c), ref) <= tol


@pytest.mark.parametrize("transa,transb", [(False, False), (True, False), (False, True), (True, True)])
@pytest.mark.parametrize("layout", [ops.ROW_MAJOR, ops.COL_MAJOR])
@pytest.mark.parametrize("dtype,tol", [(np.float64, TOL_F64), (np.float32, TOL_F32)])
def test_gemm_transposes_and_layouts(rt, transa, transb, layout, dtype, tol):
    rng = np.random.RandomState(7)
    m, n, k = 72, 40, 56
    A = rng.randn(*((k, m) if transa else (m, k))).astype(dtype)
    B = rng.randn(*((n, k) if transb else (k, n))).astype(dtype)
    ref = ((A.T if transa else A).astype(np.float64) @ (B.T if transb else B).astype(np.float64))
    if layout == ops.ROW_MAJOR:
        got = host(ops.gemm(dev(A), dev(B), transa=transa, transb=transb))
    else:
        got = host(ops.gemm(dev(np.ascontiguousarray(A.T)), dev(np.ascontiguousarray(B.T)), transa=transa, transb=transb,
                            layout=layout)).T
    assert relerr(got, ref) <= tol


def test_gemm_fp32_large_tensor_core_path(rt):
    # fp32 GEMM runs as three bf16 tcgen05 passes; 1e-4 is the fp32 budget
    rng = np.random.RandomState(11)
    a, b = rng.randn(512, 1024).astype(np.float32), rng.randn(1024, 768).astype(np.float32)
    got = host(ops.gemm(dev(a), dev(b)))
    ref = a.astype(np.float64) @ b.astype(np.float64)
    assert relerr(got, ref) <= TOL_F32
    exact = host(ops.gemm(dev(a), dev(b), flags=ops.FLAG_FP32_EXACT))
    assert relerr(exact, ref) <= 1e-5
    sub = oracle.gemm(a[:16], b)
    assert relerr(got[:16], sub) <= TOL_F32


def test_gemm_bf16(rt):
    torch.manual_seed(5)
    a = torch.randn(300, 256, device="cuda").bfloat16()
    b = torch.randn(256, 200, device="cuda").bfloat16()
    got = host(ops.gemm(a, b))
    ref = a.float().cpu().numpy().astype(np.float64) @ b.float().cpu().numpy().astype(np.float64)
    assert relerr(got, ref) <= TOL_16
    bt = b.t().contiguous()
    got_t = host(ops.gemm(a, bt, transb=True))
    assert relerr(got_t, ref) <= TOL_16


# Problems large enough for the CTA-pair kernel (K-major operands, at least 74 tiles of 256x256): ragged M and N,
# the 256x512 tile of a long K, fp32 as three passes, and the fused epilogue. The reference is torch in fp64 on the
# GPU (the oracle's scalar loops would take minutes at these sizes); a row block is also checked against the oracle.
@pytest.mark.parametrize("m,n,k", [(2500, 2700, 1000), (2560, 2048, 512), (4096, 4352, 4096)])
def test_gemm_bf16_cta_pair_paths(rt, m, n, k):
    torch.manual_seed(21)
    a = torch.randn(m, k, device="cuda").bfloat16()
    bt = torch.randn(n, k, device="cuda").bfloat16()
    got = ops.gemm(a, bt, transb=True)
    ops.sync()
    ref = a.double() @ bt.double().t()
    assert ((got.double() - ref).abs().max() / ref.abs().max()).item() <= TOL_16
    sub = oracle.gemm(a[-8:].float().cpu().numpy(), bt.float().cpu().numpy(), transb=True)
    assert relerr(got[-8:].float().cpu().numpy(), sub) <= TOL_16


def test_gemm_fp32_and_linear_cta_pair_paths(rt):
    torch.manual_seed(22)
    a = torch.randn(2304, 1536, device="cuda")
    bt = torch.randn(2816, 1536, device="cuda")
    got = ops.gemm(a, bt, transb=True)
    ops.sync()
    ref = a.double() @ bt.double().t()
    assert ((got.double() - ref).abs().max() / ref.abs().max()).item() <= TOL_F32
    x = torch.randn(2048, 1024, device="cuda").bfloat16()
    w = torch.randn(2560, 1024, device="cuda").bfloat16() / 32
    bias = torch.randn(2560, device="cuda")
    res = torch.randn(2048, 2560, device="cuda").bfloat16()
    y = ops.linear(x, w, bias, ops.ACT_GELU_ERF, res)
    ops.sync()
    ref = torch.nn.functional.gelu(x.double() @ w.double().t() + bias.double()) + res.double()
    assert ((y.double() - ref).abs().max() / ref.abs().max()).item() <= TOL_16
    with pytest.raises(TypeError):
        ops.linear(x, w, bias.bfloat16())  # the ABI reads the bias of a 16-bit layer as fp32


def test_gemm_beta_zero_ignores_nan_in_c(rt):
    a = torch.ones(70, 70, device="cuda", dtype=torch.float64)
    c = torch.full((70, 70), float("nan"), device="cuda", dtype=torch.float64)
    ops.gemm(a, a, c, beta=0.0)
    assert np.all(host(c) == 70.0)


def test_matmul_batched_and_broadcast(rt):
    rng = np.random.RandomState(9)
    a, b = rng.randn(3, 40, 24), rng.randn(24, 16)
    assert relerr(host(ops.matmul(dev(a), dev(b))), oracle.matmul(a, b)) <= TOL_F64
    a32, b32 = rng.randn(4, 130, 64).astype(np.float32), rng.randn(4, 64, 72).astype(np.float32)
    assert relerr(host(ops.matmul(dev(a32), dev(b32))), oracle.matmul(a32, b32)) <= TOL_F32


def test_linear_fused_epilogue(rt):
    rng = np.random.RandomState(10)
    x, w = rng.randn(200, 96).astype(np.float32), rng.randn(160, 96).astype(np.float32)
    bias, res = rng.randn(160).astype(np.float32), rng.randn(200, 160).astype(np.float32)
    ref = oracle.linear(x, w, bias, oracle.ACT_GELU_ERF, res)
    got = host(ops.linear(dev(x), dev(w), dev(bias), ops.ACT_GELU_ERF, dev(res)))
    assert relerr(got, ref) <= TOL_F32
    assert relerr(ops.linear(x, w, bias, ops.ACT_GELU_ERF, res), ref) <= TOL_F32  # host pointers


def test_linear_fp64_bias_is_read_as_fp64(rt):
    rng = np.random.RandomState(14)
    x, w = rng.randn(50, 40), rng.randn(30, 40)
    bias, res = rng.randn(30), rng.randn(50, 30)
    ref = x @ w.T + bias + res
    assert relerr(host(ops.linear(dev(x), dev(w), dev(bias), residual=dev(res))), ref) <= TOL_F64
    assert relerr(ops.linear(x, w, bias, residual=res), ref) <= TOL_F64  # host pointers: staged as 8-byte elements
    with pytest.raises(TypeError):
        ops.linear(x, w, bias.astype(np.float32))
    with pytest.raises(ValueError):
        ops.linear(x, w, bias, residual=res[:1])  # a residual that would have to broadcast
    with pytest.raises(ValueError):
        ops.linear(x, w[:, :39], bias)


# ---- softmax / reductions ----------------------------------------------------------------------------
def test_softmax_config2(rt):
    torch.manual_seed(1)
    x = 3 * torch.randn(8192, 4096)
    y = host(ops.softmax(x.cuda(), [-1]))
    sample = np.r_[0:64, 4000:4064, 8128:8192]  # oracle on a slab of rows; every row is independent
    assert relerr(y[sample], oracle.softmax(x.numpy()[sample], [-1])) <= TOL_F32
    # size-independent properties on the full tensor: rows sum to one, entries in [0,1], order preserved
    assert np.allclose(y.sum(axis=1, dtype=np.float64), 1.0, atol=1e-5)
    assert y.min() >= 0.0 and y.max() <= 1.0
    assert np.array_equal(y.argmax(axis=1), x.numpy().argmax(axis=1))
    # softmax is shift invariant
    y2 = host(ops.softmax((x + 7.0).cuda(), [-1]))
    assert relerr(y2, y) <= TOL_F32


@pytest.mark.parametrize("shape,axes", [((10, 10), [0]), ((10, 10), [1]), ((10, 10), [0, 1]), ((4, 5, 6), [1]),
                                        ((4, 5, 6), [0, 2]), ((3, 1000), [-1]), ((7, 33), [-1]), ((5, 4096), [1]),
                                        ((2, 40000), [1]), ((300, 17, 3), [1]), ((2, 3, 4, 5), [2, 3]), ((1, 1), [0])])
@pytest.mark.parametrize("dtype,tol", [(np.float32, TOL_F32), (np.float64, TOL_F64)])
def test_softmax_shapes(rt, shape, axes, dtype, tol):
    x = (np.random.RandomState(len(shape) + sum(shape)).randn(*shape) * 3).astype(dtype)
    ref = oracle.softmax(x, axes)
    assert relerr(host(ops.softmax(dev(x), axes)), ref) <= tol
    assert relerr(ops.softmax(x, axes), ref) <= tol


def test_softmax_edge_cases(rt):
    assert ops.softmax(np.zeros((0, 8), dtype=np.float32), [1]).shape == (0, 8)
    x = np.array([[1e30, -1e30, 0.0, 1e30]], dtype=np.float32)
    assert np.allclose(ops.softmax(x, [1]), [[0.5, 0.0, 0.0, 0.5]])
    big = np.full((2, 64), 1e4, dtype=np.float32)
    assert np.allclose(ops.softmax(big, [1]), 1.0 / 64)
    with pytest.raises(_lib.DoccB200Error) as e:
        ops.softmax(np.zeros((2, 2), dtype=np.float32), [2])
    assert e.value.status == 1  # axis out of bounds, as SoftmaxNode::expand throws


def test_softmax_16bit(rt):
    torch.manual_seed(8)
    x = (torch.randn(64, 512) * 3).bfloat16()
    ref = torch.softmax(x.float(), dim=-1).numpy()
    assert relerr(host(ops.softmax(x.cuda(), [-1])), ref) <= TOL_16


@pytest.mark.parametrize("op", [ops.RED_SUM, ops.RED_MAX, ops.RED_MIN, ops.RED_MEAN, ops.RED_STD])
def test_reduce(rt, op):
    x = np.random.RandomState(2).randn(6, 50, 7)
    for axes in ([0], [1], [2], [0, 2], [0, 1, 2]):
        assert relerr(host(ops.reduce(op, dev(x), axes)), oracle.reduce(op, x, axes)) <= 1e-11
    x32 = np.random.RandomState(3).randn(40, 3000).astype(np.float32)
    assert relerr(host(ops.reduce(op, dev(x32), [1])), oracle.reduce(op, x32, [1])) <= TOL_F32


# ---- conv ----------------------------------------------------------------------------------------------
@pytest.mark.parametrize("stride,pad,dil,groups", [(1, 0, 1, 1), (1, 1, 1, 1), (2, 1, 1, 1), (1, 2, 2, 1), (1, 1, 1, 2)])
def test_conv2d_variants(rt, stride, pad, dil, groups):
    rng = np.random.RandomState(2)
    x, w = rng.randn(2, 4, 9, 10).astype(np.float32), rng.randn(6, 4 // groups, 3, 3).astype(np.float32)
    b = rng.randn(6).astype(np.float32)
    kw = dict(strides=[stride] * 2, pads=[pad] * 4, dilations=[dil] * 2, group=groups)
    ref = oracle.conv(x, w, b, **kw)
    assert relerr(host(ops.conv(dev(x), dev(w), dev(b), **kw)), ref) <= TOL_F32
    assert relerr(ops.conv(x, w, b, **kw), ref) <= TOL_F32


def test_conv1d_conv3d_fp64(rt):
    rng = np.random.RandomState(5)
    x, w = rng.randn(2, 3, 11), rng.randn(4, 3, 3)
    assert relerr(ops.conv(x, w, pads=[1, 1]), oracle.conv(x, w, pads=[1, 1])) <= TOL_F64
    x, w = rng.randn(1, 2, 5, 6, 7), rng.randn(3, 2, 2, 3, 3)
    assert relerr(ops.conv(x, w), oracle.conv(x, w)) <= TOL_F64


def test_conv_config3_shape_reduced_batch(rt):
    # BASELINE config 3 with batch 2 (the oracle's 576-term scalar loop is slow): [2,64,56,56] * [128,64,3,3], s1 p1
    torch.manual_seed(2)
    x = torch.randn(2, 64, 56, 56)
    w = torch.nn.init.kaiming_normal_(torch.empty(128, 64, 3, 3))
    b = torch.zeros(128)
    ref = oracle.conv(x.numpy(), w.numpy(), b.numpy(), pads=[1, 1, 1, 1])
    got = host(ops.conv(x.cuda(), w.cuda(), b.cuda(), pads=[1, 1, 1, 1]))
    assert relerr(got, ref) <= TOL_F32
    xb, wb = x.bfloat16(), w.bfloat16()
    ref16 = oracle.conv(xb.float().numpy(), wb.float().numpy(), b.numpy(), pads=[1, 1, 1, 1])
    got16 = host(ops.conv(xb.cuda(), wb.cuda(), b.cuda(), pads=[1, 1, 1, 1]))
    assert got16.dtype == np.float32
    assert relerr(got16, ref16) <= TOL_16


# Tensor-core convolution geometries (C_in a multiple of 64): narrow images take the kernel that loads each
# tile's input neighbourhood once (ragged widths, partial channel tiles, 1x1 to 7x7 filters, two channel
# blocks), images wider than 62 output pixels the per-tap kernel.
@pytest.mark.parametrize("n,c,h,w,co,k,pad", [
    (2, 64, 20, 30, 96, 3, 1),    # rows not a multiple of 16 bytes: direct stores; C_out below one tile
    (1, 128, 9, 62, 130, 3, 1),   # widest narrow case, two channel blocks, second channel tile nearly empty
    (1, 64, 40, 80, 64, 3, 1),    # wide image
    (2, 64, 12, 12, 32, 5, 2),
    (1, 64, 16, 16, 64, 1, 0),
    (1, 64, 10, 24, 64, 7, 3),
    (1, 64, 7, 7, 128, 3, 0),     # no padding, output 5x5
])
def test_conv_tensor_core_geometries(rt, n, c, h, w, co, k, pad):
    torch.manual_seed(7)
    x = torch.randn(n, c, h, w)
    wt = torch.randn(co, c, k, k) / (c * k * k) ** 0.5
    b = torch.randn(co)
    pads = [pad, pad, pad, pad]
    ref = oracle.conv(x.numpy(), wt.numpy(), b.numpy(), pads=pads)
    got = host(ops.conv(x.cuda(), wt.cuda(), b.cuda(), pads=pads))
    assert got.shape == ref.shape
    assert relerr(got, ref) <= TOL_F32
    xb, wb = x.bfloat16(), wt.bfloat16()
    ref16 = oracle.conv(xb.float().numpy(), wb.float().numpy(), b.numpy(), pads=pads)
    got16 = host(ops.conv(xb.cuda(), wb.cuda(), b.cuda(), pads=pads))
    assert relerr(got16, ref16) <= TOL_16


# 16-bit NCHW inputs of narrow images whose rows are a multiple of 16 bytes are read in place by the fused kernel (TMA
# staging, transposer warps fill the tensor-core layout); other widths and unaligned bases keep the path through the
# re-laid copy. Both must agree with the oracle, for bf16 and fp16, with tiles that start and end inside an image and
# images whose rows span CTAs.
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("n,c,h,w,co,k,pad", [
    (3, 64, 56, 56, 128, 3, 1),   # config 3 geometry, three images
    (5, 64, 13, 22, 40, 3, 1),    # few rows per image: tiles cut at image ends
    (2, 128, 17, 31, 64, 3, 1),   # odd width: re-laid copy
    (1, 64, 30, 58, 64, 3, 0),    # no padding
    (2, 64, 9, 16, 64, 3, 2),     # padding wider than the filter needs
    (160, 64, 6, 8, 16, 3, 1),    # many small images: more tiles than SMs
    (2, 128, 20, 48, 130, 3, 1),  # two channel blocks, two channel tiles, columns 48..55 of the box outside the image
    (1, 64, 9, 64, 64, 1, 0),     # no padding, full-width box
    (2, 64, 14, 40, 48, 5, 2),    # 5x5 filter
    (1, 64, 12, 24, 64, 7, 3),    # 7x7 filter: shallow rings
    (1, 64, 30, 56, 128, 3, 1),
    (8, 64, 1000, 16, 32, 3, 1),  # tall images: more tiles per CTA than its precomputed tile list holds (resident weights)
    (4, 128, 1000, 16, 32, 3, 1), # the same with streamed weights (two channel blocks)
])
def test_conv_16bit_nchw_in_place(rt, dtype, n, c, h, w, co, k, pad):
    torch.manual_seed(11)
    x = torch.randn(n, c, h, w).to(dtype)
    wt = (torch.randn(co, c, k, k) / (c * k * k) ** 0.5).to(dtype)
    b = torch.randn(co)
    pads = [pad, pad, pad, pad]
    # the tensor cores run both 16-bit types in bf16, so the fp16 reference rounds its operands the same way
    xr, wr = (t_.bfloat16().float().numpy() for t_ in (x, wt))
    ref = oracle.conv(xr, wr, b.numpy(), pads=pads)
    got = host(ops.conv(x.cuda(), wt.cuda(), b.cuda(), pads=pads))
    assert got.shape == ref.shape
    assert relerr(got, ref) <= (1e-5 if dtype == torch.bfloat16 else TOL_16)
    # an input that starts 2 bytes off a 4-byte boundary cannot be read in pixel pairs: same result through the copy
    flat = torch.empty(x.numel() + 1, dtype=dtype, device="cuda")
    flat[1:] = x.cuda().reshape(-1)
    got_off = host(ops.conv(flat[1:].view(n, c, h, w), wt.cuda(), b.cuda(), pads=pads))
    assert relerr(got_off, ref) <= (1e-5 if dtype == torch.bfloat16 else TOL_16)


def test_conv_linearity_full_config3(rt):
    # size-independent property at the full config: conv(x1 + x2) == conv(x1) + conv(x2)
    torch.manual_seed(2)
    x1, x2 = torch.randn(32, 64, 56, 56, device="cuda"), torch.randn(32, 64, 56, 56, device="cuda")
    w = torch.nn.init.kaiming_normal_(torch.empty(128, 64, 3, 3)).cuda()
    p = dict(pads=[1, 1, 1, 1])
    y12 = host(ops.conv(x1 + x2, w, **p))
    ysum = host(ops.conv(x1, w, **p)) + host(ops.conv(x2, w, **p))
    assert relerr(y12, ysum) <= TOL_F32


# ---- attention ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", [(1, 2, 33, 16), (2, 3, 128, 64), (1, 2, 200, 128), (1, 1, 7, 40)])
def test_attention_fp32(rt, shape, causal):
    rng = np.random.RandomState(3)
    q, k, v = (rng.randn(*shape).astype(np.float32) for _ in range(3))
    ref = oracle.attention(q, k, v, causal=causal)
    assert relerr(host(ops.attention(dev(q), dev(k), dev(v), causal=causal)), ref) <= TOL_F32


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("B,H,S,D", [(1, 2, 256, 128), (2, 2, 384, 64), (1, 1, 130, 128), (1, 2, 77, 64)])
def test_attention_bf16(rt, B, H, S, D, causal):
    torch.manual_seed(3)
    q, k, v = (torch.randn(B, H, S, D).bfloat16() for _ in range(3))
    ref = oracle.attention(q.float().numpy(), k.float().numpy(), v.float().numpy(), causal=causal)
    got = host(ops.attention(q.cuda(), k.cuda(), v.cuda(), causal=causal))
    assert relerr(got, ref) <= TOL_16


# fp32 attention with head_dim 64 runs on the tensor cores as bf16 hi/lo planes (three products per contraction).
# Longer than one 128-row tile it takes the two-tile kernels: persistent without a mask (B*H*ceil(S/256) above the
# SM count makes every CTA walk several items), one CTA per tile pair with a causal mask. These are the kernels the
# fp32 encoder block of BASELINE config 5 (16 heads of 64, sequence 512) launches.
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("B,H,S", [(1, 2, 256), (2, 3, 384), (6, 16, 512), (1, 2, 300), (1, 1, 129)])
def test_attention_fp32_head64_multi_tile(rt, B, H, S, causal):
    rng = np.random.RandomState(S + B)
    q, k, v = (rng.randn(B, H, S, 64).astype(np.float32) for _ in range(3))
    ref = oracle.attention(q, k, v, causal=causal)
    got = host(ops.attention(dev(q), dev(k), dev(v), causal=causal))
    assert relerr(got, ref) <= TOL_F32


@pytest.mark.parametrize("causal", [False, True])
def test_attention_fp32_cross_lengths(rt, causal):
    # Sq != Skv: the causal mask aligns the last query with the last key
    rng = np.random.RandomState(17)
    q = rng.randn(2, 2, 256, 64).astype(np.float32)
    k, v = (rng.randn(2, 2, 448, 64).astype(np.float32) for _ in range(2))
    ref = oracle.attention(q, k, v, causal=causal)
    assert relerr(host(ops.attention(dev(q), dev(k), dev(v), causal=causal)), ref) <= TOL_F32


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("B,H,S,D", [(5, 16, 512, 64), (3, 20, 640, 128), (9, 16, 768, 64)])
def test_attention_bf16_persistent_walk(rt, B, H, S, D, causal):
    # more (batch, head, tile pair) items than SMs: the persistent kernel's hand-over between items; under a causal mask the
    # items are dealt heaviest first in alternating direction (two and three rounds here, odd tile counts included)
    torch.manual_seed(S)
    q, k, v = (torch.randn(B, H, S, D).bfloat16() for _ in range(3))
    ref = oracle.attention(q.float().numpy(), k.float().numpy(), v.float().numpy(), causal=causal)
    got = host(ops.attention(q.cuda(), k.cuda(), v.cuda(), causal=causal))
    assert relerr(got, ref) <= TOL_16


def test_attention_config4_properties(rt):
    # full config 4; the oracle checks two (batch, head) slices, the rest through properties
    torch.manual_seed(3)
    q, k, v = (torch.randn(8, 16, 2048, 128).bfloat16().cuda() for _ in range(3))
    for causal in (False, True):
        o = ops.attention(q, k, v, causal=causal)
        got = host(o)
        for (b, h) in ((0, 0), (7, 15)):
            sl = lambda t: t[b:b + 1, h:h + 1, :256 if causal else 2048].float().cpu().numpy()
            ref = oracle.attention(sl(q)[:, :, :256], sl(k), sl(v), causal=causal) if causal else oracle.attention(
                sl(q)[:, :, :64], sl(k), sl(v))
            n = ref.shape[2]
            assert relerr(got[b:b + 1, h:h + 1, :n], ref) <= TOL_16
        # rows of P sum to one => with V == 1 the output is 1
        ones = torch.ones_like(v)
        assert np.allclose(host(ops.attention(q, k, ones, causal=causal)), 1.0, atol=2e-2)
    # causal: the first query sees only the first key
    o = host(ops.attention(q, k, v, causal=True))
    assert relerr(o[:, :, 0], v[:, :, 0].float().cpu().numpy()) <= TOL_16


# ---- LayerNorm / element-wise ----------------------------------------------------------------------------------
@pytest.mark.parametrize("rows,cols", [(5, 48), (64, 1024), (3, 1000), (2, 8192), (4, 17)])
def test_layernorm(rt, rows, cols):
    rng = np.random.RandomState(rows + cols)
    x = (rng.randn(rows, cols) * 2 + 1).astype(np.float32)
    g, b = rng.rand(cols).astype(np.float32) + 0.5, rng.randn(cols).astype(np.float32)
    ref = oracle.layernorm(x, g, b)
    assert relerr(host(ops.layernorm(dev(x), dev(g), dev(b))), ref) <= TOL_F32
    assert relerr(ops.layernorm(x), oracle.layernorm(x)) <= TOL_F32


# Many rows take the persistent kernel that stages rows through shared memory with bulk copies (a ring per warp):
# row counts that are not a multiple of the warps in the grid, widths that leave lanes idle, with and without parameters.
@pytest.mark.parametrize("rows,cols,dtype", [(16384, 1024, torch.bfloat16), (5000, 1024, torch.float32), (4801, 768, torch.bfloat16),
                                             (6007, 2048, torch.bfloat16), (9000, 520, torch.float32), (4736, 256, torch.float16)])
def test_layernorm_many_rows(rt, rows, cols, dtype):
    torch.manual_seed(rows)
    x = (torch.randn(rows, cols) * 2 + 0.5).to(dtype)
    g, b = torch.rand(cols) + 0.5, torch.randn(cols)
    tol = TOL_F32 if dtype == torch.float32 else TOL_16
    ref = torch.nn.functional.layer_norm(x.double(), (cols,), g.double(), b.double()).numpy()
    got = host(ops.layernorm(x.cuda(), g.cuda(), b.cuda()))
    assert relerr(got, ref) <= tol
    sl = slice(rows - 40, rows)  # the oracle on the last rows (the ones the ring handles in its final, partial round)
    if dtype != torch.float16:
        ref_o = oracle.layernorm(x[sl].float().numpy(), g.numpy(), b.numpy())
        assert relerr(got[sl], ref_o) <= tol
    assert relerr(host(ops.layernorm(x.cuda())), torch.nn.functional.layer_norm(x.double(), (cols,)).numpy()) <= tol


def test_layernorm_bf16(rt):
    torch.manual_seed(6)
    x = torch.randn(32, 1024).bfloat16()
    g, b = torch.rand(1024) + 0.5, torch.randn(1024)
    ref = torch.nn.functional.layer_norm(x.float(), (1024,), g, b).numpy()
    assert relerr(host(ops.layernorm(x.cuda(), g.cuda(), b.cuda())), ref) <= TOL_16


@pytest.mark.parametrize("act", range(9))
def test_bias_act(rt, act):
    rng = np.random.RandomState(act)
    x = rng.rand(37, 64).astype(np.float32) + 0.1  # positive: sqrt is in the list
    bias, res = rng.rand(64).astype(np.float32), rng.randn(37, 64).astype(np.float32)
    ref = oracle.bias_act(x, 0.5, bias, act, res)
    assert relerr(host(ops.bias_act(dev(x), 0.5, dev(bias), act, dev(res))), ref) <= TOL_F32
    x3 = rng.rand(5, 7).astype(np.float32)
    assert relerr(ops.bias_act(x3, act=act), oracle.bias_act(x3, act=act)) <= TOL_F32


def test_binary_and_cast(rt):
    rng = np.random.RandomState(4)
    a, b = rng.randn(1000).astype(np.float32), rng.rand(1000).astype(np.float32) + 0.5
    for op in range(6):
        assert np.array_equal(ops.binary(op, a, b), oracle.binary(op, a, b))  # single IEEE ops: bit-exact
    assert np.array_equal(ops.cast(a, np.float64), a.astype(np.float64))
    assert np.array_equal(ops.cast(a.astype(np.float64), np.float32), a)
    import ml_dtypes

    got = host(ops.cast(dev(a), torch.bfloat16))
    assert np.array_equal(got, a.astype(ml_dtypes.bfloat16).astype(np.float32))


# ---- transformer block -----------------------------------------------------------------------------------------
def make_block(d, dff, seed=4):
    torch.manual_seed(seed)
    p = {"ln1_g": torch.ones(d), "ln1_b": torch.zeros(d), "ln2_g": torch.ones(d), "ln2_b": torch.zeros(d)}
    for name, shape in (("w_qkv", (3 * d, d)), ("w_o", (d, d)), ("w_1", (dff, d)), ("w_2", (d, dff))):
        p[name] = torch.nn.init.xavier_uniform_(torch.empty(*shape))
    for name, n in (("b_qkv", 3 * d), ("b_o", d), ("b_1", dff), ("b_2", d)):
        p[name] = torch.zeros(n)
    return p


def test_transformer_block_fp32(rt):
    d, heads, dff = 128, 2, 256
    p = make_block(d, dff)
    x = torch.randn(2, 48, d)
    ref = oracle.transformer_block(x.numpy(), {k: v.numpy() for k, v in p.items()}, heads)
    got = host(ops.transformer_block(x.cuda(), {k: v.cuda() for k, v in p.items()}, heads))
    assert relerr(got, ref) <= TOL_F32
    got_h = ops.transformer_block(x.numpy(), {k: v.numpy() for k, v in p.items()}, heads)
    assert relerr(got_h, ref) <= TOL_F32


@pytest.mark.parametrize("batch,seq", [(40, 128), (12, 448)])
def test_transformer_block_fp32_fused_operand_planes(rt, batch, seq):
    # Enough rows (>= 2 * 16 * SMs) for the LayerNorms to write the next GEMM's bf16 hi / lo planes themselves. With one query
    # tile per head (seq 128) the attention kernel writes plain fp32 and the out-projection splits as usual; with several
    # (seq 448) the persistent kernel writes the out-projection's planes too. Second opinion as for the config-5 tests: the
    # fp64 composition on the device (the oracle's loops would take minutes at these row counts).
    d, heads, dff = 256, 4, 512
    torch.manual_seed(batch)
    p = make_block_nontrivial(d, dff)
    x = torch.randn(batch, seq, d)
    got = host(ops.transformer_block(x.cuda(), {k: v.cuda() for k, v in p.items()}, heads))
    assert relerr(got, torch_block_f64(x, p, heads)) <= TOL_F32
    sub = oracle.transformer_block(x[:1].numpy(), {k: v.numpy() for k, v in p.items()}, heads)  # one sequence through the oracle
    assert relerr(got[:1], sub) <= TOL_F32


def test_transformer_block_bf16(rt):
    d, heads, dff = 256, 4, 512
    p = make_block(d, dff)
    x = torch.randn(2, 128, d)
    ref = oracle.transformer_block(x.numpy(), {k: v.numpy() for k, v in p.items()}, heads)
    small = ("ln1_g", "ln1_b", "ln2_g", "ln2_b", "b_qkv", "b_o", "b_1", "b_2")
    pd = {k: (v.cuda() if k in small else v.bfloat16().cuda()) for k, v in p.items()}
    got = host(ops.transformer_block(x.bfloat16().cuda(), pd, heads))
    assert relerr(got, ref) <= TOL_16


# BASELINE config 5 at its own geometry (d_model 1024, 16 heads of 64, FFN 4096, sequence 512) with a reduced batch:
# same tiles, same attention instantiation (two-tile persistent, head_dim 64; hi/lo planes for fp32) and same fused
# epilogues as the benchmarked block. The oracle composes the block from the restated nodes; torch in fp64 is the
# second opinion on the whole output.
def torch_block_f64(x, p, heads):
    import torch.nn.functional as F

    x = x.double().cuda()  # cuBLAS fp64 on the device: a second opinion, not the oracle
    p = {k: v.double().cuda() for k, v in p.items()}
    Bn, S, d = x.shape
    h1 = F.layer_norm(x, (d,), p["ln1_g"], p["ln1_b"])
    qkv = F.linear(h1, p["w_qkv"], p["b_qkv"]).reshape(Bn, S, 3, heads, d // heads)
    q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))
    a = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(Bn, S, d)
    h = x + F.linear(a, p["w_o"], p["b_o"])
    f = F.gelu(F.linear(F.layer_norm(h, (d,), p["ln2_g"], p["ln2_b"]), p["w_1"], p["b_1"]))
    return (h + F.linear(f, p["w_2"], p["b_2"])).cpu().numpy()


def make_block_nontrivial(d, dff, seed=4):
    # config 5 has zero biases and unit LayerNorm scales; random ones make the bias and LayerNorm paths visible
    p = make_block(d, dff, seed)
    g = torch.Generator().manual_seed(seed + 100)
    for name in ("b_qkv", "b_o", "b_1", "b_2", "ln1_b", "ln2_b"):
        p[name] = torch.randn(p[name].shape, generator=g) * 0.1
    for name in ("ln1_g", "ln2_g"):
        p[name] = torch.rand(p[name].shape, generator=g) + 0.5
    return p


@pytest.mark.parametrize("batch,maker", [(1, make_block), (2, make_block_nontrivial), (10, make_block_nontrivial)])
def test_transformer_block_config5_geometry_fp32(rt, batch, maker):
    d, heads, dff, seq = 1024, 16, 4096, 512
    p = maker(d, dff)
    torch.manual_seed(40 + batch)
    x = torch.randn(batch, seq, d)
    got = host(ops.transformer_block(x.cuda(), {k: v.cuda() for k, v in p.items()}, heads))
    assert relerr(got, torch_block_f64(x, p, heads)) <= TOL_F32
    nb = min(batch, 2)  # sequences are independent: the oracle takes the first two
    ref = oracle.transformer_block(x[:nb].numpy(), {k: v.numpy() for k, v in p.items()}, heads)
    assert relerr(got[:nb], ref) <= TOL_F32


@pytest.mark.parametrize("batch,maker", [(1, make_block), (2, make_block_nontrivial), (10, make_block_nontrivial)])
def test_transformer_block_config5_geometry_bf16(rt, batch, maker):
    d, heads, dff, seq = 1024, 16, 4096, 512
    p = maker(d, dff)
    torch.manual_seed(50 + batch)
    small = ("ln1_g", "ln1_b", "ln2_g", "ln2_b", "b_qkv", "b_o", "b_1", "b_2")
    p16 = {k: (v if k in small else v.bfloat16()) for k, v in p.items()}
    x = torch.randn(batch, seq, d).bfloat16()
    got = host(ops.transformer_block(x.cuda(), {k: v.cuda() for k, v in p16.items()}, heads))
    # the fp32 reference sees the same rounded weights and input
    pf = {k: v.float() for k, v in p16.items()}
    assert relerr(got, torch_block_f64(x.float(), pf, heads)) <= TOL_16
    nb = min(batch, 2)
    ref = oracle.transformer_block(x[:nb].float().numpy(), {k: v.numpy() for k, v in pf.items()}, heads)
    assert relerr(got[:nb], ref) <= TOL_16


# ---- runtime behaviour ---------------------------------------------------------------------------------------------
def test_pool_and_transfers(rt):
    p = _lib._vp()
    _lib.call("docc_b200_malloc", __import__("ctypes").byref(p), 1 << 20)
    src = np.arange(1 << 18, dtype=np.float32)
    dst = np.zeros_like(src)
    _lib.call("docc_b200_h2d", p, src.ctypes.data, src.nbytes)
    _lib.call("docc_b200_d2h", dst.ctypes.data, p, src.nbytes)
    assert np.array_equal(src, dst)
    first = p.value
    _lib.call("docc_b200_free", p)
    q = _lib._vp()
    _lib.call("docc_b200_malloc", __import__("ctypes").byref(q), 1 << 20)
    assert q.value == first  # served from the pool, no new cudaMalloc
    _lib.call("docc_b200_free", q)
    with pytest.raises(_lib.DoccB200Error):
        _lib.call("docc_b200_free", _lib._vp(12345))


def test_alloc_limit_reports_oom_without_touching_the_gpu(rt):
    _lib.call("docc_b200_set_alloc_limit", 1)
    try:
        p = _lib._vp()
        with pytest.raises(_lib.DoccB200Error) as e:
            # a size class no other test allocates, so the pool cannot serve it from a cached block
            _lib.call("docc_b200_malloc", __import__("ctypes").byref(p), (5 << 30) + (6 << 20))
        assert e.value.status == 4
    finally:
        _lib.call("docc_b200_set_alloc_limit", 0)


def test_pool_is_stream_ordered_across_threads(rt):
    # This thread queues a long chain of kernels that keep rewriting a pooled block with 1.0 and frees the block
    # without waiting. Another host thread (its own non-blocking stream) then gets the same block and fills it
    # with 2.0. The pool has to order the second stream after the queued chain on the device: if the fill could
    # overtake the chain, the chain's late writes would put 1.0 back.
    import ctypes
    import threading

    n = 64 << 20  # one 64 MiB block: a size class no other test leaves in the pool
    rows, cols = n // 4 // 4096, 4096
    ones = np.full(n // 4, 1.0, dtype=np.float32)
    twos = torch.full((n // 4,), 2.0).pin_memory()
    p = _lib._vp()
    _lib.call("docc_b200_malloc", ctypes.byref(p), n)
    _lib.call("docc_b200_h2d", p, ones.ctypes.data, n)
    for _ in range(400):  # ~25 us each: about 10 ms of queued work that writes the block
        _lib.call("docc_b200_bias_act", ord("s"), rows, cols, p, 1.0, None, 0, None, p, 0)
    _lib.call("docc_b200_free", p)  # returns at once
    got = {}

    def other_thread():
        torch.cuda.set_device(0)
        ops.init(0)
        q = _lib._vp()
        _lib.call("docc_b200_malloc", ctypes.byref(q), n)
        got["ptr"] = q.value
        _lib.call("docc_b200_h2d", q, twos.data_ptr(), n)
        torch.cuda.synchronize()  # the first thread's chain has finished too
        out = np.empty(n // 4, dtype=np.float32)
        _lib.call("docc_b200_d2h", out.ctypes.data, q, n)
        got["data"] = out
        _lib.call("docc_b200_free", q)

    t = threading.Thread(target=other_thread)
    t.start()
    t.join()
    ops.sync()
    assert got["ptr"] == p.value  # the pool did hand over the block that had just been freed
    assert np.all(got["data"] == 2.0)


def test_set_stream_orders_the_new_stream_after_the_old(rt):
    # an fp32 GEMM keeps bf16 planes of its operands in a per-thread workspace; a second GEMM routed to another
    # stream right away must not rewrite the planes while the first one still reads them
    torch.manual_seed(31)
    a1, b1 = torch.randn(2048, 2048, device="cuda"), torch.randn(2048, 2048, device="cuda")
    a2, b2 = torch.randn(2048, 2048, device="cuda"), torch.randn(2048, 2048, device="cuda")
    torch.cuda.synchronize()
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    try:
        for _ in range(3):
            ops.set_stream(s1.cuda_stream)
            c1 = ops.gemm(a1, b1)
            ops.set_stream(s2.cuda_stream)
            c2 = ops.gemm(a2, b2)
            torch.cuda.synchronize()
            assert ((c1.double() - a1.double() @ b1.double()).abs().max() / 2048 ** 0.5).item() <= 1e-3
            assert ((c2.double() - a2.double() @ b2.double()).abs().max() / 2048 ** 0.5).item() <= 1e-3
    finally:
        ops.set_stream(torch.cuda.current_stream().cuda_stream)


def test_bounded_device_wait_reports_a_timeout_and_the_context_survives(rt):
    # one warp waits ~1e5 clocks (about 50 us) on a barrier nothing arrives at, gives up, and sets the status word
    _lib.call("docc_b200_selftest_wait_timeout", 100000)
    with pytest.raises(_lib.DoccB200Error) as e:
        ops.sync()
    assert e.value.status == 6 and "location code 900" in str(e.value)
    ops.sync()  # reported once, then cleared
    x = torch.randn(64, 256, device="cuda")
    y = ops.softmax(x, [-1])  # the context is still usable
    ops.sync()
    assert relerr(host(y), torch.softmax(x, -1).cpu().numpy()) <= TOL_F32
    with pytest.raises(_lib.DoccB200Error):
        _lib.call("docc_b200_selftest_wait_timeout", 0)


def test_invalid_arguments_are_rejected(rt):
    x = np.zeros((4, 4), dtype=np.float32)
    import ctypes

    one = ctypes.c_float(1.0)
    st = rt.docc_b200_gemm(ord("s"), 101, 111, 111, 4, 4, 4, ctypes.byref(one), x.ctypes.data, 2, x.ctypes.data, 4,
                           ctypes.byref(one), x.ctypes.data, 4, 1)
    assert st == 1 and b"lda" in rt.docc_b200_last_error()
    st = rt.docc_b200_gemm(ord("q"), 101, 111, 111, 4, 4, 4, None, None, 4, None, 4, None, None, 4, 0)
    assert st == 1
    st = rt.docc_b200_softmax(ord("s"), 2, (ctypes.c_int64 * 2)(4, 4), 1, (ctypes.c_int64 * 1)(0), None, None, 0)
    assert st == 1


def test_launch_counter_counts_our_kernels(rt):
    ops.launch_count(reset=True)
    ops.softmax(torch.randn(64, 256, device="cuda"), [-1])
    ops.sync()
    assert ops.launch_count() == 1


def test_concurrent_host_threads(rt):
    # generated code is entered from arbitrary Python threads with the GIL released
    # (compiled_sdfg.py:447): every thread gets its own context and stream, the pool is shared
    import threading

    rng = np.random.RandomState(12)
    jobs = []
    for i in range(4):
        a, b = rng.rand(150 + i, 90), rng.rand(90, 70 + i)
        x = (rng.randn(64, 300 + 16 * i) * 3).astype(np.float32)
        jobs.append((a, b, x))
    results = [None] * len(jobs)

    def worker(i):
        a, b, x = jobs[i]
        out = []
        for _ in range(5):
            out.append((ops.gemm(a, b), ops.softmax(x, [-1])))  # host pointers: staged through the shared pool
        results[i] = out

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(len(jobs))]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    for (a, b, x), outs in zip(jobs, results):
        for c, y in outs:
            assert relerr(c, a @ b) <= TOL_F64
            assert relerr(y, oracle.softmax(x, [-1])) <= TOL_F32


def test_device_array_keeps_intermediates_on_the_device(rt):
    rng = np.random.RandomState(13)
    a, b = rng.rand(40, 30), rng.rand(30, 20)
    da, db = ops.DeviceArray.from_numpy(a), ops.DeviceArray.from_numpy(b)
    dc = ops.gemm(da, db)
    dy = ops.softmax(dc, [1])
    assert isinstance(dy, ops.DeviceArray)
    assert relerr(dy.to_numpy(), oracle.softmax(oracle.gemm(a, b), [1])) <= 1e-12
    with pytest.raises(TypeError):
        ops.gemm(da, b)  # device and host operands do not mix
