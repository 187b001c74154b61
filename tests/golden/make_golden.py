"""Regenerates ``tests/golden/*.npz``.

The reference (docc) keeps no golden vector files: its tests draw random inputs and compare
against numpy (``a @ b``), ``scipy.special.softmax`` / the max-exp-sum-div numpy expression,
and torch (``nn.Conv2d``, ``nn.Linear``, ``torch.matmul``) with ``allclose``. These fixtures
freeze exactly those comparisons on seeded inputs at the shapes the reference's tests use:

  python/tests/python/functions/numpy/test_linalg.py        10x10 fp64 / fp32, batched (2,10,10)
  python/tests/python/targets/test_overrides.py             8x8 fp32
  python/tests/python/functions/scipy/test_scipy_softmax.py 10x10 fp64, axis 0 and all axes
  mlir/integration/torch/test_conv2d.py                     3->16 channels, 3x3 / 1x1 / 5x5, stride 2, batch 4
  mlir/integration/torch/test_matmul.py, test_linear.py     2-D matmul, Linear without bias

Rows the reference does not test (padded / biased conv, attention, LayerNorm, GELU) are frozen
from torch's CPU kernels as a second opinion; they are marked ``unpinned_`` in the file.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os

import numpy as np
import scipy.special
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    out = {}
    rng = np.random.RandomState(1234)

    # --- GEMM / matmul (numpy is the reference tests' ground truth) ---
    a, b = rng.rand(10, 10), rng.rand(10, 10)
    out["gemm_f64_a"], out["gemm_f64_b"], out["gemm_f64_y"] = a, b, a @ b
    a32, b32 = rng.rand(10, 10).astype(np.float32), rng.rand(10, 10).astype(np.float32)
    out["gemm_f32_a"], out["gemm_f32_b"], out["gemm_f32_y"] = a32, b32, a32 @ b32
    a8, b8 = rng.rand(8, 8).astype(np.float32), rng.rand(8, 8).astype(np.float32)
    out["gemm_f32_8_a"], out["gemm_f32_8_b"], out["gemm_f32_8_y"] = a8, b8, a8 @ b8
    ab, bb = rng.rand(2, 10, 10), rng.rand(2, 10, 10)
    out["matmul_batched_a"], out["matmul_batched_b"], out["matmul_batched_y"] = ab, bb, ab @ bb
    ar, br = rng.rand(7, 13), rng.rand(13, 5)
    out["gemm_rect_a"], out["gemm_rect_b"], out["gemm_rect_y"] = ar, br, ar @ br

    # --- softmax (scipy / numpy expression) ---
    x = rng.rand(10, 10)
    out["softmax_x"] = x
    out["softmax_axis0_y"] = scipy.special.softmax(x, axis=0)
    out["softmax_all_y"] = scipy.special.softmax(x)
    x32 = (rng.randn(16, 40) * 3).astype(np.float32)
    e = np.exp(x32 - x32.max(axis=-1, keepdims=True))
    out["softmax_f32_x"], out["softmax_f32_y"] = x32, e / e.sum(axis=-1, keepdims=True)

    # --- conv2d, torch ground truth, the reference's tested (unpadded, unbiased) cases ---
    torch.manual_seed(815)
    cases = {
        "conv3x3": dict(x=(1, 3, 32, 32), w=(16, 3, 3, 3), stride=1),
        "conv1x1": dict(x=(1, 3, 16, 16), w=(16, 3, 1, 1), stride=1),
        "conv5x5": dict(x=(1, 3, 16, 16), w=(8, 3, 5, 5), stride=1),
        "conv_s2": dict(x=(1, 3, 17, 17), w=(16, 3, 3, 3), stride=2),
        "conv_b4": dict(x=(4, 3, 12, 12), w=(16, 3, 3, 3), stride=1),
    }
    for name, c in cases.items():
        xt, wt = torch.randn(*c["x"]), torch.randn(*c["w"]) * 0.2
        out[f"{name}_x"], out[f"{name}_w"] = xt.numpy(), wt.numpy()
        out[f"{name}_y"] = F.conv2d(xt, wt, stride=c["stride"]).numpy()
        out[f"{name}_stride"] = np.array(c["stride"])

    # --- linear without bias (test_linear.py), 2-D torch.matmul (test_matmul.py) ---
    xt, wt = torch.randn(4, 10), torch.randn(5, 10)
    out["linear_x"], out["linear_w"], out["linear_y"] = xt.numpy(), wt.numpy(), F.linear(xt, wt).numpy()

    # --- unpinned by the reference: torch CPU as second opinion ---
    xt, wt, bt = torch.randn(2, 4, 9, 9), torch.randn(6, 4, 3, 3) * 0.2, torch.randn(6)
    out["unpinned_conv_pad_x"], out["unpinned_conv_pad_w"], out["unpinned_conv_pad_b"] = xt.numpy(), wt.numpy(), bt.numpy()
    out["unpinned_conv_pad_y"] = F.conv2d(xt, wt, bt, stride=1, padding=1).numpy()
    q, k, v = (torch.randn(2, 2, 24, 16) for _ in range(3))
    out["unpinned_attn_q"], out["unpinned_attn_k"], out["unpinned_attn_v"] = q.numpy(), k.numpy(), v.numpy()
    out["unpinned_attn_y"] = F.scaled_dot_product_attention(q, k, v).numpy()
    out["unpinned_attn_causal_y"] = F.scaled_dot_product_attention(q, k, v, is_causal=True).numpy()
    xt, g, bta = torch.randn(6, 48), torch.rand(48) + 0.5, torch.randn(48)
    out["unpinned_ln_x"], out["unpinned_ln_g"], out["unpinned_ln_b"] = xt.numpy(), g.numpy(), bta.numpy()
    out["unpinned_ln_y"] = F.layer_norm(xt, (48,), g, bta, 1e-5).numpy()
    out["unpinned_gelu_y"] = F.gelu(xt).numpy()

    np.savez_compressed(os.path.join(HERE, "reference_cases.npz"), **out)
    print("wrote", os.path.join(HERE, "reference_cases.npz"), len(out), "arrays")


if __name__ == "__main__":
    main()
