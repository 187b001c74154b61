// Interface between the conv entry point (conv.cu) and the implicit-GEMM kernel (conv_tc.cu).
#pragma once

#include "common.cuh"

namespace docc_b200 {

struct ConvTcProblem {
    int64_t N, C, H, W, c_out, kh, kw, pad_h, pad_w, Ho, Wo;
    int prec_in;  // 's' (split into bf16 hi/lo, three passes) or 'b'
};

// 2-D, stride 1, dilation 1, group 1 convolution as an implicit GEMM on tcgen05. X is NCHW of
// prec_in, Wt is [c_out, C, kh, kw] of prec_in, bias/Y are fp32. Returns
// DOCC_B200_ERR_UNSUPPORTED for shapes outside the kernel's tiling rules.
int conv_tc(Ctx* ctx, const ConvTcProblem& p, const void* X, const void* Wt, const float* bias, float* Y);

}  // namespace docc_b200
