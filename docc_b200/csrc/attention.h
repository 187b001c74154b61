// Interface between the attention entry point (attention.cu) and the tcgen05 flash kernel
// (attention_tc.cu).
#pragma once

#include "common.cuh"

namespace docc_b200 {

struct AttnProblem {
    int prec;  // 'b' or 'h'
    int64_t B, H, Sq, Skv, D;
    float scale;
    int causal;
    int64_t qs[3], ks[3], vs[3], os[3];  // element strides: batch, head, sequence (D is contiguous)
    // fp32 only, optional: when set, a kernel that can do so writes O as two bf16 planes (hi = bf16(o), lo = bf16(o - hi), element
    // strides `os`) instead of fp32, the operand form of the fp32 tensor-core GEMM, and sets *planes_done; otherwise O is written
    // as usual and *planes_done stays false.
    void* o_hi = nullptr;
    void* o_lo = nullptr;
    bool* planes_done = nullptr;
};

// Returns DOCC_B200_ERR_UNSUPPORTED for shapes the tensor-core kernel does not tile.
int attention_tc(Ctx* ctx, const AttnProblem& p, const void* Q, const void* K, const void* V, void* O);

// fp32 inputs and output, head_dim 64: split-bf16 tensor-core path (three products per contraction).
int attention_tc_f32(Ctx* ctx, const AttnProblem& p, const void* Q, const void* K, const void* V, void* O);

}  // namespace docc_b200
