// Host interface of the tcgen05 contraction engine (gemm_tc.cu).
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace docc_b200 {

// One 16-bit operand of D = sum_p A_p * B_p.
//   A: k_major -> memory is [M][K] (K contiguous); otherwise [K][M].
//   B: k_major -> memory is [N][K] (K contiguous); otherwise [K][N].
// `ld` is the row stride in elements, `batch_stride` the distance between batch items.
struct TcOperand {
    const void* ptr = nullptr;
    int64_t ld = 0;
    int64_t batch_stride = 0;
    bool k_major = true;
};

struct TcEpilogue {
    float alpha = 1.f;
    float beta = 0.f;              // != 0: out is read as C
    const float* bias = nullptr;
    int bias_mode = 0;             // 0 none, 1 per column (n), 2 per row (m)
    int act = DOCC_B200_ACT_NONE;
    const void* residual = nullptr;  // same element type as out
    int64_t ldr = 0;
    int64_t residual_batch_stride = 0;
    void* out = nullptr;
    int64_t ldo = 0;
    int64_t out_batch_stride = 0;
    int out_prec = DOCC_B200_PREC_S;  // 's', 'b' or 'h'
};

// Operand element format: 0 = fp16, 1 = bf16.
// Runs D[b] = epilogue(sum_{p<npass} A[pa[p]][b] * B[pb[p]][b]) for b < batch on the calling
// thread's stream. Returns DOCC_B200_ERR_UNSUPPORTED when alignment rules of TMA are not met.
int tc_gemm(Ctx* ctx, int ab_format, int64_t M, int64_t N, int64_t K, int64_t batch, int npass, const TcOperand* A,
            const int* pa, const TcOperand* B, const int* pb, const TcEpilogue& ep);

// fp32 [rows x cols] (row stride ld) -> bf16 hi / lo planes with row stride ld_out
// (hi = bf16(x), lo = bf16(x - hi)). transpose: output is [cols x rows].
int split_f32_to_bf16x2(Ctx* ctx, const float* X, int64_t rows, int64_t cols, int64_t ld, int64_t batch,
                        int64_t batch_stride, bool transpose, __nv_bfloat16* hi, __nv_bfloat16* lo, int64_t ld_out,
                        int64_t out_batch_stride);

// Encodes a tiled tensor map with 128-byte swizzle for a 16-bit tensor (up to 4 dims, innermost
// first). Strides are in bytes for dims 1.. and must be multiples of 16.
int encode_tmap_16bit(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                      const uint32_t* box);
int encode_tmap(CUtensorMap* map, CUtensorMapDataType dtype, size_t elem_size, CUtensorMapSwizzle swizzle, const void* base,
                int rank, const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box);

}  // namespace docc_b200
