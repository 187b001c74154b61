// Bandwidth-bound nodes: LayerNorm, fused scale/bias/activation/residual, same-shape binary
// ops and casts. On docc's CUDA target each of these is a chain of one-op loop-nest kernels
// (elementwise_node.cpp:86-339 expanded and scheduled by cuda_map_dispatcher.cpp:42-333),
// one HBM round trip per primitive. Here each call is one pass: every input byte is read once
// with 128-bit accesses and every output byte written once.
#include <type_traits>

#include "common.cuh"
#include "device_math.cuh"
#include "ptx.cuh"

namespace docc_b200 {
namespace {

// ---- LayerNorm -----------------------------------------------------------------------------
// One warp per row while a row fits in registers (cols <= 32*VPT*VEC), else block per row.
// Two-pass statistics in registers: mean, then sum((x-mean)^2) — the form torch lowers to and
// the numerically safe one; population variance as in StdNode (std_node.cpp:147-222).
// Both LayerNorm kernels run under programmatic stream serialization: nothing is read before the wait.
__device__ __forceinline__ void griddep_wait_all() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <typename T, int VPT, int TPR, int BLOCK>
__global__ void __launch_bounds__(BLOCK) layernorm_kernel(const T* __restrict__ X, const float* __restrict__ gamma,
                                                          const float* __restrict__ beta, float eps, T* __restrict__ Y,
                                                          int64_t rows, int64_t cols) {
    griddep_wait_all();
    constexpr int VEC = 16 / sizeof(T);
    using P = Pack<T, VEC>;
    constexpr int RPB = BLOCK / TPR;
    constexpr int WPR = TPR / 32;
    __shared__ float red[2][RPB][WPR];
    const int t = threadIdx.x % TPR, rib = threadIdx.x / TPR, wir = t / 32;
    const int64_t packs = cols / VEC;
    const int64_t groups = (rows + RPB - 1) / RPB;
    for (int64_t g = blockIdx.x; g < groups; g += gridDim.x) {
        const int64_t row = g * RPB + rib;
        const bool ok = row < rows;
        const P* xr = reinterpret_cast<const P*>(X + row * cols);
        float v[VPT][VEC];
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < VPT; i++) {
            const int64_t p = int64_t(i) * TPR + t;
            if (ok && p < packs) {
                const P pk = load_pack(xr + p);
#pragma unroll
                for (int e = 0; e < VEC; e++) {
                    v[i][e] = to_float(pk.v[e]);
                    s += v[i][e];
                }
            } else {
#pragma unroll
                for (int e = 0; e < VEC; e++) v[i][e] = 0.f;
            }
        }
        s = warp_sum_f(s);
        if (WPR > 1) {
            if ((t & 31) == 0) red[0][rib][wir] = s;
            __syncthreads();
            s = 0.f;
#pragma unroll
            for (int w = 0; w < WPR; w++) s += red[0][rib][w];
        }
        const float mean = s / float(cols);
        float q = 0.f;
#pragma unroll
        for (int i = 0; i < VPT; i++) {
            const int64_t p = int64_t(i) * TPR + t;
            if (ok && p < packs) {
#pragma unroll
                for (int e = 0; e < VEC; e++) {
                    const float d = v[i][e] - mean;
                    q += d * d;
                }
            }
        }
        q = warp_sum_f(q);
        if (WPR > 1) {
            if ((t & 31) == 0) red[1][rib][wir] = q;
            __syncthreads();
            q = 0.f;
#pragma unroll
            for (int w = 0; w < WPR; w++) q += red[1][rib][w];
        }
        const float rstd = rsqrtf(q / float(cols) + eps);
        P* yr = reinterpret_cast<P*>(Y + row * cols);
#pragma unroll
        for (int i = 0; i < VPT; i++) {
            const int64_t p = int64_t(i) * TPR + t;
            if (ok && p < packs) {
                P pk;
                // gamma / beta as 16-byte vectors (VEC is 4 or 8 and the arrays are 16-byte aligned here)
                float gm[VEC], bt[VEC];
#pragma unroll
                for (int q4 = 0; q4 < VEC / 4; q4++) {
                    const float4 g4 = gamma ? __ldg(reinterpret_cast<const float4*>(gamma + p * VEC) + q4) : make_float4(1.f, 1.f, 1.f, 1.f);
                    const float4 b4 = beta ? __ldg(reinterpret_cast<const float4*>(beta + p * VEC) + q4) : make_float4(0.f, 0.f, 0.f, 0.f);
                    gm[q4 * 4 + 0] = g4.x; gm[q4 * 4 + 1] = g4.y; gm[q4 * 4 + 2] = g4.z; gm[q4 * 4 + 3] = g4.w;
                    bt[q4 * 4 + 0] = b4.x; bt[q4 * 4 + 1] = b4.y; bt[q4 * 4 + 2] = b4.z; bt[q4 * 4 + 3] = b4.w;
                }
#pragma unroll
                for (int e = 0; e < VEC; e++) pk.v[e] = from_float<T>((v[i][e] - mean) * rstd * gm[e] + bt[e]);
                store_pack(yr + p, pk);
            }
        }
        if (WPR > 1) __syncthreads();
    }
}

// Rows that fit one warp's registers, many rows per warp, rows staged through shared memory by bulk copies.
// A warp-per-row LayerNorm holds a row in registers, so the bytes a warp can have in flight are bounded by its
// registers: with a 1024-wide bf16 row that was 2 KB per warp, 32 KB per SM, too little to cover HBM latency
// (measured 3.4 TB/s). Here every warp owns a ring of kLnStages row buffers in shared memory that one lane keeps
// filled with cp.async.bulk copies (completion on an mbarrier per slot): 3 rows per warp and 16 warps per SM are in
// flight whatever the register count. The warp walks rows w, w + W, w + 2W, ... (W = warps in the grid), reads its row
// and the gamma / beta slice from shared memory, and stores the result straight from registers (coalesced 16-byte
// stores). gamma / beta are staged once per block.
constexpr int kLnStages = 3;
constexpr int kLnWarps = 16;

// `hi` / `lo` (fp32 rows only): instead of Y the kernel writes the result as two bf16 planes, value = hi + lo to about 16
// mantissa bits, the form in which the fp32 tensor-core GEMM takes its operands; a LayerNorm that feeds a linear layer
// then saves that GEMM's split pass over the activations (one read and one write of the fp32 tensor).
template <typename T, int VPT>
__global__ void __launch_bounds__(kLnWarps * 32, 1) layernorm_bulk_kernel(const T* __restrict__ X, const float* __restrict__ gamma,
                                                                         const float* __restrict__ beta, float eps, T* __restrict__ Y,
                                                                         int64_t rows, int64_t cols, __nv_bfloat16* __restrict__ hi,
                                                                         __nv_bfloat16* __restrict__ lo) {
    constexpr int VEC = 16 / sizeof(T);
    using P = Pack<T, VEC>;
    extern __shared__ __align__(128) uint8_t ln_smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t row_bytes = uint32_t(cols) * uint32_t(sizeof(T));
    const uint32_t row_pitch = (row_bytes + 127u) & ~127u;
    // layout: gamma [cols] fp32, beta [cols] fp32, mbarriers [warps][stages], row buffers [warps][stages][row_pitch]
    float* s_gamma = reinterpret_cast<float*>(ln_smem);
    float* s_beta = s_gamma + cols;
    const uint32_t bars = ptx::smem_u32(ln_smem) + ((uint32_t(cols) * 8u + 127u) & ~127u);
    const uint32_t bufs = bars + ((uint32_t(kLnWarps * kLnStages) * 8u + 127u) & ~127u);
    const uint32_t my_bar = bars + uint32_t(warp * kLnStages) * 8u;
    const uint32_t my_buf = bufs + uint32_t(warp * kLnStages) * row_pitch;
    if (lane == 0) {
        for (int s = 0; s < kLnStages; s++) ptx::mbar_init(my_bar + 8u * s, 1);
        ptx::fence_barrier_init();
    }
    __syncwarp();
    griddep_wait_all();  // nothing above touches global memory
    const int64_t packs = cols / VEC;
    const int64_t warps = int64_t(gridDim.x) * kLnWarps;
    const int64_t first = int64_t(blockIdx.x) * kLnWarps + warp;
    // fill this warp's ring, then stage the parameters while those copies fly
    if (lane == 0) {
        for (int s = 0; s < kLnStages; s++) {
            const int64_t r = first + int64_t(s) * warps;
            if (r < rows) {
                ptx::mbar_arrive_expect_tx(my_bar + 8u * s, row_bytes);
                ptx::bulk_load_1d(my_buf + uint32_t(s) * row_pitch, X + r * cols, row_bytes, my_bar + 8u * s);
            }
        }
    }
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
        s_gamma[c] = gamma ? gamma[c] : 1.f;
        s_beta[c] = beta ? beta[c] : 0.f;
    }
    __syncthreads();
    const float inv_cols = 1.f / float(cols);
    uint32_t stage = 0, phase = 0;
    for (int64_t row = first; row < rows; row += warps) {
        if (!ptx::mbar_wait(my_bar + 8u * stage, phase)) return;  // bounded; a copy that never lands ends the warp
        P cur[VPT];
        const uint32_t src = my_buf + stage * row_pitch;
#pragma unroll
        for (int i = 0; i < VPT; i++) {
            const int64_t p = int64_t(i) * 32 + lane;
            if (p < packs) {
                uint4 w;
                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w) : "r"(src + uint32_t(p) * 16u) : "memory");
                cur[i] = *reinterpret_cast<const P*>(&w);
            }
        }
        __syncwarp();  // every lane has its part of the row in registers: the slot can be refilled
        if (lane == 0) {
            const int64_t r = row + int64_t(kLnStages) * warps;
            if (r < rows) {
                ptx::mbar_arrive_expect_tx(my_bar + 8u * stage, row_bytes);
                ptx::bulk_load_1d(my_buf + stage * row_pitch, X + r * cols, row_bytes, my_bar + 8u * stage);
            }
        }
        if (++stage == uint32_t(kLnStages)) {
            stage = 0;
            phase ^= 1u;
        }
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < VPT; i++) {
            if (int64_t(i) * 32 + lane < packs) {
#pragma unroll
                for (int e = 0; e < VEC; e++) s += to_float(cur[i].v[e]);
            }
        }
        const float mean = warp_sum_f(s) * inv_cols;
        float q = 0.f;
#pragma unroll
        for (int i = 0; i < VPT; i++) {
            if (int64_t(i) * 32 + lane < packs) {
#pragma unroll
                for (int e = 0; e < VEC; e++) {
                    const float d = to_float(cur[i].v[e]) - mean;
                    q += d * d;
                }
            }
        }
        const float rstd = rsqrtf(warp_sum_f(q) * inv_cols + eps);
        P* yr = reinterpret_cast<P*>(Y + row * cols);
#pragma unroll
        for (int i = 0; i < VPT; i++) {
            const int64_t p = int64_t(i) * 32 + lane;
            if (p < packs) {
                P pk;
#pragma unroll
                for (int q4 = 0; q4 < VEC / 4; q4++) {
                    const float4 g4 = *reinterpret_cast<const float4*>(s_gamma + p * VEC + q4 * 4);
                    const float4 b4 = *reinterpret_cast<const float4*>(s_beta + p * VEC + q4 * 4);
                    pk.v[q4 * 4 + 0] = from_float<T>((to_float(cur[i].v[q4 * 4 + 0]) - mean) * rstd * g4.x + b4.x);
                    pk.v[q4 * 4 + 1] = from_float<T>((to_float(cur[i].v[q4 * 4 + 1]) - mean) * rstd * g4.y + b4.y);
                    pk.v[q4 * 4 + 2] = from_float<T>((to_float(cur[i].v[q4 * 4 + 2]) - mean) * rstd * g4.z + b4.z);
                    pk.v[q4 * 4 + 3] = from_float<T>((to_float(cur[i].v[q4 * 4 + 3]) - mean) * rstd * g4.w + b4.w);
                }
                if constexpr (std::is_same<T, float>::value) {
                    if (hi) {  // VEC == 4: four values -> 8 bytes of each plane
                        __nv_bfloat16 h[4], l[4];
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            h[e] = __float2bfloat16_rn(pk.v[e]);
                            l[e] = __float2bfloat16_rn(pk.v[e] - __bfloat162float(h[e]));
                        }
                        *reinterpret_cast<uint2*>(hi + row * cols + p * 4) = *reinterpret_cast<const uint2*>(h);
                        *reinterpret_cast<uint2*>(lo + row * cols + p * 4) = *reinterpret_cast<const uint2*>(l);
                        continue;
                    }
                }
                store_pack(yr + p, pk);
            }
        }
    }
}

// Any cols / alignment: block per row, three passes over global memory.
template <typename T>
__global__ void __launch_bounds__(256) layernorm_generic_kernel(const T* __restrict__ X, const float* __restrict__ gamma,
                                                                const float* __restrict__ beta, float eps,
                                                                T* __restrict__ Y, int64_t rows, int64_t cols) {
    __shared__ float smem[8];
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* xr = X + row * cols;
        float s = 0.f;
        for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) s += to_float(xr[c]);
        const float mean = block_sum_f(s, smem) / float(cols);
        float q = 0.f;
        for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
            const float d = to_float(xr[c]) - mean;
            q += d * d;
        }
        const float rstd = rsqrtf(block_sum_f(q, smem) / float(cols) + eps);
        for (int64_t c = threadIdx.x; c < cols; c += blockDim.x)
            Y[row * cols + c] =
                from_float<T>((to_float(xr[c]) - mean) * rstd * (gamma ? gamma[c] : 1.f) + (beta ? beta[c] : 0.f));
    }
}

template <typename T, int VPT>
int launch_ln_bulk(Ctx* ctx, const T* X, const float* g, const float* b, float eps, T* Y, int64_t rows, int64_t cols,
                   __nv_bfloat16* hi = nullptr, __nv_bfloat16* lo = nullptr) {
    static bool attr_done[16] = {};  // per instantiation and device
    const size_t row_pitch = (size_t(cols) * sizeof(T) + 127) & ~size_t(127);
    const size_t smem = ((size_t(cols) * 8 + 127) & ~size_t(127)) + ((size_t(kLnWarps * kLnStages) * 8 + 127) & ~size_t(127)) +
                        size_t(kLnWarps * kLnStages) * row_pitch;
    auto kern = layernorm_bulk_kernel<T, VPT>;
    if (!attr_done[ctx->device & 15]) {
        DOCC_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        attr_done[ctx->device & 15] = true;
    }
    int64_t blocks = ceil_div(rows, kLnWarps);
    if (blocks > ctx->sm_count) blocks = ctx->sm_count;
    DOCC_CUDA_TRY(launch_pdl(kern, dim3(unsigned(blocks)), dim3(kLnWarps * 32), smem, ctx->stream, X, g, b, eps, Y, rows, cols, hi, lo));
    return after_launch(ctx, "layernorm_bulk_kernel");
}

template <typename T, int VPT, int TPR>
int launch_ln(Ctx* ctx, const T* X, const float* g, const float* b, float eps, T* Y, int64_t rows, int64_t cols) {
    constexpr int BLOCK = TPR > 256 ? TPR : 256;
    const int64_t groups = ceil_div(rows, BLOCK / TPR);
    // one row group per block (the block scheduler balances the SMs; a resident-size grid with a stride loop leaves SMs
    // idle in the last partial round of groups)
    const int64_t cap = 0x7fffffff;
    DOCC_CUDA_TRY(launch_pdl(layernorm_kernel<T, VPT, TPR, BLOCK>, dim3(unsigned(groups < cap ? groups : cap)), dim3(BLOCK), 0, ctx->stream,
                             X, g, b, eps, Y, rows, cols));
    return after_launch(ctx, "layernorm_kernel");
}

template <typename T>
int layernorm_device(Ctx* ctx, int64_t rows, int64_t cols, const T* X, const float* g, const float* b, double eps, T* Y) {
    if (rows == 0 || cols == 0) return DOCC_B200_OK;
    constexpr int VEC = 16 / sizeof(T);
    const bool aligned = cols % VEC == 0 && reinterpret_cast<uintptr_t>(X) % 16 == 0 && reinterpret_cast<uintptr_t>(Y) % 16 == 0 &&
                         reinterpret_cast<uintptr_t>(g) % 16 == 0 && reinterpret_cast<uintptr_t>(b) % 16 == 0;
    const int64_t packs = cols / VEC;
    if (aligned && packs <= 2048) {
        if (packs <= 32) return launch_ln<T, 1, 32>(ctx, X, g, b, float(eps), Y, rows, cols);
        if (packs <= 64) return launch_ln<T, 2, 32>(ctx, X, g, b, float(eps), Y, rows, cols);
        // many rows: the persistent kernel that stages rows through shared memory (rows up to 4 KB keep 48 of them per SM
        // in flight inside the 227 KB budget)
        const bool many = rows >= int64_t(ctx->sm_count) * kLnWarps * 2 && size_t(cols) * sizeof(T) <= 4096;
        if (many && packs <= 64) return launch_ln_bulk<T, 2>(ctx, X, g, b, float(eps), Y, rows, cols);
        if (many && packs <= 128) return launch_ln_bulk<T, 4>(ctx, X, g, b, float(eps), Y, rows, cols);
        if (many && packs <= 256) return launch_ln_bulk<T, 8>(ctx, X, g, b, float(eps), Y, rows, cols);
        if (packs <= 128) return launch_ln<T, 4, 32>(ctx, X, g, b, float(eps), Y, rows, cols);
        if (packs <= 256) return launch_ln<T, 8, 32>(ctx, X, g, b, float(eps), Y, rows, cols);
        if (packs <= 512) return launch_ln<T, 4, 128>(ctx, X, g, b, float(eps), Y, rows, cols);
        if (packs <= 1024) return launch_ln<T, 8, 128>(ctx, X, g, b, float(eps), Y, rows, cols);
        return launch_ln<T, 8, 256>(ctx, X, g, b, float(eps), Y, rows, cols);
    }
    const int64_t cap = int64_t(ctx->sm_count) * 8;
    layernorm_generic_kernel<T><<<int(rows < cap ? rows : cap), 256, 0, ctx->stream>>>(X, g, b, float(eps), Y, rows, cols);
    return after_launch(ctx, "layernorm_generic_kernel");
}

// ---- fused scale / bias / activation / residual ----------------------------------------------------
template <typename T, bool VECTOR>
__global__ void __launch_bounds__(256) bias_act_kernel(const T* __restrict__ X, float scale, const float* __restrict__ bias,
                                                       int act, const T* __restrict__ residual, T* __restrict__ Y,
                                                       int64_t total, int64_t cols) {
    constexpr int VEC = VECTOR ? 16 / sizeof(T) : 1;
    using P = Pack<T, VEC>;
    const int64_t n_packs = total / VEC;
    for (int64_t p = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; p < n_packs; p += int64_t(gridDim.x) * blockDim.x) {
        const P x = load_pack(reinterpret_cast<const P*>(X) + p);
        P r;
        if (residual) r = load_pack(reinterpret_cast<const P*>(residual) + p);
        const int64_t c0 = (p * VEC) % cols;
        P y;
#pragma unroll
        for (int e = 0; e < VEC; e++) {
            float v = to_float(x.v[e]) * scale;
            if (bias) v += bias[c0 + e];
            v = apply_act(act, v);
            if (residual) v += to_float(r.v[e]);
            y.v[e] = from_float<T>(v);
        }
        store_pack(reinterpret_cast<P*>(Y) + p, y);
    }
}

__global__ void __launch_bounds__(256) bias_act_f64_kernel(const double* __restrict__ X, double scale,
                                                           const float* __restrict__ bias, int act,
                                                           const double* __restrict__ residual, double* __restrict__ Y,
                                                           int64_t total, int64_t cols) {
    for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x) {
        double v = X[i] * scale;
        if (bias) v += double(bias[i % cols]);
        v = apply_act_f64(act, v);
        if (residual) v += residual[i];
        Y[i] = v;
    }
}

template <typename T>
int bias_act_device(Ctx* ctx, int64_t rows, int64_t cols, const T* X, float scale, const float* bias, int act,
                    const T* residual, T* Y) {
    const int64_t total = rows * cols;
    if (total == 0) return DOCC_B200_OK;
    constexpr int VEC = 16 / sizeof(T);
    const bool vec = cols % VEC == 0 && reinterpret_cast<uintptr_t>(X) % 16 == 0 && reinterpret_cast<uintptr_t>(Y) % 16 == 0 &&
                     reinterpret_cast<uintptr_t>(residual) % 16 == 0;
    const int64_t items = vec ? total / VEC : total;
    const int64_t blocks = ceil_div(items, 256);
    const int64_t cap = int64_t(ctx->sm_count) * 16;
    const int grid = int(blocks < cap ? blocks : cap);
    if (vec) bias_act_kernel<T, true><<<grid, 256, 0, ctx->stream>>>(X, scale, bias, act, residual, Y, total, cols);
    else bias_act_kernel<T, false><<<grid, 256, 0, ctx->stream>>>(X, scale, bias, act, residual, Y, total, cols);
    return after_launch(ctx, "bias_act_kernel");
}

// ---- binary ops and casts -------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) binary_kernel(int op, const T* __restrict__ A, const T* __restrict__ B,
                                                     T* __restrict__ Y, int64_t n) {
    for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x) {
        const T a = A[i], b = B[i];
        T y;
        switch (op) {
            case DOCC_B200_EW_ADD: y = a + b; break;
            case DOCC_B200_EW_SUB: y = a - b; break;
            case DOCC_B200_EW_MUL: y = a * b; break;
            case DOCC_B200_EW_DIV: y = a / b; break;
            case DOCC_B200_EW_MAX: y = fmax(a, b); break;
            default: y = fmin(a, b); break;
        }
        Y[i] = y;
    }
}

template <typename TI, typename TO>
__global__ void __launch_bounds__(256) cast_kernel(const TI* __restrict__ X, TO* __restrict__ Y, int64_t n) {
    for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x)
        Y[i] = cast_to<TO>(X[i]);
}

template <typename TI>
int cast_dispatch_out(Ctx* ctx, int prec_out, int64_t n, const void* X, void* Y) {
    const int64_t blocks = ceil_div(n, 256);
    const int64_t cap = int64_t(ctx->sm_count) * 16;
    const int grid = int(blocks < cap ? blocks : cap);
    const TI* x = static_cast<const TI*>(X);
    switch (prec_out) {
        case DOCC_B200_PREC_D: cast_kernel<TI, double><<<grid, 256, 0, ctx->stream>>>(x, static_cast<double*>(Y), n); break;
        case DOCC_B200_PREC_S: cast_kernel<TI, float><<<grid, 256, 0, ctx->stream>>>(x, static_cast<float*>(Y), n); break;
        case DOCC_B200_PREC_H: cast_kernel<TI, __half><<<grid, 256, 0, ctx->stream>>>(x, static_cast<__half*>(Y), n); break;
        case DOCC_B200_PREC_B:
            cast_kernel<TI, __nv_bfloat16><<<grid, 256, 0, ctx->stream>>>(x, static_cast<__nv_bfloat16*>(Y), n);
            break;
        default: return set_error(DOCC_B200_ERR_INVALID_ARG, "cast: unknown output precision %d", prec_out);
    }
    return after_launch(ctx, "cast_kernel");
}

// Runs `fn(device pointers...)` with host arrays staged through pooled device buffers.
struct Staged {
    const void* host_in[3];
    size_t bytes_in[3];
    int n_in = 0;
    void* host_out = nullptr;
    size_t bytes_out = 0;
};

template <typename F>
int with_transfers(Ctx* ctx, const Staged& s, F fn) {
    TempBuffers tmp;
    void* din[3] = {nullptr, nullptr, nullptr};
    void* dout = nullptr;
    for (int i = 0; i < s.n_in; i++) {
        if (!s.host_in[i]) continue;
        DOCC_TRY(tmp.alloc(&din[i], s.bytes_in[i]));
        DOCC_CUDA_TRY(cudaMemcpyAsync(din[i], s.host_in[i], s.bytes_in[i], cudaMemcpyHostToDevice, ctx->stream));
    }
    DOCC_TRY(tmp.alloc(&dout, s.bytes_out));
    DOCC_TRY(fn(din, dout));
    DOCC_CUDA_TRY(cudaMemcpyAsync(s.host_out, dout, s.bytes_out, cudaMemcpyDeviceToHost, ctx->stream));
    DOCC_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    return DOCC_B200_OK;
}

}  // namespace

// Used by the transformer block.
int layernorm_f32(Ctx* ctx, int64_t rows, int64_t cols, const float* X, const float* g, const float* b, double eps, float* Y) {
    return layernorm_device<float>(ctx, rows, cols, X, g, b, eps, Y);
}
// fp32 LayerNorm whose result leaves as bf16 hi / lo planes of row pitch `cols` (see layernorm_bulk_kernel). Only the
// many-rows kernel has this form: DOCC_B200_ERR_UNSUPPORTED tells the caller to normalise into fp32 and split as usual.
int layernorm_f32_split(Ctx* ctx, int64_t rows, int64_t cols, const float* X, const float* g, const float* b, double eps,
                        __nv_bfloat16* hi, __nv_bfloat16* lo) {
    const bool aligned = cols % 8 == 0 && reinterpret_cast<uintptr_t>(X) % 16 == 0 && reinterpret_cast<uintptr_t>(g) % 16 == 0 &&
                         reinterpret_cast<uintptr_t>(b) % 16 == 0 && reinterpret_cast<uintptr_t>(hi) % 16 == 0 &&
                         reinterpret_cast<uintptr_t>(lo) % 16 == 0;
    const int64_t packs = cols / 4;
    const bool many = rows >= int64_t(ctx->sm_count) * kLnWarps * 2 && size_t(cols) * 4 <= 4096;
    if (!aligned || !many || packs <= 32) return DOCC_B200_ERR_UNSUPPORTED;
    if (packs <= 64) return launch_ln_bulk<float, 2>(ctx, X, g, b, float(eps), nullptr, rows, cols, hi, lo);
    if (packs <= 128) return launch_ln_bulk<float, 4>(ctx, X, g, b, float(eps), nullptr, rows, cols, hi, lo);
    return launch_ln_bulk<float, 8>(ctx, X, g, b, float(eps), nullptr, rows, cols, hi, lo);
}
int layernorm_bf16(Ctx* ctx, int64_t rows, int64_t cols, const __nv_bfloat16* X, const float* g, const float* b, double eps,
                   __nv_bfloat16* Y) {
    return layernorm_device<__nv_bfloat16>(ctx, rows, cols, X, g, b, eps, Y);
}

}  // namespace docc_b200

using namespace docc_b200;

extern "C" int docc_b200_layernorm(int prec, int64_t rows, int64_t cols, const void* X, const void* gamma, const void* beta,
                                   double eps, void* Y, int flags) {
    Ctx* ctx;
    DOCC_TRY(get_ctx(&ctx));
    DOCC_REQUIRE(rows >= 0 && cols >= 0, "layernorm: negative extent");
    DOCC_REQUIRE(rows * cols == 0 || (X && Y), "layernorm: NULL data pointer");
    DOCC_REQUIRE(prec == DOCC_B200_PREC_S || prec == DOCC_B200_PREC_B || prec == DOCC_B200_PREC_H,
                 "layernorm: precision %d not supported (use 's', 'b' or 'h')", prec);
    const size_t es = prec_size(prec);
    auto run = [&](const void* x, const float* g, const float* b, void* y) {
        if (prec == DOCC_B200_PREC_S)
            return layernorm_device<float>(ctx, rows, cols, static_cast<const float*>(x), g, b, eps, static_cast<float*>(y));
        if (prec == DOCC_B200_PREC_H)
            return layernorm_device<__half>(ctx, rows, cols, static_cast<const __half*>(x), g, b, eps, static_cast<__half*>(y));
        return layernorm_device<__nv_bfloat16>(ctx, rows, cols, static_cast<const __nv_bfloat16*>(x), g, b, eps,
                                               static_cast<__nv_bfloat16*>(y));
    };
    if (!(flags & DOCC_B200_FLAG_HOST_PTRS)) return run(X, static_cast<const float*>(gamma), static_cast<const float*>(beta), Y);
    Staged s;
    s.host_in[0] = X; s.bytes_in[0] = size_t(rows * cols) * es;
    s.host_in[1] = gamma; s.bytes_in[1] = size_t(cols) * 4;
    s.host_in[2] = beta; s.bytes_in[2] = size_t(cols) * 4;
    s.n_in = 3; s.host_out = Y; s.bytes_out = size_t(rows * cols) * es;
    if (rows * cols == 0) return DOCC_B200_OK;
    return with_transfers(ctx, s, [&](void** din, void* dout) {
        return run(din[0], static_cast<const float*>(din[1]), static_cast<const float*>(din[2]), dout);
    });
}

extern "C" int docc_b200_bias_act(int prec, int64_t rows, int64_t cols, const void* X, float scale, const void* bias, int act,
                                  const void* residual, void* Y, int flags) {
    Ctx* ctx;
    DOCC_TRY(get_ctx(&ctx));
    DOCC_REQUIRE(rows >= 0 && cols >= 0, "bias_act: negative extent");
    DOCC_REQUIRE(rows * cols == 0 || (X && Y), "bias_act: NULL data pointer");
    DOCC_REQUIRE(act >= DOCC_B200_ACT_NONE && act <= DOCC_B200_ACT_ABS, "bias_act: unknown activation %d", act);
    const size_t es = prec_size(prec);
    DOCC_REQUIRE(prec == DOCC_B200_PREC_S || prec == DOCC_B200_PREC_B || prec == DOCC_B200_PREC_D || prec == DOCC_B200_PREC_H,
                 "bias_act: unknown precision %d", prec);
    auto run = [&](const void* x, const float* b, const void* r, void* y) -> int {
        switch (prec) {
            case DOCC_B200_PREC_S:
                return bias_act_device<float>(ctx, rows, cols, static_cast<const float*>(x), scale, b, act,
                                              static_cast<const float*>(r), static_cast<float*>(y));
            case DOCC_B200_PREC_B:
                return bias_act_device<__nv_bfloat16>(ctx, rows, cols, static_cast<const __nv_bfloat16*>(x), scale, b, act,
                                                      static_cast<const __nv_bfloat16*>(r), static_cast<__nv_bfloat16*>(y));
            case DOCC_B200_PREC_H:
                return bias_act_device<__half>(ctx, rows, cols, static_cast<const __half*>(x), scale, b, act,
                                               static_cast<const __half*>(r), static_cast<__half*>(y));
            default: {
                const int64_t total = rows * cols;
                if (total == 0) return DOCC_B200_OK;
                const int64_t blocks = ceil_div(total, 256);
                const int64_t cap = int64_t(ctx->sm_count) * 16;
                bias_act_f64_kernel<<<int(blocks < cap ? blocks : cap), 256, 0, ctx->stream>>>(
                    static_cast<const double*>(x), double(scale), b, act, static_cast<const double*>(r),
                    static_cast<double*>(y), total, cols);
                return after_launch(ctx, "bias_act_f64_kernel");
            }
        }
    };
    if (!(flags & DOCC_B200_FLAG_HOST_PTRS)) return run(X, static_cast<const float*>(bias), residual, Y);
    if (rows * cols == 0) return DOCC_B200_OK;
    Staged s;
    s.host_in[0] = X; s.bytes_in[0] = size_t(rows * cols) * es;
    s.host_in[1] = bias; s.bytes_in[1] = size_t(cols) * 4;
    s.host_in[2] = residual; s.bytes_in[2] = size_t(rows * cols) * es;
    s.n_in = 3; s.host_out = Y; s.bytes_out = size_t(rows * cols) * es;
    return with_transfers(ctx, s, [&](void** din, void* dout) { return run(din[0], static_cast<const float*>(din[1]), din[2], dout); });
}

extern "C" int docc_b200_binary(int op, int prec, int64_t n, const void* X1, const void* X2, void* Y, int flags) {
    Ctx* ctx;
    DOCC_TRY(get_ctx(&ctx));
    DOCC_REQUIRE(n >= 0, "binary: negative size");
    DOCC_REQUIRE(op >= DOCC_B200_EW_ADD && op <= DOCC_B200_EW_MIN, "binary: unknown op %d", op);
    DOCC_REQUIRE(prec == DOCC_B200_PREC_S || prec == DOCC_B200_PREC_D, "binary: precision %d not supported (use 's' or 'd')", prec);
    if (n == 0) return DOCC_B200_OK;
    DOCC_REQUIRE(X1 && X2 && Y, "binary: NULL data pointer");
    auto run = [&](const void* a, const void* b, void* y) -> int {
        const int64_t blocks = ceil_div(n, 256);
        const int64_t cap = int64_t(ctx->sm_count) * 16;
        const int grid = int(blocks < cap ? blocks : cap);
        if (prec == DOCC_B200_PREC_S)
            binary_kernel<float><<<grid, 256, 0, ctx->stream>>>(op, static_cast<const float*>(a), static_cast<const float*>(b),
                                                                static_cast<float*>(y), n);
        else
            binary_kernel<double><<<grid, 256, 0, ctx->stream>>>(op, static_cast<const double*>(a),
                                                                 static_cast<const double*>(b), static_cast<double*>(y), n);
        return after_launch(ctx, "binary_kernel");
    };
    if (!(flags & DOCC_B200_FLAG_HOST_PTRS)) return run(X1, X2, Y);
    const size_t es = prec_size(prec);
    Staged s;
    s.host_in[0] = X1; s.bytes_in[0] = size_t(n) * es;
    s.host_in[1] = X2; s.bytes_in[1] = size_t(n) * es;
    s.n_in = 2; s.host_out = Y; s.bytes_out = size_t(n) * es;
    return with_transfers(ctx, s, [&](void** din, void* dout) { return run(din[0], din[1], dout); });
}

extern "C" int docc_b200_cast(int prec_in, int prec_out, int64_t n, const void* X, void* Y, int flags) {
    Ctx* ctx;
    DOCC_TRY(get_ctx(&ctx));
    DOCC_REQUIRE(n >= 0, "cast: negative size");
    DOCC_REQUIRE(prec_size(prec_in) && prec_size(prec_out), "cast: unknown precision code");
    if (n == 0) return DOCC_B200_OK;
    DOCC_REQUIRE(X && Y, "cast: NULL data pointer");
    auto run = [&](const void* x, void* y) -> int {
        switch (prec_in) {
            case DOCC_B200_PREC_D: return cast_dispatch_out<double>(ctx, prec_out, n, x, y);
            case DOCC_B200_PREC_S: return cast_dispatch_out<float>(ctx, prec_out, n, x, y);
            case DOCC_B200_PREC_H: return cast_dispatch_out<__half>(ctx, prec_out, n, x, y);
            default: return cast_dispatch_out<__nv_bfloat16>(ctx, prec_out, n, x, y);
        }
    };
    if (!(flags & DOCC_B200_FLAG_HOST_PTRS)) return run(X, Y);
    Staged s;
    s.host_in[0] = X; s.bytes_in[0] = size_t(n) * prec_size(prec_in);
    s.n_in = 1; s.host_out = Y; s.bytes_out = size_t(n) * prec_size(prec_out);
    return with_transfers(ctx, s, [&](void** din, void* dout) { return run(din[0], dout); });
}
