// GEMM entry points of the C ABI and the non-tcgen05 contraction kernels.
//
//   docc_b200_gemm           GEMMNode (gemm_node.h:16-87) — replaces the cuBLAS sequence of
//                            opt/src/targets/cuda/blas/gemm.cpp:33-185.
//   docc_b200_matmul         batch loop MatMulNode::expand builds (matmul_node.cpp:353-489).
//   docc_b200_gemm_epilogue  GEMM fused with the element-wise nodes that follow it.
//
// fp64 runs on the DMMA pipe (mma.sync m8n8k4.f64; tcgen05 has no fp64 kind). fp32 and 16-bit
// inputs run on the tcgen05 engine in gemm_tc.cu whenever TMA's 16-byte alignment rules hold;
// a tiled FFMA kernel covers the rest (odd leading dimensions, DOCC_B200_FLAG_FP32_EXACT).
#include "device_math.cuh"
#include "gemm_tc.h"
#include "ptx.cuh"

namespace docc_b200 {
namespace {

// Element (i,k) of op(A) is A[i*a_rs + k*a_cs]; element (k,j) of op(B) is B[k*b_rs + j*b_cs].
struct GemmView {
    int64_t M, N, K;
    int64_t a_rs, a_cs, b_rs, b_cs, ldc;
    int64_t a_bs, b_bs, c_bs;  // batch strides (elements)
};

struct SimtEpilogue {
    double alpha, beta;
    const void* bias;      // per column; fp64 when bias_f64 (the 'd' path), fp32 otherwise
    bool bias_f64;
    int act;
    const void* residual;  // same type as C
    int64_t ldr;
};

// ---- fp64: DMMA ------------------------------------------------------------------------------
// 64x64 block tile, BK = 16, 4 warps (2x2), each warp 32x32 = 4x4 m8n8k4 tiles.
// Shared tiles are padded so the fragment loads (8-byte, 16 lanes per wavefront) are conflict free:
// A[m][k] pitch 20, B[k][n] pitch 68 (both = 4 mod 16 eight-byte banks).
constexpr int DM = 64, DN = 64, DK = 16, DA_PITCH = 20, DB_PITCH = 68;

__device__ __forceinline__ void dmma(double& d0, double& d1, double a, double b) {
    asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};" : "+d"(d0), "+d"(d1) : "d"(a), "d"(b));
}

__global__ void __launch_bounds__(128) gemm_f64_dmma_kernel(const double* __restrict__ A, const double* __restrict__ B,
                                                            double* __restrict__ C, GemmView g, double alpha, double beta) {
    __shared__ double As[2][DM * DA_PITCH];
    __shared__ double Bs[2][DK * DB_PITCH];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wm = (warp >> 1) * 32, wn = (warp & 1) * 32;
    const int64_t m0 = int64_t(blockIdx.y) * DM, n0 = int64_t(blockIdx.x) * DN;
    A += blockIdx.z * g.a_bs;
    B += blockIdx.z * g.b_bs;
    C += blockIdx.z * g.c_bs;
    // launched with programmatic stream serialization: no global access before the launch before this one has completed
    ptx::griddep_wait();
    ptx::griddep_launch_dependents();

    // global -> register staging; thread mapping follows whichever index is contiguous in memory
    const bool a_k_fast = g.a_cs == 1, b_n_fast = g.b_cs == 1;
    double ra[8], rb[8];
    auto load_tiles = [&](int64_t k0) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int e = tid + i * 128;
            const int m = a_k_fast ? e / DK : e % DM;
            const int k = a_k_fast ? e % DK : e / DM;
            const int64_t gm = m0 + m, gk = k0 + k;
            ra[i] = (gm < g.M && gk < g.K) ? A[gm * g.a_rs + gk * g.a_cs] : 0.0;
            const int n = b_n_fast ? e % DN : e / DK;
            const int kb = b_n_fast ? e / DN : e % DK;
            const int64_t gn = n0 + n, gkb = k0 + kb;
            rb[i] = (gn < g.N && gkb < g.K) ? B[gkb * g.b_rs + gn * g.b_cs] : 0.0;
        }
    };
    auto store_tiles = [&](int buf) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int e = tid + i * 128;
            const int m = a_k_fast ? e / DK : e % DM;
            const int k = a_k_fast ? e % DK : e / DM;
            As[buf][m * DA_PITCH + k] = ra[i];
            const int n = b_n_fast ? e % DN : e / DK;
            const int kb = b_n_fast ? e / DN : e % DK;
            Bs[buf][kb * DB_PITCH + n] = rb[i];
        }
    };

    double acc[4][4][2];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j][0] = acc[i][j][1] = 0.0;

    const int64_t nk = (g.K + DK - 1) / DK;
    load_tiles(0);
    store_tiles(0);
    __syncthreads();
    for (int64_t kt = 0; kt < nk; kt++) {
        const int buf = int(kt & 1);
        if (kt + 1 < nk) load_tiles((kt + 1) * DK);
        const double* as = As[buf];
        const double* bs = Bs[buf];
#pragma unroll
        for (int k4 = 0; k4 < DK; k4 += 4) {
            double af[4], bf[4];
#pragma unroll
            for (int i = 0; i < 4; i++) af[i] = as[(wm + i * 8 + (lane >> 2)) * DA_PITCH + k4 + (lane & 3)];
#pragma unroll
            for (int j = 0; j < 4; j++) bf[j] = bs[(k4 + (lane & 3)) * DB_PITCH + wn + j * 8 + (lane >> 2)];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) dmma(acc[i][j][0], acc[i][j][1], af[i], bf[j]);
        }
        if (kt + 1 < nk) store_tiles(buf ^ 1);
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int64_t row = m0 + wm + i * 8 + (lane >> 2);
        if (row >= g.M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int64_t col = n0 + wn + j * 8 + (lane & 3) * 2;
#pragma unroll
            for (int e = 0; e < 2; e++) {
                if (col + e < g.N) {
                    double* c = C + row * g.ldc + col + e;
                    const double v = alpha * acc[i][j][e];
                    *c = (beta == 0.0) ? v : v + beta * *c;
                }
            }
        }
    }
}

// ---- tiled FFMA / DFMA kernel for everything the tensor paths do not take -----------------------------
template <typename T> struct AccOf { using type = float; };
template <> struct AccOf<double> { using type = double; };
__device__ __forceinline__ double to_acc(double v, double) { return v; }
template <typename T> __device__ __forceinline__ float to_acc(T v, float) { return to_float(v); }
template <typename T> __device__ __forceinline__ T from_acc(float v) { return from_float<T>(v); }
template <typename T> __device__ __forceinline__ T from_acc(double v) { return T(v); }

template <typename T>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const T* __restrict__ A, const T* __restrict__ B, T* __restrict__ C,
                                                        GemmView g, SimtEpilogue ep) {
    using Acc = typename AccOf<T>::type;
    constexpr int TM = 64, TN = 64, TK = 16;
    __shared__ Acc As[TK][TM + 4];
    __shared__ Acc Bs[TK][TN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int64_t m0 = int64_t(blockIdx.y) * TM, n0 = int64_t(blockIdx.x) * TN;
    A += blockIdx.z * g.a_bs;
    B += blockIdx.z * g.b_bs;
    C += blockIdx.z * g.c_bs;
    const T* R = ep.residual ? static_cast<const T*>(ep.residual) + blockIdx.z * g.c_bs : nullptr;
    const bool a_k_fast = g.a_cs == 1, b_n_fast = g.b_cs == 1;
    Acc acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = Acc(0);
    for (int64_t k0 = 0; k0 < g.K; k0 += TK) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int e = tid + i * 256;
            const int m = a_k_fast ? e / TK : e % TM;
            const int k = a_k_fast ? e % TK : e / TM;
            const int64_t gm = m0 + m, gk = k0 + k;
            As[k][m] = (gm < g.M && gk < g.K) ? to_acc(A[gm * g.a_rs + gk * g.a_cs], Acc(0)) : Acc(0);
            const int n = b_n_fast ? e % TN : e / TK;
            const int kb = b_n_fast ? e / TN : e % TK;
            const int64_t gn = n0 + n, gkb = k0 + kb;
            Bs[kb][n] = (gn < g.N && gkb < g.K) ? to_acc(B[gkb * g.b_rs + gn * g.b_cs], Acc(0)) : Acc(0);
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < TK; k++) {
            Acc a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) b[j] = Bs[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fma(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int64_t row = m0 + ty * 4 + i;
        if (row >= g.M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int64_t col = n0 + tx * 4 + j;
            if (col >= g.N) continue;
            Acc v = Acc(ep.alpha) * acc[i][j];
            if (ep.beta != 0.0) v += Acc(ep.beta) * to_acc(C[row * g.ldc + col], Acc(0));
            if (ep.bias) v += ep.bias_f64 ? Acc(static_cast<const double*>(ep.bias)[col]) : Acc(static_cast<const float*>(ep.bias)[col]);
            if (ep.act != DOCC_B200_ACT_NONE) {
                if constexpr (sizeof(Acc) == 8) v = apply_act_f64(ep.act, v);
                else v = apply_act(ep.act, v);
            }
            if (R) v += to_acc(R[row * ep.ldr + col], Acc(0));
            C[row * g.ldc + col] = from_acc<T>(v);
        }
    }
}

template <typename T>
int launch_simt(Ctx* ctx, const void* A, const void* B, void* C, const GemmView& g, const SimtEpilogue& ep, int64_t batch) {
    if (g.M == 0 || g.N == 0 || batch == 0) return DOCC_B200_OK;
    dim3 grid(unsigned(ceil_div(g.N, 64)), unsigned(ceil_div(g.M, 64)), unsigned(batch));
    if (grid.y > 65535 || grid.z > 65535) return set_error(DOCC_B200_ERR_UNSUPPORTED, "gemm: extent too large for the fallback kernel");
    gemm_simt_kernel<T><<<grid, 256, 0, ctx->stream>>>(static_cast<const T*>(A), static_cast<const T*>(B), static_cast<T*>(C), g, ep);
    return after_launch(ctx, "gemm_simt_kernel");
}

int launch_simt_prec(Ctx* ctx, int prec, const void* A, const void* B, void* C, const GemmView& g, const SimtEpilogue& ep,
                     int64_t batch) {
    switch (prec) {
        case DOCC_B200_PREC_D: return launch_simt<double>(ctx, A, B, C, g, ep, batch);
        case DOCC_B200_PREC_S: return launch_simt<float>(ctx, A, B, C, g, ep, batch);
        case DOCC_B200_PREC_H: return launch_simt<__half>(ctx, A, B, C, g, ep, batch);
        case DOCC_B200_PREC_B: return launch_simt<__nv_bfloat16>(ctx, A, B, C, g, ep, batch);
    }
    return set_error(DOCC_B200_ERR_INVALID_ARG, "gemm: unknown precision code %d", prec);
}

int launch_dmma(Ctx* ctx, const void* A, const void* B, void* C, const GemmView& g, double alpha, double beta, int64_t batch) {
    if (g.M == 0 || g.N == 0 || batch == 0) return DOCC_B200_OK;
    dim3 grid(unsigned(ceil_div(g.N, DN)), unsigned(ceil_div(g.M, DM)), unsigned(batch));
    if (grid.y > 65535 || grid.z > 65535) return set_error(DOCC_B200_ERR_UNSUPPORTED, "gemm: extent too large");
    DOCC_CUDA_TRY(launch_pdl(gemm_f64_dmma_kernel, grid, dim3(128), 0, ctx->stream, static_cast<const double*>(A), static_cast<const double*>(B),
                             static_cast<double*>(C), g, alpha, beta));
    return after_launch(ctx, "gemm_f64_dmma_kernel");
}

int64_t round_up8(int64_t v) { return (v + 7) / 8 * 8; }

// fp32 / 16-bit GEMM on the tcgen05 engine. Row-major views only (column-major problems are
// transposed by the caller). Returns DOCC_B200_ERR_UNSUPPORTED when the engine cannot take it.
// `a_presplit` (fp32, K-major A, one batch): the caller has already written the bf16 hi / lo planes of A into workspace
// slot 0 in the layout below ([M][round_up8(K)], lo behind hi); A itself is not read.
int run_tc(Ctx* ctx, int prec, const void* A, const void* B, const GemmView& g, int64_t batch, const TcEpilogue& ep,
           bool a_presplit = false) {
    if (g.K == 0) return set_error(DOCC_B200_ERR_UNSUPPORTED, "K == 0");
    const bool a_kmajor = g.a_cs == 1;  // op(A)[i][k] contiguous in k
    const bool b_kmajor = g.b_rs == 1;  // op(B)[k][j] contiguous in k
    if (!a_kmajor && g.a_rs != 1) return set_error(DOCC_B200_ERR_UNSUPPORTED, "A has no unit stride");
    if (!b_kmajor && g.b_cs != 1) return set_error(DOCC_B200_ERR_UNSUPPORTED, "B has no unit stride");
    if (prec == DOCC_B200_PREC_B || prec == DOCC_B200_PREC_H) {
        TcOperand a, b;
        a.ptr = A; a.ld = a_kmajor ? g.a_rs : g.a_cs; a.batch_stride = g.a_bs; a.k_major = a_kmajor;
        b.ptr = B; b.ld = b_kmajor ? g.b_cs : g.b_rs; b.batch_stride = g.b_bs; b.k_major = b_kmajor;
        const int pa[1] = {0}, pb[1] = {0};
        return tc_gemm(ctx, prec == DOCC_B200_PREC_B ? 1 : 0, g.M, g.N, g.K, batch, 1, &a, pa, &b, pb, ep);
    }
    // fp32: split both operands into bf16 hi/lo planes, always K-major (the split transposes when needed)
    const int64_t kp = round_up8(g.K);
    const bool a_shared = batch > 1 && g.a_bs == 0, b_shared = batch > 1 && g.b_bs == 0;
    const int64_t a_planes = a_shared ? 1 : batch, b_planes = b_shared ? 1 : batch;
    const size_t a_elems = size_t(g.M) * kp, b_elems = size_t(g.N) * kp;
    void *wa, *wb;
    DOCC_TRY(get_workspace(ctx, 0, a_elems * a_planes * 2 * sizeof(__nv_bfloat16), &wa));
    DOCC_TRY(get_workspace(ctx, 1, b_elems * b_planes * 2 * sizeof(__nv_bfloat16), &wb));
    __nv_bfloat16* a_hi = static_cast<__nv_bfloat16*>(wa);
    __nv_bfloat16* a_lo = a_hi + a_elems * a_planes;
    __nv_bfloat16* b_hi = static_cast<__nv_bfloat16*>(wb);
    __nv_bfloat16* b_lo = b_hi + b_elems * b_planes;
    // A as stored: k-major -> [M][K] rows; otherwise memory is [K][M] and is transposed into [M][K]
    if (a_presplit) {
        if (!a_kmajor || batch != 1) return set_error(DOCC_B200_ERR_INVALID_ARG, "gemm: pre-split A needs a K-major operand and one batch");
    } else if (a_kmajor) DOCC_TRY(split_f32_to_bf16x2(ctx, static_cast<const float*>(A), g.M, g.K, g.a_rs, a_planes, g.a_bs, false, a_hi, a_lo, kp, int64_t(a_elems)));
    else DOCC_TRY(split_f32_to_bf16x2(ctx, static_cast<const float*>(A), g.K, g.M, g.a_cs, a_planes, g.a_bs, true, a_hi, a_lo, kp, int64_t(a_elems)));
    if (b_kmajor) DOCC_TRY(split_f32_to_bf16x2(ctx, static_cast<const float*>(B), g.N, g.K, g.b_cs, b_planes, g.b_bs, false, b_hi, b_lo, kp, int64_t(b_elems)));
    else DOCC_TRY(split_f32_to_bf16x2(ctx, static_cast<const float*>(B), g.K, g.N, g.b_rs, b_planes, g.b_bs, true, b_hi, b_lo, kp, int64_t(b_elems)));
    TcOperand a[2], b[2];
    a[0].ptr = a_hi; a[1].ptr = a_lo; b[0].ptr = b_hi; b[1].ptr = b_lo;
    for (int i = 0; i < 2; i++) {
        a[i].ld = kp; a[i].batch_stride = a_shared ? 0 : int64_t(a_elems); a[i].k_major = true;
        b[i].ld = kp; b[i].batch_stride = b_shared ? 0 : int64_t(b_elems); b[i].k_major = true;
    }
    // small terms first, the dominant hi*hi product last
    const int pa[3] = {1, 0, 0}, pb[3] = {0, 1, 0};
    return tc_gemm(ctx, 1, g.M, g.N, g.K, batch, 3, a, pa, b, pb, ep);
}

struct GemmCall {
    int prec;
    GemmView g;
    int64_t batch;
    double alpha, beta;
    const void* bias;  // element type of C for 's' and 'd', fp32 for 16-bit operands
    int act;
    const void* residual;
    int64_t ldr;
    int flags;
    bool a_presplit = false;  // fp32 only: A's bf16 planes are already in workspace slot 0 (run_tc)
};

// Device-pointer GEMM on a row-major view.
int gemm_device(Ctx* ctx, const GemmCall& c, const void* A, const void* B, void* C) {
    const GemmView& g = c.g;
    if (g.M == 0 || g.N == 0 || c.batch == 0) return DOCC_B200_OK;
    SimtEpilogue sep{c.alpha, c.beta, c.bias, c.prec == DOCC_B200_PREC_D, c.act, c.residual, c.ldr};
    if (c.prec == DOCC_B200_PREC_D) {
        if (c.bias || c.act != DOCC_B200_ACT_NONE || c.residual) return launch_simt<double>(ctx, A, B, C, g, sep, c.batch);
        return launch_dmma(ctx, A, B, C, g, c.alpha, c.beta, c.batch);
    }
    const bool want_tc = !(c.flags & DOCC_B200_FLAG_FP32_EXACT) && g.K > 0;
    if (want_tc) {
        TcEpilogue ep;
        ep.alpha = float(c.alpha); ep.beta = float(c.beta);
        ep.bias = static_cast<const float*>(c.bias); ep.bias_mode = c.bias ? 1 : 0; ep.act = c.act;
        ep.residual = c.residual; ep.ldr = c.ldr; ep.residual_batch_stride = g.c_bs;
        ep.out = C; ep.ldo = g.ldc; ep.out_batch_stride = g.c_bs; ep.out_prec = c.prec;
        int s = run_tc(ctx, c.prec, A, B, g, c.batch, ep, c.a_presplit);
        if (s != DOCC_B200_ERR_UNSUPPORTED) return s;
    }
    if (c.a_presplit) return set_error(DOCC_B200_ERR_UNSUPPORTED, "gemm: pre-split A has no fallback off the tensor-core path");
    return launch_simt_prec(ctx, c.prec, A, B, C, g, sep, c.batch);
}

size_t span_elems(int64_t rows, int64_t cols, int64_t rs, int64_t cs) {
    if (rows == 0 || cols == 0) return 0;
    return size_t((rows - 1) * rs + (cols - 1) * cs + 1);
}

// Host-pointer variant: stage op(A), op(B) (and C when beta != 0 or a residual is given) through
// pooled device buffers — what GEMMNodeDispatcher_CUBLASWithTransfers emits inline
// (opt/src/targets/cuda/blas/gemm.cpp:64-98), minus the per-call handle and cudaMalloc.
int gemm_host(Ctx* ctx, const GemmCall& c, const void* A, const void* B, void* C) {
    const GemmView& g = c.g;
    if (g.M == 0 || g.N == 0 || c.batch == 0) return DOCC_B200_OK;
    const size_t es = prec_size(c.prec);
    const size_t a_n = (c.batch - 1) * size_t(g.a_bs) + span_elems(g.M, g.K, g.a_rs, g.a_cs);
    const size_t b_n = (c.batch - 1) * size_t(g.b_bs) + span_elems(g.K, g.N, g.b_rs, g.b_cs);
    const size_t c_n = (c.batch - 1) * size_t(g.c_bs) + span_elems(g.M, g.N, g.ldc, 1);
    TempBuffers tmp;
    void *dA = nullptr, *dB = nullptr, *dC = nullptr, *dBias = nullptr, *dRes = nullptr;
    DOCC_TRY(tmp.alloc(&dA, a_n * es));
    DOCC_TRY(tmp.alloc(&dB, b_n * es));
    DOCC_TRY(tmp.alloc(&dC, c_n * es));
    if (a_n) DOCC_CUDA_TRY(cudaMemcpyAsync(dA, A, a_n * es, cudaMemcpyHostToDevice, ctx->stream));
    if (b_n) DOCC_CUDA_TRY(cudaMemcpyAsync(dB, B, b_n * es, cudaMemcpyHostToDevice, ctx->stream));
    // C travels to the device when it is an input (beta != 0) or when ldc leaves gaps that must survive
    if (c.beta != 0.0 || g.ldc != g.N) DOCC_CUDA_TRY(cudaMemcpyAsync(dC, C, c_n * es, cudaMemcpyHostToDevice, ctx->stream));
    GemmCall d = c;
    if (c.bias) {
        const size_t bias_bytes = size_t(g.N) * (c.prec == DOCC_B200_PREC_D ? 8 : 4);
        DOCC_TRY(tmp.alloc(&dBias, bias_bytes));
        DOCC_CUDA_TRY(cudaMemcpyAsync(dBias, c.bias, bias_bytes, cudaMemcpyHostToDevice, ctx->stream));
        d.bias = dBias;
    }
    if (c.residual) {
        const size_t r_n = (c.batch - 1) * size_t(g.c_bs) + span_elems(g.M, g.N, c.ldr, 1);
        DOCC_TRY(tmp.alloc(&dRes, r_n * es));
        DOCC_CUDA_TRY(cudaMemcpyAsync(dRes, c.residual, r_n * es, cudaMemcpyHostToDevice, ctx->stream));
        d.residual = dRes;
    }
    DOCC_TRY(gemm_device(ctx, d, dA, dB, dC));
    DOCC_CUDA_TRY(cudaMemcpyAsync(C, dC, c_n * es, cudaMemcpyDeviceToHost, ctx->stream));
    DOCC_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    return DOCC_B200_OK;
}

double read_scalar(int prec, const void* p, double dflt) {
    if (!p) return dflt;
    if (prec == DOCC_B200_PREC_D) return *static_cast<const double*>(p);
    return double(*static_cast<const float*>(p));
}

}  // namespace

// Used by the transformer block and conv: device-pointer linear layer Y = act(X W^T + bias) + residual.
int linear_device(Ctx* ctx, int prec, int64_t M, int64_t N, int64_t K, const void* X, int64_t ldx, const void* W, int64_t ldw,
                  const float* bias, int act, const void* residual, int64_t ldr, void* Y, int64_t ldy, bool x_presplit) {
    GemmCall c;
    c.a_presplit = x_presplit;
    c.prec = prec;
    c.g = GemmView{M, N, K, ldx, 1, 1, ldw, ldy, 0, 0, 0};
    c.batch = 1; c.alpha = 1.0; c.beta = 0.0; c.bias = bias; c.act = act; c.residual = residual; c.ldr = ldr; c.flags = 0;
    return gemm_device(ctx, c, X, W, Y);
}

}  // namespace docc_b200

using namespace docc_b200;

extern "C" int docc_b200_gemm(int prec, int layout, int transa, int transb, int64_t m, int64_t n, int64_t k, const void* alpha,
                              const void* A, int64_t lda, const void* B, int64_t ldb, const void* beta, void* C, int64_t ldc,
                              int flags) {
    Ctx* ctx;
    DOCC_TRY(get_ctx(&ctx));
    DOCC_REQUIRE(prec_size(prec) != 0, "gemm: unknown precision code %d", prec);
    DOCC_REQUIRE(layout == DOCC_B200_ROW_MAJOR || layout == DOCC_B200_COL_MAJOR, "gemm: unknown layout %d", layout);
    DOCC_REQUIRE(transa >= DOCC_B200_NO_TRANS && transa <= DOCC_B200_CONJ_TRANS, "gemm: unknown transA %d", transa);
    DOCC_REQUIRE(transb >= DOCC_B200_NO_TRANS && transb <= DOCC_B200_CONJ_TRANS, "gemm: unknown transB %d", transb);
    DOCC_REQUIRE(m >= 0 && n >= 0 && k >= 0, "gemm: negative dimension");
    if (m == 0 || n == 0) return DOCC_B200_OK;
    DOCC_REQUIRE(C != nullptr && (k == 0 || (A && B)), "gemm: NULL matrix pointer");
    // real types: conjugate transpose == transpose
    bool ta = transa != DOCC_B200_NO_TRANS, tb = transb != DOCC_B200_NO_TRANS;
    // column-major C = op(A) op(B)  <=>  row-major C^T = op(B)^T op(A)^T  (same swap as gemm.cpp:157-167)
    if (layout == DOCC_B200_COL_MAJOR) {
        const void* tp = A; A = B; B = tp;
        int64_t tl = lda; lda = ldb; ldb = tl;
        int64_t tm = m; m = n; n = tm;
        bool tt = ta; ta = tb; tb = tt;
    }
    // cblas leading-dimension rules for the row-major problem
    DOCC_REQUIRE(lda >= (ta ? (m > 1 ? m : 1) : (k > 1 ? k : 1)), "gemm: lda %lld too small", (long long)lda);
    DOCC_REQUIRE(ldb >= (tb ? (k > 1 ? k : 1) : (n > 1 ? n : 1)), "gemm: ldb %lld too small", (long long)ldb);
    DOCC_REQUIRE(ldc >= (n > 1 ? n : 1), "gemm: ldc %lld too small", (long long)ldc);
    GemmCall c;
    c.prec = prec;
    c.g.M = m; c.g.N = n; c.g.K = k;
    c.g.a_rs = ta ? 1 : lda; c.g.a_cs = ta ? lda : 1;
    c.g.b_rs = tb ? 1 : ldb; c.g.b_cs = tb ? ldb : 1;
    c.g.ldc = ldc; c.g.a_bs = c.g.b_bs = c.g.c_bs = 0;
    c.batch = 1;
    c.alpha = read_scalar(prec, alpha, 1.0);
    c.beta = read_scalar(prec, beta, 0.0);
    c.bias = nullptr; c.act = DOCC_B200_ACT_NONE; c.residual = nullptr; c.ldr = 0; c.flags = flags;
    if (flags & DOCC_B200_FLAG_HOST_PTRS) return gemm_host(ctx, c, A, B, C);
    return gemm_device(ctx, c, A, B, C);
}

extern "C" int docc_b200_matmul(int prec, int64_t batch, int64_t m, int64_t n, int64_t k, const void* A, int64_t lda,
                                int64_t batch_stride_a, const void* B, int64_t ldb, int64_t batch_stride_b, void* Y, int64_t ldy,
                                int64_t batch_stride_y, int flags) {
    Ctx* ctx;
    DOCC_TRY(get_ctx(&ctx));
    // integer element types are rejected by MatMulNode::expand (matmul_node.cpp:338-341); the ABI only has float codes
    DOCC_REQUIRE(prec_size(prec) != 0, "matmul: unknown precision code %d", prec);
    DOCC_REQUIRE(batch >= 0 && m >= 0 && n >= 0 && k >= 0, "matmul: negative dimension");
    if (batch == 0 || m == 0 || n == 0) return DOCC_B200_OK;
    DOCC_REQUIRE(Y != nullptr && (k == 0 || (A && B)), "matmul: NULL matrix pointer");
    DOCC_REQUIRE(lda >= (k > 1 ? k : 1) && ldb >= (n > 1 ? n : 1) && ldy >= (n > 1 ? n : 1), "matmul: leading dimension too small");
    DOCC_REQUIRE(batch_stride_a >= 0 && batch_stride_b >= 0 && batch_stride_y >= 0, "matmul: negative batch stride");
    GemmCall c;
    c.prec = prec;
    c.g = GemmView{m, n, k, lda, 1, ldb, 1, ldy, batch_stride_a, batch_stride_b, batch_stride_y};
    c.batch = batch; c.alpha = 1.0; c.beta = 0.0;
    c.bias = nullptr; c.act = DOCC_B200_ACT_NONE; c.residual = nullptr; c.ldr = 0; c.flags = flags;
    if (flags & DOCC_B200_FLAG_HOST_PTRS) return gemm_host(ctx, c, A, B, Y);
    return gemm_device(ctx, c, A, B, Y);
}

extern "C" int docc_b200_gemm_epilogue(int prec, int transb, int64_t m, int64_t n, int64_t k, float alpha, const void* A,
                                       int64_t lda, const void* B, int64_t ldb, const void* bias, int act, const void* residual,
                                       int64_t ldr, void* Y, int64_t ldy, int flags) {
    Ctx* ctx;
    DOCC_TRY(get_ctx(&ctx));
    DOCC_REQUIRE(prec == DOCC_B200_PREC_S || prec == DOCC_B200_PREC_B || prec == DOCC_B200_PREC_H || prec == DOCC_B200_PREC_D,
                 "gemm_epilogue: unknown precision code %d", prec);
    DOCC_REQUIRE(transb == DOCC_B200_NO_TRANS || transb == DOCC_B200_TRANS, "gemm_epilogue: unknown transB %d", transb);
    DOCC_REQUIRE(act >= DOCC_B200_ACT_NONE && act <= DOCC_B200_ACT_ABS, "gemm_epilogue: unknown activation %d", act);
    DOCC_REQUIRE(m >= 0 && n >= 0 && k >= 0, "gemm_epilogue: negative dimension");
    if (m == 0 || n == 0) return DOCC_B200_OK;
    DOCC_REQUIRE(Y != nullptr && (k == 0 || (A && B)), "gemm_epilogue: NULL matrix pointer");
    const bool tb = transb == DOCC_B200_TRANS;
    DOCC_REQUIRE(lda >= (k > 1 ? k : 1), "gemm_epilogue: lda too small");
    DOCC_REQUIRE(ldb >= (tb ? (k > 1 ? k : 1) : (n > 1 ? n : 1)), "gemm_epilogue: ldb too small");
    DOCC_REQUIRE(ldy >= (n > 1 ? n : 1) && (!residual || ldr >= (n > 1 ? n : 1)), "gemm_epilogue: ldy/ldr too small");
    GemmCall c;
    c.prec = prec;
    c.g.M = m; c.g.N = n; c.g.K = k;
    c.g.a_rs = lda; c.g.a_cs = 1;
    c.g.b_rs = tb ? 1 : ldb; c.g.b_cs = tb ? ldb : 1;
    c.g.ldc = ldy; c.g.a_bs = c.g.b_bs = c.g.c_bs = 0;
    c.batch = 1; c.alpha = alpha; c.beta = 0.0;
    c.bias = bias; c.act = act; c.residual = residual; c.ldr = ldr; c.flags = flags;
    if (flags & DOCC_B200_FLAG_HOST_PTRS) return gemm_host(ctx, c, A, B, Y);
    return gemm_device(ctx, c, A, B, Y);
}
