// Attention entry point of the C ABI: O = softmax(scale * Q K^T [+ causal mask]) V.
//
// docc has no attention node; through its frontends the computation is two MatMulNodes around a
// SoftmaxNode, i.e. the S x S score matrix makes four trips through HBM. Both kernels here are
// flash-style: scores live in registers / tensor memory and only Q, K, V, O touch HBM.
//   * attention_tc.cu — tcgen05 kernel for 16-bit inputs with head_dim 64 or 128;
//   * the kernel below — one warp per query row with an online softmax, for fp32 inputs, other
//     head sizes and unaligned strides.
#include "attention.h"
#include "device_math.cuh"

namespace docc_b200 {
namespace {

// One warp owns one query row. Lane l holds elements l, l+32, .. of q and of the output
// accumulator (D <= 32*DPL). Keys are visited in order; per key one warp-wide dot product and the
// online-softmax update (running max m, running sum l, rescaled accumulator).
template <typename T, int DPL>
__global__ void __launch_bounds__(256) attention_rows_kernel(const T* __restrict__ Q, const T* __restrict__ K,
                                                             const T* __restrict__ V, T* __restrict__ O, AttnProblem p) {
    const int lane = threadIdx.x & 31;
    const int64_t warp_global = (blockIdx.x * int64_t(blockDim.x) + threadIdx.x) >> 5;
    const int64_t n_warps = (int64_t(gridDim.x) * blockDim.x) >> 5;
    const int64_t total_rows = p.B * p.H * p.Sq;
    for (int64_t r = warp_global; r < total_rows; r += n_warps) {
        const int64_t i = r % p.Sq;
        const int64_t h = (r / p.Sq) % p.H;
        const int64_t b = r / (p.Sq * p.H);
        const T* q = Q + b * p.qs[0] + h * p.qs[1] + i * p.qs[2];
        const T* kbase = K + b * p.ks[0] + h * p.ks[1];
        const T* vbase = V + b * p.vs[0] + h * p.vs[1];
        float qr[DPL], acc[DPL];
#pragma unroll
        for (int e = 0; e < DPL; e++) {
            const int d = lane + 32 * e;
            qr[e] = d < p.D ? to_float(q[d]) * p.scale : 0.f;
            acc[e] = 0.f;
        }
        int64_t lim = p.causal ? i + p.Skv - p.Sq + 1 : p.Skv;
        if (lim > p.Skv) lim = p.Skv;
        float m = -INFINITY, l = 0.f;
        for (int64_t j = 0; j < lim; j++) {
            const T* kr = kbase + j * p.ks[2];
            float s = 0.f;
#pragma unroll
            for (int e = 0; e < DPL; e++) {
                const int d = lane + 32 * e;
                if (d < p.D) s = fmaf(qr[e], to_float(kr[d]), s);
            }
            s = warp_sum_f(s);
            const float m_new = fmaxf(m, s);
            const float corr = __expf(m - m_new);  // exp(-inf) = 0 on the first key
            const float pj = __expf(s - m_new);
            l = l * corr + pj;
            const T* vr = vbase + j * p.vs[2];
#pragma unroll
            for (int e = 0; e < DPL; e++) {
                const int d = lane + 32 * e;
                if (d < p.D) acc[e] = fmaf(pj, to_float(vr[d]), acc[e] * corr);
            }
            m = m_new;
        }
        T* o = O + b * p.os[0] + h * p.os[1] + i * p.os[2];
        const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
        for (int e = 0; e < DPL; e++) {
            const int d = lane + 32 * e;
            if (d < p.D) o[d] = from_float<T>(acc[e] * inv);
        }
    }
}

template <typename T>
int launch_rows(Ctx* ctx, const AttnProblem& p, const void* Q, const void* K, const void* V, void* O) {
    const int64_t rows = p.B * p.H * p.Sq;
    const int64_t blocks = ceil_div(rows, 8);
    const int64_t cap = int64_t(ctx->sm_count) * 8;
    const int grid = int(blocks < cap ? blocks : cap);
    const T *q = static_cast<const T*>(Q), *k = static_cast<const T*>(K), *v = static_cast<const T*>(V);
    T* o = static_cast<T*>(O);
    if (p.D <= 32) attention_rows_kernel<T, 1><<<grid, 256, 0, ctx->stream>>>(q, k, v, o, p);
    else if (p.D <= 64) attention_rows_kernel<T, 2><<<grid, 256, 0, ctx->stream>>>(q, k, v, o, p);
    else if (p.D <= 128) attention_rows_kernel<T, 4><<<grid, 256, 0, ctx->stream>>>(q, k, v, o, p);
    else if (p.D <= 256) attention_rows_kernel<T, 8><<<grid, 256, 0, ctx->stream>>>(q, k, v, o, p);
    else return set_error(DOCC_B200_ERR_UNSUPPORTED, "attention: head_dim %lld > 256", (long long)p.D);
    return after_launch(ctx, "attention_rows_kernel");
}

}  // namespace

int attention_device(Ctx* ctx, const AttnProblem& p, const void* Q, const void* K, const void* V, void* O, int flags) {
    if (p.B * p.H * p.Sq * p.D == 0) return DOCC_B200_OK;
    if ((p.prec == DOCC_B200_PREC_B || p.prec == DOCC_B200_PREC_H) && !(flags & DOCC_B200_FLAG_FP32_EXACT)) {
        int s = attention_tc(ctx, p, Q, K, V, O);
        if (s != DOCC_B200_ERR_UNSUPPORTED) return s;
    }
    if (p.prec == DOCC_B200_PREC_S && !(flags & DOCC_B200_FLAG_FP32_EXACT)) {
        int s = attention_tc_f32(ctx, p, Q, K, V, O);
        if (s != DOCC_B200_ERR_UNSUPPORTED) return s;
    }
    switch (p.prec) {
        case DOCC_B200_PREC_S: return launch_rows<float>(ctx, p, Q, K, V, O);
        case DOCC_B200_PREC_B: return launch_rows<__nv_bfloat16>(ctx, p, Q, K, V, O);
        case DOCC_B200_PREC_H: return launch_rows<__half>(ctx, p, Q, K, V, O);
    }
    return set_error(DOCC_B200_ERR_INVALID_ARG, "attention: precision %d not supported (use 's', 'b' or 'h')", p.prec);
}

}  // namespace docc_b200

using namespace docc_b200;

extern "C" int docc_b200_attention(int prec, int64_t B, int64_t H, int64_t Sq, int64_t Skv, int64_t D, float scale, int causal,
                                   const void* Q, const int64_t* q_strides, const void* K, const int64_t* k_strides,
                                   const void* V, const int64_t* v_strides, void* O, const int64_t* o_strides, int flags) {
    Ctx* ctx;
    DOCC_TRY(get_ctx(&ctx));
    DOCC_REQUIRE(prec == DOCC_B200_PREC_S || prec == DOCC_B200_PREC_B || prec == DOCC_B200_PREC_H,
                 "attention: precision %d not supported (use 's', 'b' or 'h')", prec);
    DOCC_REQUIRE(B >= 0 && H >= 0 && Sq >= 0 && Skv >= 0 && D >= 0, "attention: negative extent");
    if (B * H * Sq * D == 0) return DOCC_B200_OK;
    DOCC_REQUIRE(Q && K && V && O, "attention: NULL data pointer");
    AttnProblem p;
    p.prec = prec; p.B = B; p.H = H; p.Sq = Sq; p.Skv = Skv; p.D = D; p.scale = scale; p.causal = causal ? 1 : 0;
    const int64_t dq[3] = {H * Sq * D, Sq * D, D}, dk[3] = {H * Skv * D, Skv * D, D};
    for (int i = 0; i < 3; i++) {
        p.qs[i] = q_strides ? q_strides[i] : dq[i];
        p.ks[i] = k_strides ? k_strides[i] : dk[i];
        p.vs[i] = v_strides ? v_strides[i] : dk[i];
        p.os[i] = o_strides ? o_strides[i] : dq[i];
    }
    if (!(flags & DOCC_B200_FLAG_HOST_PTRS)) return attention_device(ctx, p, Q, K, V, O, flags);
    DOCC_REQUIRE(!q_strides && !k_strides && !v_strides && !o_strides, "attention: host pointers require contiguous [B,H,S,D] tensors");
    const size_t es = prec_size(prec);
    const size_t q_b = size_t(B * H * Sq * D) * es, k_b = size_t(B * H * Skv * D) * es;
    TempBuffers tmp;
    void *dQ, *dK, *dV, *dO;
    DOCC_TRY(tmp.alloc(&dQ, q_b));
    DOCC_TRY(tmp.alloc(&dK, k_b));
    DOCC_TRY(tmp.alloc(&dV, k_b));
    DOCC_TRY(tmp.alloc(&dO, q_b));
    DOCC_CUDA_TRY(cudaMemcpyAsync(dQ, Q, q_b, cudaMemcpyHostToDevice, ctx->stream));
    if (k_b) DOCC_CUDA_TRY(cudaMemcpyAsync(dK, K, k_b, cudaMemcpyHostToDevice, ctx->stream));
    if (k_b) DOCC_CUDA_TRY(cudaMemcpyAsync(dV, V, k_b, cudaMemcpyHostToDevice, ctx->stream));
    DOCC_TRY(attention_device(ctx, p, dQ, dK, dV, dO, flags));
    DOCC_CUDA_TRY(cudaMemcpyAsync(O, dO, q_b, cudaMemcpyDeviceToHost, ctx->stream));
    DOCC_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    return DOCC_B200_OK;
}
