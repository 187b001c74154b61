// Pre-LN transformer encoder block as one device-resident chain of the node kernels:
//   h = x + Wo * attn(LN1(x) Wqkv^T + bqkv) + bo ;  y = h + W2 * gelu(W1 LN2(h) + b1) + b2
// Seven launches for bf16 (LN, QKV GEMM+bias, attention, out-proj GEMM+bias+residual, LN,
// FFN1 GEMM+bias+GELU, FFN2 GEMM+bias+residual); fp32 adds the hi/lo split launches in front of
// each GEMM. Every bias / activation / residual is fused into a GEMM epilogue, and no
// intermediate leaves the device — the schedule docc's DataTransferMinimizationPass
// (loop_scheduling_pass.cpp:130-133) aims for around consecutive library nodes.
#include "attention.h"
#include "common.cuh"

namespace docc_b200 {

int linear_device(Ctx* ctx, int prec, int64_t M, int64_t N, int64_t K, const void* X, int64_t ldx, const void* W, int64_t ldw,
                  const float* bias, int act, const void* residual, int64_t ldr, void* Y, int64_t ldy, bool x_presplit = false);
int attention_device(Ctx* ctx, const AttnProblem& p, const void* Q, const void* K, const void* V, void* O, int flags);
int layernorm_f32(Ctx* ctx, int64_t rows, int64_t cols, const float* X, const float* g, const float* b, double eps, float* Y);
int layernorm_f32_split(Ctx* ctx, int64_t rows, int64_t cols, const float* X, const float* g, const float* b, double eps,
                        __nv_bfloat16* hi, __nv_bfloat16* lo);
int layernorm_bf16(Ctx* ctx, int64_t rows, int64_t cols, const __nv_bfloat16* X, const float* g, const float* b, double eps,
                   __nv_bfloat16* Y);

namespace {

int layernorm_any(Ctx* ctx, int prec, int64_t rows, int64_t cols, const void* X, const void* g, const void* b, double eps, void* Y) {
    if (prec == DOCC_B200_PREC_S)
        return layernorm_f32(ctx, rows, cols, static_cast<const float*>(X), static_cast<const float*>(g),
                             static_cast<const float*>(b), eps, static_cast<float*>(Y));
    return layernorm_bf16(ctx, rows, cols, static_cast<const __nv_bfloat16*>(X), static_cast<const float*>(g),
                          static_cast<const float*>(b), eps, static_cast<__nv_bfloat16*>(Y));
}

int block_device(Ctx* ctx, int prec, const docc_b200_block_params& p, const void* X, void* Y) {
    const int64_t T = p.batch * p.seq, d = p.d_model, dff = p.d_ff, dh = d / p.n_heads;
    const size_t es = prec_size(prec);
    void* ws;
    DOCC_TRY(get_workspace(ctx, 2, size_t(T) * size_t(7 * d + dff) * es, &ws));
    char* base = static_cast<char*>(ws);
    void* h1 = base;
    void* qkv = base + size_t(T) * d * es;
    void* att = base + size_t(T) * 4 * d * es;
    void* h = base + size_t(T) * 5 * d * es;
    void* h2 = base + size_t(T) * 6 * d * es;
    void* f = base + size_t(T) * 7 * d * es;

    // fp32: a LayerNorm that feeds a linear layer writes the GEMM's bf16 hi / lo operand planes itself (workspace slot 0,
    // where the GEMM would put them: same size request, same pointer), which saves the split pass over the activations.
    // Returns true when the planes are in place, false when the shape is not one the fused kernel takes.
    auto ln_into_planes = [&](const void* src, const void* g, const void* b, bool* fused) -> int {
        *fused = false;
        if (prec != DOCC_B200_PREC_S || d % 8 != 0) return DOCC_B200_OK;
        void* planes;
        DOCC_TRY(get_workspace(ctx, 0, size_t(T) * size_t(d) * 2 * sizeof(__nv_bfloat16), &planes));
        __nv_bfloat16* hi = static_cast<__nv_bfloat16*>(planes);
        const int st = layernorm_f32_split(ctx, T, d, static_cast<const float*>(src), static_cast<const float*>(g),
                                           static_cast<const float*>(b), p.eps, hi, hi + size_t(T) * size_t(d));
        if (st == DOCC_B200_ERR_UNSUPPORTED) return DOCC_B200_OK;
        *fused = st == DOCC_B200_OK;
        return st;
    };
    bool fused = false;
    DOCC_TRY(ln_into_planes(X, p.ln1_g, p.ln1_b, &fused));
    if (!fused) DOCC_TRY(layernorm_any(ctx, prec, T, d, X, p.ln1_g, p.ln1_b, p.eps, h1));
    DOCC_TRY(linear_device(ctx, prec, T, 3 * d, d, h1, d, p.w_qkv, d, static_cast<const float*>(p.b_qkv), DOCC_B200_ACT_NONE,
                           nullptr, 0, qkv, 3 * d, fused));
    AttnProblem a;
    a.prec = prec; a.B = p.batch; a.H = p.n_heads; a.Sq = p.seq; a.Skv = p.seq; a.D = dh;
    a.scale = 1.0f / sqrtf(float(dh)); a.causal = 0;
    a.qs[0] = a.ks[0] = a.vs[0] = p.seq * 3 * d; a.qs[1] = a.ks[1] = a.vs[1] = dh; a.qs[2] = a.ks[2] = a.vs[2] = 3 * d;
    a.os[0] = p.seq * d; a.os[1] = dh; a.os[2] = d;
    const char* q = static_cast<const char*>(qkv);
    // fp32: the attention kernel may write its output as the out-projection's operand planes (same workspace slot and
    // layout as above: [T][d], lo behind hi); `att` then stays unwritten and the out-projection skips its split pass
    bool att_planes = false;
    if (prec == DOCC_B200_PREC_S && d % 8 == 0) {
        void* planes;
        DOCC_TRY(get_workspace(ctx, 0, size_t(T) * size_t(d) * 2 * sizeof(__nv_bfloat16), &planes));
        a.o_hi = planes;
        a.o_lo = static_cast<__nv_bfloat16*>(planes) + size_t(T) * size_t(d);
        a.planes_done = &att_planes;
    }
    DOCC_TRY(attention_device(ctx, a, q, q + size_t(d) * es, q + size_t(2 * d) * es, att, 0));
    DOCC_TRY(linear_device(ctx, prec, T, d, d, att, d, p.w_o, d, static_cast<const float*>(p.b_o), DOCC_B200_ACT_NONE, X, d, h, d,
                           att_planes));
    DOCC_TRY(ln_into_planes(h, p.ln2_g, p.ln2_b, &fused));
    if (!fused) DOCC_TRY(layernorm_any(ctx, prec, T, d, h, p.ln2_g, p.ln2_b, p.eps, h2));
    DOCC_TRY(linear_device(ctx, prec, T, dff, d, h2, d, p.w_1, d, static_cast<const float*>(p.b_1), DOCC_B200_ACT_GELU_ERF, nullptr,
                           0, f, dff, fused));
    DOCC_TRY(linear_device(ctx, prec, T, d, dff, f, dff, p.w_2, dff, static_cast<const float*>(p.b_2), DOCC_B200_ACT_NONE, h, d, Y, d));
    return DOCC_B200_OK;
}

}  // namespace
}  // namespace docc_b200

using namespace docc_b200;

extern "C" int docc_b200_transformer_block(int prec, const docc_b200_block_params* p, const void* X, void* Y, int flags) {
    Ctx* ctx;
    DOCC_TRY(get_ctx(&ctx));
    DOCC_REQUIRE(p != nullptr, "transformer_block: params is NULL");
    DOCC_REQUIRE(prec == DOCC_B200_PREC_S || prec == DOCC_B200_PREC_B, "transformer_block: precision %d not supported (use 's' or 'b')", prec);
    DOCC_REQUIRE(p->batch >= 0 && p->seq >= 0 && p->d_model > 0 && p->n_heads > 0 && p->d_ff > 0, "transformer_block: bad extent");
    DOCC_REQUIRE(p->d_model % p->n_heads == 0, "transformer_block: d_model %% n_heads != 0");
    DOCC_REQUIRE(p->w_qkv && p->w_o && p->w_1 && p->w_2, "transformer_block: NULL weight pointer");
    const int64_t T = p->batch * p->seq;
    if (T == 0) return DOCC_B200_OK;
    DOCC_REQUIRE(X && Y, "transformer_block: NULL data pointer");
    if (!(flags & DOCC_B200_FLAG_HOST_PTRS)) return block_device(ctx, prec, *p, X, Y);

    const size_t es = prec_size(prec);
    const int64_t d = p->d_model, dff = p->d_ff;
    docc_b200_block_params dp = *p;
    void *dX, *dY;
    struct Item { const void** field; size_t bytes; };
    Item items[] = {{&dp.ln1_g, size_t(d) * 4}, {&dp.ln1_b, size_t(d) * 4}, {&dp.w_qkv, size_t(3 * d * d) * es},
                    {&dp.b_qkv, size_t(3 * d) * 4}, {&dp.w_o, size_t(d * d) * es}, {&dp.b_o, size_t(d) * 4},
                    {&dp.ln2_g, size_t(d) * 4}, {&dp.ln2_b, size_t(d) * 4}, {&dp.w_1, size_t(dff * d) * es},
                    {&dp.b_1, size_t(dff) * 4}, {&dp.w_2, size_t(d * dff) * es}, {&dp.b_2, size_t(d) * 4}};
    void* staged[14];
    int n_staged = 0;
    int status = DOCC_B200_OK;
    auto stage = [&](const void* host, size_t bytes, void** dev) -> int {
        DOCC_TRY(pool_alloc(dev, bytes));
        staged[n_staged++] = *dev;
        DOCC_CUDA_TRY(cudaMemcpyAsync(*dev, host, bytes, cudaMemcpyHostToDevice, ctx->stream));
        return DOCC_B200_OK;
    };
    for (auto& it : items) {
        if (!*it.field) continue;
        void* dev;
        status = stage(*it.field, it.bytes, &dev);
        if (status != DOCC_B200_OK) break;
        *it.field = dev;
    }
    if (status == DOCC_B200_OK) status = stage(X, size_t(T * d) * es, &dX);
    if (status == DOCC_B200_OK) {
        status = pool_alloc(&dY, size_t(T * d) * es);
        if (status == DOCC_B200_OK) staged[n_staged++] = dY;
    }
    if (status == DOCC_B200_OK) status = block_device(ctx, prec, dp, dX, dY);
    if (status == DOCC_B200_OK) {
        cudaError_t e = cudaMemcpyAsync(Y, dY, size_t(T * d) * es, cudaMemcpyDeviceToHost, ctx->stream);
        if (e != cudaSuccess) status = set_error(DOCC_B200_ERR_CUDA, "D2H: %s", cudaGetErrorString(e));
    }
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess && status == DOCC_B200_OK) status = set_error(DOCC_B200_ERR_CUDA, "sync: %s", cudaGetErrorString(e));
    for (int i = 0; i < n_staged; i++) pool_free(staged[i]);
    return status;
}
