// Conv entry point of the C ABI: N-D cross-correlation in NC(D..) layout (ConvNode,
// conv_node.h:87-200). docc expands the node into one loop nest with a sequential
// C_in*k0*k1.. FMA chain per output element (conv_node.cpp:243-399), which its CUDA scheduler
// turns into a one-thread-per-output kernel with uncoalesced weight reads.
//
// Two kernels here:
//   * implicit-GEMM on the tcgen05 engine (conv_tc.cu) for 2-D, stride 1, dilation 1, group 1,
//     C_in % 16 == 0 — the shape class of ResNet-style layers;
//   * a direct kernel for every other configuration (any rank <= 3, stride, dilation, groups).
#include "conv.h"
#include "device_math.cuh"

namespace docc_b200 {
namespace {

struct ConvGeom {
    int sr;
    int64_t N, C, c_out, group;
    int64_t in_d[3], k_d[3], s_d[3], pb[3], d_d[3], o_d[3];  // right-aligned into three spatial slots
};

template <typename TI, typename TA, typename TO>
__global__ void __launch_bounds__(256) conv_direct_kernel(const TI* __restrict__ X, const TI* __restrict__ W,
                                                          const TO* __restrict__ Bias, TO* __restrict__ Y, ConvGeom g) {
    const int64_t o_sp = g.o_d[0] * g.o_d[1] * g.o_d[2];
    const int64_t in_sp = g.in_d[0] * g.in_d[1] * g.in_d[2];
    const int64_t k_sp = g.k_d[0] * g.k_d[1] * g.k_d[2];
    const int64_t cg = g.C / g.group, og = g.c_out / g.group;
    const int64_t total = g.N * g.c_out * o_sp;
    for (int64_t idx = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; idx < total; idx += int64_t(gridDim.x) * blockDim.x) {
        int64_t t = idx;
        const int64_t o2 = t % g.o_d[2]; t /= g.o_d[2];
        const int64_t o1 = t % g.o_d[1]; t /= g.o_d[1];
        const int64_t o0 = t % g.o_d[0]; t /= g.o_d[0];
        const int64_t oc = t % g.c_out;
        const int64_t n = t / g.c_out;
        const int64_t grp = oc / og;
        TA acc = TA(0);
        for (int64_t ic = 0; ic < cg; ic++) {
            const TI* xc = X + (n * g.C + grp * cg + ic) * in_sp;
            const TI* wc = W + (oc * cg + ic) * k_sp;
            for (int64_t k0 = 0; k0 < g.k_d[0]; k0++) {
                const int64_t i0 = o0 * g.s_d[0] - g.pb[0] + k0 * g.d_d[0];
                if (i0 < 0 || i0 >= g.in_d[0]) continue;
                for (int64_t k1 = 0; k1 < g.k_d[1]; k1++) {
                    const int64_t i1 = o1 * g.s_d[1] - g.pb[1] + k1 * g.d_d[1];
                    if (i1 < 0 || i1 >= g.in_d[1]) continue;
                    for (int64_t k2 = 0; k2 < g.k_d[2]; k2++) {
                        const int64_t i2 = o2 * g.s_d[2] - g.pb[2] + k2 * g.d_d[2];
                        if (i2 < 0 || i2 >= g.in_d[2]) continue;
                        const TA x = TA(to_float_or_double(xc[(i0 * g.in_d[1] + i1) * g.in_d[2] + i2], TA(0)));
                        const TA w = TA(to_float_or_double(wc[(k0 * g.k_d[1] + k1) * g.k_d[2] + k2], TA(0)));
                        acc = fma(x, w, acc);
                    }
                }
            }
        }
        if (Bias) acc += TA(to_float_or_double(Bias[oc], TA(0)));
        Y[idx] = from_acc_value<TO>(acc);
    }
}

template <typename TI, typename TA, typename TO>
int launch_direct(Ctx* ctx, const void* X, const void* W, const void* B, void* Y, const ConvGeom& g) {
    const int64_t total = g.N * g.c_out * g.o_d[0] * g.o_d[1] * g.o_d[2];
    if (total == 0) return DOCC_B200_OK;
    const int64_t blocks = ceil_div(total, 256);
    const int64_t cap = int64_t(ctx->sm_count) * 32;
    conv_direct_kernel<TI, TA, TO><<<int(blocks < cap ? blocks : cap), 256, 0, ctx->stream>>>(
        static_cast<const TI*>(X), static_cast<const TI*>(W), static_cast<const TO*>(B), static_cast<TO*>(Y), g);
    return after_launch(ctx, "conv_direct_kernel");
}

int conv_device(Ctx* ctx, int prec_in, int prec_out, const ConvGeom& g, const void* X, const void* W, const void* B, void* Y,
                int flags) {
    // fast path: 2-D, unit stride/dilation, one group, channel count TMA can tile
    if (g.sr == 2 && g.group == 1 && g.s_d[1] == 1 && g.s_d[2] == 1 && g.d_d[1] == 1 && g.d_d[2] == 1 &&
        (prec_in == DOCC_B200_PREC_S || prec_in == DOCC_B200_PREC_B) && prec_out == DOCC_B200_PREC_S &&
        !(flags & DOCC_B200_FLAG_FP32_EXACT)) {
        ConvTcProblem p;
        p.N = g.N; p.C = g.C; p.H = g.in_d[1]; p.W = g.in_d[2]; p.c_out = g.c_out;
        p.kh = g.k_d[1]; p.kw = g.k_d[2]; p.pad_h = g.pb[1]; p.pad_w = g.pb[2]; p.Ho = g.o_d[1]; p.Wo = g.o_d[2];
        p.prec_in = prec_in;
        int s = conv_tc(ctx, p, X, W, static_cast<const float*>(B), static_cast<float*>(Y));
        if (s != DOCC_B200_ERR_UNSUPPORTED) return s;
    }
    if (prec_in == DOCC_B200_PREC_D) return launch_direct<double, double, double>(ctx, X, W, B, Y, g);
    if (prec_in == DOCC_B200_PREC_S) return launch_direct<float, float, float>(ctx, X, W, B, Y, g);
    if (prec_in == DOCC_B200_PREC_B) {
        if (prec_out == DOCC_B200_PREC_S) return launch_direct<__nv_bfloat16, float, float>(ctx, X, W, B, Y, g);
        return launch_direct<__nv_bfloat16, float, __nv_bfloat16>(ctx, X, W, B, Y, g);
    }
    if (prec_out == DOCC_B200_PREC_S) return launch_direct<__half, float, float>(ctx, X, W, B, Y, g);
    return launch_direct<__half, float, __half>(ctx, X, W, B, Y, g);
}

}  // namespace
}  // namespace docc_b200

using namespace docc_b200;

extern "C" int docc_b200_conv(int prec_in, int prec_out, int spatial_rank, const int64_t* x_shape, const int64_t* k_shape,
                              const int64_t* strides, const int64_t* pads, const int64_t* dilations, int64_t c_out,
                              int64_t group, const void* X, const void* W, const void* B_or_null, void* Y, int flags) {
    Ctx* ctx;
    DOCC_TRY(get_ctx(&ctx));
    DOCC_REQUIRE(spatial_rank >= 1 && spatial_rank <= 3, "conv: spatial rank %d outside [1,3]", spatial_rank);
    DOCC_REQUIRE(x_shape && k_shape && strides && pads && dilations, "conv: NULL shape array");
    DOCC_REQUIRE(prec_size(prec_in) != 0, "conv: unknown input precision %d", prec_in);
    DOCC_REQUIRE(prec_out == prec_in || (prec_out == DOCC_B200_PREC_S && prec_size(prec_in) == 2),
                 "conv: output precision must equal the input precision, or be 's' for 16-bit inputs");
    DOCC_REQUIRE(group >= 1 && c_out >= 0, "conv: group must be >= 1");
    ConvGeom g;
    g.sr = spatial_rank;
    g.N = x_shape[0]; g.C = x_shape[1]; g.c_out = c_out; g.group = group;
    DOCC_REQUIRE(g.N >= 0 && g.C >= 0, "conv: negative extent");
    DOCC_REQUIRE(g.C % group == 0 && c_out % group == 0, "conv: channels not divisible by group");
    for (int i = 0; i < 3; i++) { g.in_d[i] = 1; g.k_d[i] = 1; g.s_d[i] = 1; g.pb[i] = 0; g.d_d[i] = 1; g.o_d[i] = 1; }
    for (int i = 0; i < spatial_rank; i++) {
        const int s = 3 - spatial_rank + i;
        DOCC_REQUIRE(x_shape[2 + i] >= 0 && k_shape[i] >= 1 && strides[i] >= 1 && dilations[i] >= 1 && pads[i] >= 0 &&
                         pads[spatial_rank + i] >= 0,
                     "conv: bad extent/stride/pad/dilation in spatial dim %d", i);
        g.in_d[s] = x_shape[2 + i]; g.k_d[s] = k_shape[i]; g.s_d[s] = strides[i]; g.pb[s] = pads[i]; g.d_d[s] = dilations[i];
        // output extent: conv_node.cpp:225-233
        const int64_t num = x_shape[2 + i] + pads[i] + pads[spatial_rank + i] - dilations[i] * (k_shape[i] - 1) - 1;
        g.o_d[s] = num < 0 ? 0 : num / strides[i] + 1;
    }
    const int64_t in_sp = g.in_d[0] * g.in_d[1] * g.in_d[2], k_sp = g.k_d[0] * g.k_d[1] * g.k_d[2];
    const int64_t o_sp = g.o_d[0] * g.o_d[1] * g.o_d[2];
    const int64_t y_n = g.N * c_out * o_sp;
    if (y_n == 0) return DOCC_B200_OK;
    DOCC_REQUIRE(X && W && Y, "conv: NULL data pointer");
    if (!(flags & DOCC_B200_FLAG_HOST_PTRS)) return conv_device(ctx, prec_in, prec_out, g, X, W, B_or_null, Y, flags);
    const size_t ei = prec_size(prec_in), eo = prec_size(prec_out);
    TempBuffers tmp;
    void *dX, *dW, *dB = nullptr, *dY;
    const size_t x_b = size_t(g.N * g.C * in_sp) * ei, w_b = size_t(c_out * (g.C / group) * k_sp) * ei;
    DOCC_TRY(tmp.alloc(&dX, x_b));
    DOCC_TRY(tmp.alloc(&dW, w_b));
    DOCC_TRY(tmp.alloc(&dY, size_t(y_n) * eo));
    DOCC_CUDA_TRY(cudaMemcpyAsync(dX, X, x_b, cudaMemcpyHostToDevice, ctx->stream));
    DOCC_CUDA_TRY(cudaMemcpyAsync(dW, W, w_b, cudaMemcpyHostToDevice, ctx->stream));
    if (B_or_null) {
        DOCC_TRY(tmp.alloc(&dB, size_t(c_out) * eo));
        DOCC_CUDA_TRY(cudaMemcpyAsync(dB, B_or_null, size_t(c_out) * eo, cudaMemcpyHostToDevice, ctx->stream));
    }
    DOCC_TRY(conv_device(ctx, prec_in, prec_out, g, dX, dW, dB, dY, flags));
    DOCC_CUDA_TRY(cudaMemcpyAsync(Y, dY, size_t(y_n) * eo, cudaMemcpyDeviceToHost, ctx->stream));
    DOCC_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    return DOCC_B200_OK;
}
