// Device-side helpers shared by the bandwidth kernels: 16-byte packs, type conversion,
// activations and warp / block reductions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdint>

#include "docc_b200/rt.h"

namespace docc_b200 {

template <typename T, int VEC> struct alignas(sizeof(T) * VEC) Pack { T v[VEC]; };

// 16-byte packs use streaming (evict-first) accesses: every byte is touched exactly once.
template <typename P> __device__ __forceinline__ P load_pack(const P* p) {
    if constexpr (sizeof(P) == 16) {
        const float4 f = __ldcs(reinterpret_cast<const float4*>(p));
        return *reinterpret_cast<const P*>(&f);
    } else {
        return *p;
    }
}
template <typename P> __device__ __forceinline__ void store_pack(P* p, const P& v) {
    if constexpr (sizeof(P) == 16) {
        __stcs(reinterpret_cast<float4*>(p), *reinterpret_cast<const float4*>(&v));
    } else {
        *p = v;
    }
}

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(double v) { return float(v); }
__device__ __forceinline__ float to_float(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ double from_float<double>(float v) { return double(v); }
template <> __device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename TO, typename TI> __device__ __forceinline__ TO cast_to(TI v) {
    if constexpr (sizeof(TI) == 8 && sizeof(TO) == 8) return v;
    else if constexpr (sizeof(TI) == 8) return from_float<TO>(float(v));  // double -> narrower goes through fp32 rounding once for 16-bit targets
    else if constexpr (sizeof(TO) == 8) return double(to_float(v));
    else return from_float<TO>(to_float(v));
}
template <> __device__ __forceinline__ float cast_to<float, double>(double v) { return float(v); }

__device__ __forceinline__ float apply_act(int act, float x) {
    switch (act) {
        case DOCC_B200_ACT_GELU_ERF: return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f));
        case DOCC_B200_ACT_RELU: return x > 0.f ? x : 0.f;
        case DOCC_B200_ACT_TANH: return tanhf(x);
        case DOCC_B200_ACT_SIGMOID: return 1.0f / (1.0f + expf(-x));
        case DOCC_B200_ACT_EXP: return expf(x);
        case DOCC_B200_ACT_ERF: return erff(x);
        case DOCC_B200_ACT_SQRT: return sqrtf(x);
        case DOCC_B200_ACT_ABS: return fabsf(x);
        default: return x;
    }
}
// erf by Abramowitz & Stegun 7.1.26 (|error| <= 1.5e-7): two SFU operations and a degree-5 polynomial,
// about a third of the instructions of erff. Used in GEMM epilogues, where the activation runs on the
// critical path of the accumulator drain.
__device__ __forceinline__ float erf_fast(float x) {
    const float ax = fabsf(x);
    float t;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(fmaf(0.3275911f, ax, 1.0f)));
    float poly = fmaf(t, 1.061405429f, -1.453152027f);
    poly = fmaf(t, poly, 1.421413741f);
    poly = fmaf(t, poly, -0.284496736f);
    poly = fmaf(t, poly, 0.254829592f);
    poly *= t;
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-ax * ax * 1.4426950408889634f));
    return copysignf(fmaf(-poly, e, 1.0f), x);
}
// GELU for results that are rounded to a 16-bit type: erf(z) = tanh(z * (c0 + c1 z^2 + c2 z^4)) with the polynomial
// fitted to |error| <= 3.7e-5 over the whole line, evaluated with the hardware tanh (relative error 2^-11).
// |error of the result| <= 2.7e-4 * |x|, a fraction of half a bf16 / fp16 ulp wherever the result is not tiny, at
// eight instructions per element against eighteen for the erf_fast form: the GELU epilogue of a K = 1024 GEMM then
// drains a tile faster than the tensor core produces the next one. fp32 results keep erf_fast.
__device__ __forceinline__ float gelu_erf_16bit(float x) {
    const float z = x * 0.70710678118654752440f;
    const float u = z * z;
    float poly = fmaf(u, -0.00178647f, 0.10408119f);
    poly = fmaf(u, poly, 1.12814338f);
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(z * poly));
    const float h = 0.5f * x;
    return fmaf(h, t, h);
}
__device__ __forceinline__ float apply_act_fast(int act, float x) {
    if (act == DOCC_B200_ACT_GELU_ERF) return 0.5f * x * (1.0f + erf_fast(x * 0.70710678118654752440f));
    if (act == DOCC_B200_ACT_ERF) return erf_fast(x);
    return apply_act(act, x);
}

__device__ __forceinline__ double apply_act_f64(int act, double x) {
    switch (act) {
        case DOCC_B200_ACT_GELU_ERF: return 0.5 * x * (1.0 + erf(x * 0.70710678118654752440));
        case DOCC_B200_ACT_RELU: return x > 0. ? x : 0.;
        case DOCC_B200_ACT_TANH: return tanh(x);
        case DOCC_B200_ACT_SIGMOID: return 1.0 / (1.0 + exp(-x));
        case DOCC_B200_ACT_EXP: return exp(x);
        case DOCC_B200_ACT_ERF: return erf(x);
        case DOCC_B200_ACT_SQRT: return sqrt(x);
        case DOCC_B200_ACT_ABS: return fabs(x);
        default: return x;
    }
}

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Sum over a block of up to 1024 threads; `smem` holds at least blockDim.x/32 floats.
__device__ __forceinline__ float block_sum_f(float v, float* smem) {
    v = warp_sum_f(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    float r = 0.f;
    for (int w = 0; w < nwarps; w++) r += smem[w];
    return r;
}

}  // namespace docc_b200

namespace docc_b200 {
// Widening loads / narrowing stores used by kernels templated on an accumulate type.
__device__ __forceinline__ double to_float_or_double(double v, double) { return v; }
template <typename T> __device__ __forceinline__ float to_float_or_double(T v, float) { return to_float(v); }
template <typename TO> __device__ __forceinline__ TO from_acc_value(float v) { return from_float<TO>(v); }
template <typename TO> __device__ __forceinline__ TO from_acc_value(double v) { return TO(v); }
}  // namespace docc_b200
