#include <cuda_runtime.h>
#include <docc_b200/rt.h>
// element-wise map: 16-byte accesses of the widest operand, grid-stride loop, scalar tail
#ifndef DOCC_B200_VEC_DEFINED
#define DOCC_B200_VEC_DEFINED
template <typename T, int V> struct alignas(sizeof(T) * V) docc_b200_vec { T v[V]; };
#endif
template <int V>
__global__ void __launch_bounds__(256) kernel_axpby_3(const float* __restrict__ a_ptr, const float* __restrict__ b_ptr, float* __restrict__ out_ptr, float alpha, long long _s0, long long __n) {
    const long long __groups = __n / V;
    const long long __stride = (long long)gridDim.x * blockDim.x;
    for (long long __g = (long long)blockIdx.x * blockDim.x + threadIdx.x; __g < __groups; __g += __stride) {
        const docc_b200_vec<float, V> a_in = *reinterpret_cast<const docc_b200_vec<float, V>*>(a_ptr + __g * V);
        const docc_b200_vec<float, V> b_in = *reinterpret_cast<const docc_b200_vec<float, V>*>(b_ptr + __g * V);
        docc_b200_vec<float, V> out_out;
#pragma unroll
        for (int __e = 0; __e < V; __e++) {
            const float a = a_in.v[__e];
            const float b = b_in.v[__e];
            float out;
            out = fmaf(alpha, a, b);
            out_out.v[__e] = out;
        }
        *reinterpret_cast<docc_b200_vec<float, V>*>(out_ptr + __g * V) = out_out;
    }
    // tail: the last __n % V elements, one per thread of the first block
    if (blockIdx.x == 0) {
        for (long long __i = __groups * V + threadIdx.x; __i < __n; __i += blockDim.x) {
            const float a = a_ptr[__i];
            const float b = b_ptr[__i];
            float out;
            out = fmaf(alpha, a, b);
            out_ptr[__i] = out;
        }
    }
}
extern "C" void kernel_axpby_3_launch(const float* a_ptr, const float* b_ptr, float* out_ptr, float alpha, long long _s0) {
    const long long __n = (long long)(_s0);
    if (__n <= 0) return;
    void* __stream = 0;
    docc_b200_get_stream(&__stream);
    bool __vec = true;
    __vec = __vec && ((unsigned long long)(a_ptr) % 16 == 0);
    __vec = __vec && ((unsigned long long)(b_ptr) % 16 == 0);
    __vec = __vec && ((unsigned long long)(out_ptr) % 16 == 0);
    int __sms = 0, __dev = 0;
    cudaGetDevice(&__dev);
    cudaDeviceGetAttribute(&__sms, cudaDevAttrMultiProcessorCount, __dev);
    const long long __work = __vec ? (__n + 4 - 1) / 4 : __n;
    long long __blocks = (__work + 255) / 256;
    if (__blocks > 8LL * __sms) __blocks = 8LL * __sms;
    if (__vec) kernel_axpby_3<4><<<(unsigned)__blocks, 256, 0, (cudaStream_t)__stream>>>(a_ptr, b_ptr, out_ptr, alpha, _s0, __n);
    else kernel_axpby_3<1><<<(unsigned)__blocks, 256, 0, (cudaStream_t)__stream>>>(a_ptr, b_ptr, out_ptr, alpha, _s0, __n);
}
// element-wise map: 16-byte accesses of the widest operand, grid-stride loop, scalar tail
#ifndef DOCC_B200_VEC_DEFINED
#define DOCC_B200_VEC_DEFINED
template <typename T, int V> struct alignas(sizeof(T) * V) docc_b200_vec { T v[V]; };
#endif
template <int V>
__global__ void __launch_bounds__(256) kernel_widen_7(const float* __restrict__ x_ptr, double* __restrict__ y_ptr, long long _s0, long long _s1, long long __n) {
    const long long __groups = __n / V;
    const long long __stride = (long long)gridDim.x * blockDim.x;
    for (long long __g = (long long)blockIdx.x * blockDim.x + threadIdx.x; __g < __groups; __g += __stride) {
        const docc_b200_vec<float, V> x_in = *reinterpret_cast<const docc_b200_vec<float, V>*>(x_ptr + __g * V);
        docc_b200_vec<double, V> y_out;
#pragma unroll
        for (int __e = 0; __e < V; __e++) {
            const float x = x_in.v[__e];
            double y;
            y = sqrt(fabs((double)x)) + 0.5;
            y_out.v[__e] = y;
        }
        *reinterpret_cast<docc_b200_vec<double, V>*>(y_ptr + __g * V) = y_out;
    }
    // tail: the last __n % V elements, one per thread of the first block
    if (blockIdx.x == 0) {
        for (long long __i = __groups * V + threadIdx.x; __i < __n; __i += blockDim.x) {
            const float x = x_ptr[__i];
            double y;
            y = sqrt(fabs((double)x)) + 0.5;
            y_ptr[__i] = y;
        }
    }
}
extern "C" void kernel_widen_7_launch(const float* x_ptr, double* y_ptr, long long _s0, long long _s1) {
    const long long __n = (long long)(_s0 * _s1);
    if (__n <= 0) return;
    void* __stream = 0;
    docc_b200_get_stream(&__stream);
    bool __vec = true;
    __vec = __vec && ((unsigned long long)(x_ptr) % 8 == 0);
    __vec = __vec && ((unsigned long long)(y_ptr) % 16 == 0);
    int __sms = 0, __dev = 0;
    cudaGetDevice(&__dev);
    cudaDeviceGetAttribute(&__sms, cudaDevAttrMultiProcessorCount, __dev);
    const long long __work = __vec ? (__n + 2 - 1) / 2 : __n;
    long long __blocks = (__work + 255) / 256;
    if (__blocks > 8LL * __sms) __blocks = 8LL * __sms;
    if (__vec) kernel_widen_7<2><<<(unsigned)__blocks, 256, 0, (cudaStream_t)__stream>>>(x_ptr, y_ptr, _s0, _s1, __n);
    else kernel_widen_7<1><<<(unsigned)__blocks, 256, 0, (cudaStream_t)__stream>>>(x_ptr, y_ptr, _s0, _s1, __n);
}
// element-wise map: 16-byte accesses of the widest operand, grid-stride loop, scalar tail
#ifndef DOCC_B200_VEC_DEFINED
#define DOCC_B200_VEC_DEFINED
template <typename T, int V> struct alignas(sizeof(T) * V) docc_b200_vec { T v[V]; };
#endif
template <int V>
__global__ void __launch_bounds__(256) kernel_sumdiff_9(const unsigned short* __restrict__ p_ptr, const unsigned short* __restrict__ q_ptr, unsigned short* __restrict__ s_ptr, unsigned short* __restrict__ d_ptr, long long _s0, long long __n) {
    const long long __groups = __n / V;
    const long long __stride = (long long)gridDim.x * blockDim.x;
    for (long long __g = (long long)blockIdx.x * blockDim.x + threadIdx.x; __g < __groups; __g += __stride) {
        const docc_b200_vec<unsigned short, V> p_in = *reinterpret_cast<const docc_b200_vec<unsigned short, V>*>(p_ptr + __g * V);
        const docc_b200_vec<unsigned short, V> q_in = *reinterpret_cast<const docc_b200_vec<unsigned short, V>*>(q_ptr + __g * V);
        docc_b200_vec<unsigned short, V> s_out;
        docc_b200_vec<unsigned short, V> d_out;
#pragma unroll
        for (int __e = 0; __e < V; __e++) {
            const unsigned short p = p_in.v[__e];
            const unsigned short q = q_in.v[__e];
            unsigned short s;
            unsigned short d;
            s = (unsigned short)(p + q); d = (unsigned short)(p - q);
            s_out.v[__e] = s;
            d_out.v[__e] = d;
        }
        *reinterpret_cast<docc_b200_vec<unsigned short, V>*>(s_ptr + __g * V) = s_out;
        *reinterpret_cast<docc_b200_vec<unsigned short, V>*>(d_ptr + __g * V) = d_out;
    }
    // tail: the last __n % V elements, one per thread of the first block
    if (blockIdx.x == 0) {
        for (long long __i = __groups * V + threadIdx.x; __i < __n; __i += blockDim.x) {
            const unsigned short p = p_ptr[__i];
            const unsigned short q = q_ptr[__i];
            unsigned short s;
            unsigned short d;
            s = (unsigned short)(p + q); d = (unsigned short)(p - q);
            s_ptr[__i] = s;
            d_ptr[__i] = d;
        }
    }
}
extern "C" void kernel_sumdiff_9_launch(const unsigned short* p_ptr, const unsigned short* q_ptr, unsigned short* s_ptr, unsigned short* d_ptr, long long _s0) {
    const long long __n = (long long)(_s0);
    if (__n <= 0) return;
    void* __stream = 0;
    docc_b200_get_stream(&__stream);
    bool __vec = true;
    __vec = __vec && ((unsigned long long)(p_ptr) % 16 == 0);
    __vec = __vec && ((unsigned long long)(q_ptr) % 16 == 0);
    __vec = __vec && ((unsigned long long)(s_ptr) % 16 == 0);
    __vec = __vec && ((unsigned long long)(d_ptr) % 16 == 0);
    int __sms = 0, __dev = 0;
    cudaGetDevice(&__dev);
    cudaDeviceGetAttribute(&__sms, cudaDevAttrMultiProcessorCount, __dev);
    const long long __work = __vec ? (__n + 8 - 1) / 8 : __n;
    long long __blocks = (__work + 255) / 256;
    if (__blocks > 8LL * __sms) __blocks = 8LL * __sms;
    if (__vec) kernel_sumdiff_9<8><<<(unsigned)__blocks, 256, 0, (cudaStream_t)__stream>>>(p_ptr, q_ptr, s_ptr, d_ptr, _s0, __n);
    else kernel_sumdiff_9<1><<<(unsigned)__blocks, 256, 0, (cudaStream_t)__stream>>>(p_ptr, q_ptr, s_ptr, d_ptr, _s0, __n);
}
// element-wise map: 16-byte accesses of the widest operand, grid-stride loop, scalar tail
#ifndef DOCC_B200_VEC_DEFINED
#define DOCC_B200_VEC_DEFINED
template <typename T, int V> struct alignas(sizeof(T) * V) docc_b200_vec { T v[V]; };
#endif
template <int V>
__global__ void __launch_bounds__(256) kernel_scale_12(const float* __restrict__ __daisy_cuda_w_ptr, float* __restrict__ __daisy_cuda_acc_ptr, float lr, int N, long long __n) {
    const long long __groups = __n / V;
    const long long __stride = (long long)gridDim.x * blockDim.x;
    for (long long __g = (long long)blockIdx.x * blockDim.x + threadIdx.x; __g < __groups; __g += __stride) {
        const docc_b200_vec<float, V> __daisy_cuda_w_in = *reinterpret_cast<const docc_b200_vec<float, V>*>(__daisy_cuda_w_ptr + __g * V);
        docc_b200_vec<float, V> __daisy_cuda_acc_out = *reinterpret_cast<const docc_b200_vec<float, V>*>(__daisy_cuda_acc_ptr + __g * V);
        const float* const __daisy_cuda_w = __daisy_cuda_w_in.v;
        float* const __daisy_cuda_acc = __daisy_cuda_acc_out.v;
#pragma unroll
        for (int __e = 0; __e < V; __e++) {
            const int i = __e;
            { float _in1 = __daisy_cuda_acc[i]; float _in2 = __daisy_cuda_w[i]; float _out = fmaf(-lr, _in2, _in1); __daisy_cuda_acc[i] = _out; }
        }
        *reinterpret_cast<docc_b200_vec<float, V>*>(__daisy_cuda_acc_ptr + __g * V) = __daisy_cuda_acc_out;
    }
    // tail: the last __n % V elements, one per thread of the first block
    if (blockIdx.x == 0) {
        const float* const __daisy_cuda_w = __daisy_cuda_w_ptr;
        float* const __daisy_cuda_acc = __daisy_cuda_acc_ptr;
        for (long long __i = __groups * V + threadIdx.x; __i < __n; __i += blockDim.x) {
            const long long i = __i;
            { float _in1 = __daisy_cuda_acc[i]; float _in2 = __daisy_cuda_w[i]; float _out = fmaf(-lr, _in2, _in1); __daisy_cuda_acc[i] = _out; }
        }
    }
}
extern "C" void kernel_scale_12_launch(const float* __daisy_cuda_w_ptr, float* __daisy_cuda_acc_ptr, float lr, int N) {
    const long long __n = (long long)(N);
    if (__n <= 0) return;
    void* __stream = 0;
    docc_b200_get_stream(&__stream);
    bool __vec = true;
    __vec = __vec && ((unsigned long long)(__daisy_cuda_w_ptr) % 16 == 0);
    __vec = __vec && ((unsigned long long)(__daisy_cuda_acc_ptr) % 16 == 0);
    int __sms = 0, __dev = 0;
    cudaGetDevice(&__dev);
    cudaDeviceGetAttribute(&__sms, cudaDevAttrMultiProcessorCount, __dev);
    const long long __work = __vec ? (__n + 4 - 1) / 4 : __n;
    long long __blocks = (__work + 255) / 256;
    if (__blocks > 8LL * __sms) __blocks = 8LL * __sms;
    if (__vec) kernel_scale_12<4><<<(unsigned)__blocks, 256, 0, (cudaStream_t)__stream>>>(__daisy_cuda_w_ptr, __daisy_cuda_acc_ptr, lr, N, __n);
    else kernel_scale_12<1><<<(unsigned)__blocks, 256, 0, (cudaStream_t)__stream>>>(__daisy_cuda_w_ptr, __daisy_cuda_acc_ptr, lr, N, __n);
}
extern "C" void axpby_op(const float* a_ptr, const float* b_ptr, float* out_ptr, float alpha, long long _s0) {
    kernel_axpby_3_launch(a_ptr, b_ptr, out_ptr, alpha, _s0);
}
extern "C" void widen_op(const float* x_ptr, double* y_ptr, long long _s0, long long _s1) {
    kernel_widen_7_launch(x_ptr, y_ptr, _s0, _s1);
}
extern "C" void sumdiff_op(const unsigned short* p_ptr, const unsigned short* q_ptr, unsigned short* s_ptr, unsigned short* d_ptr, long long _s0) {
    kernel_sumdiff_9_launch(p_ptr, q_ptr, s_ptr, d_ptr, _s0);
}
extern "C" void scale_op(const float* __daisy_cuda_w_ptr, float* __daisy_cuda_acc_ptr, float lr, int N) {
    kernel_scale_12_launch(__daisy_cuda_w_ptr, __daisy_cuda_acc_ptr, lr, N);
}
