// TEST INFRASTRUCTURE — NOT PART OF THE PRODUCT.
//
// CPU restatement of the semantics docc's library nodes have on its CPU targets
// (`none` / `sequential` / `openmp`). Only tests, the smoke check and the
// cpu_baseline / reference arm of the benchmark may call into this file; the
// runtime library never does.
//
// Every function follows the loop nests that the reference's expand() methods
// build (paths relative to the docc source tree):
//   GEMM      sdfg/src/data_flow/library_nodes/math/blas/gemm_node.cpp:179-311
//   MatMul    sdfg/src/data_flow/library_nodes/math/tensor/matmul_node.cpp:353-489
//   Softmax   .../tensor/reduce_ops/softmax_node.cpp:142-252 with
//             .../tensor/reduce_node.cpp:187-333, max_node.cpp:51-90, sum_node.cpp:30-48
//   Conv      .../tensor/conv_node.cpp:225-233,243-295,309-353,412-437
//   Mean/Std  .../tensor/reduce_ops/mean_node.cpp:77-118, std_node.cpp:147-222
// Parallelisation is what OMPScheduler produces: `#pragma omp parallel for
// schedule(static)` on the outermost map only
// (opt/src/passes/scheduler/omp_scheduler.cpp:15-21,
//  opt/src/targets/omp/codegen/omp_map_dispatcher.cpp:47-58).
//
// Pinning: the reference holds no golden vector files for this path. Its tests
// compare against numpy / scipy / torch with allclose; this oracle is pinned the
// same way (tests/test_oracle.py, fixtures in tests/golden/). Rows the reference
// does not test at all — padded or biased conv, attention, LayerNorm, GELU,
// 16-bit inputs — are "parity unpinned": the torch CPU result is the second opinion.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <vector>

#if defined(_OPENMP)
#include <omp.h>
#endif

namespace {

// ---- 16-bit float storage helpers -------------------------------------------------
inline float bf16_to_f32(uint16_t v) {
    uint32_t u = uint32_t(v) << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
inline uint16_t f32_to_bf16(float f) {  // round to nearest even, NaN stays NaN
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return uint16_t((u >> 16) | 0x40);
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return uint16_t(u >> 16);
}
inline float f16_to_f32(uint16_t h) {
    uint32_t sign = uint32_t(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t u;
    if (exp == 0) {
        if (man == 0) {
            u = sign;
        } else {
            int e = -1;
            do { e++; man <<= 1; } while ((man & 0x400u) == 0);
            man &= 0x3ffu;
            u = sign | uint32_t(127 - 15 - e) << 23 | (man << 13);
        }
    } else if (exp == 31) {
        u = sign | 0x7f800000u | (man << 13);
    } else {
        u = sign | ((exp + 112) << 23) | (man << 13);
    }
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
inline uint16_t f32_to_f16(float f) {  // round to nearest even
    uint32_t x;
    std::memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t mant = x & 0x007fffffu;
    int32_t exp = int32_t((x >> 23) & 0xff);
    if (exp == 255) return uint16_t(sign | 0x7c00u | (mant ? 0x200u : 0));
    int32_t e = exp - 127 + 15;
    if (e >= 31) return uint16_t(sign | 0x7c00u);
    if (e <= 0) {
        if (e < -10) return uint16_t(sign);
        mant |= 0x00800000u;
        uint32_t shift = uint32_t(14 - e);
        uint32_t half = mant >> shift;
        uint32_t rem = mant & ((1u << shift) - 1);
        uint32_t mid = 1u << (shift - 1);
        if (rem > mid || (rem == mid && (half & 1))) half++;
        return uint16_t(sign | half);
    }
    uint32_t half = (uint32_t(e) << 10) | (mant >> 13);
    uint32_t rem = mant & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) half++;
    return uint16_t(sign | half);
}

template <int PREC> struct Elem;
template <> struct Elem<'d'> { using store = double; using acc = double;
    static acc ld(const store* p, int64_t i) { return p[i]; } static void st(store* p, int64_t i, acc v) { p[i] = v; } };
template <> struct Elem<'s'> { using store = float; using acc = float;
    static acc ld(const store* p, int64_t i) { return p[i]; } static void st(store* p, int64_t i, acc v) { p[i] = v; } };
template <> struct Elem<'b'> { using store = uint16_t; using acc = float;
    static acc ld(const store* p, int64_t i) { return bf16_to_f32(p[i]); } static void st(store* p, int64_t i, acc v) { p[i] = f32_to_bf16(v); } };
template <> struct Elem<'h'> { using store = uint16_t; using acc = float;
    static acc ld(const store* p, int64_t i) { return f16_to_f32(p[i]); } static void st(store* p, int64_t i, acc v) { p[i] = f32_to_f16(v); } };

inline double fma_t(double a, double b, double c) { return std::fma(a, b, c); }
inline float fma_t(float a, float b, float c) { return std::fmaf(a, b, c); }

// ---- GEMM: gemm_node.cpp:179-311 -----------------------------------------------------
// maps _i < m, _j < n; for _k < k: sum = fma(A[lda*i+k], B[ldb*k+j], sum);
// C[ldc*i+j] = alpha*sum + beta*C[ldc*i+j] (three roundings). expand() itself refuses
// transposes (gemm_node.cpp:105-107); transposed and column-major operands follow the
// cblas_?gemm contract the BLAS dispatcher emits (gemm_node.cpp:474-505). beta == 0 does
// not read C, which is the BLAS rule the shipped (cblas) path obeys.
template <int PREC>
void gemm_t(int layout, int transa, int transb, int64_t m, int64_t n, int64_t k, double alpha_d, const void* A_,
            int64_t lda, const void* B_, int64_t ldb, double beta_d, void* C_, int64_t ldc) {
    using E = Elem<PREC>;
    using acc = typename E::acc;
    const auto* A = static_cast<const typename E::store*>(A_);
    const auto* B = static_cast<const typename E::store*>(B_);
    auto* C = static_cast<typename E::store*>(C_);
    const acc alpha = acc(alpha_d), beta = acc(beta_d);
    const bool ta = transa != 111, tb = transb != 111;
    if (layout == 102) {
        // column-major C = op(A) op(B)  <=>  row-major C^T = op(B)^T op(A)^T
        gemm_t<PREC>(101, transb, transa, n, m, k, alpha_d, B_, ldb, A_, lda, beta_d, C_, ldc);
        return;
    }
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < m; i++) {
        for (int64_t j = 0; j < n; j++) {
            acc sum = acc(0);
            for (int64_t kk = 0; kk < k; kk++) {
                acc a = ta ? E::ld(A, lda * kk + i) : E::ld(A, lda * i + kk);
                acc b = tb ? E::ld(B, ldb * j + kk) : E::ld(B, ldb * kk + j);
                sum = fma_t(a, b, sum);
            }
            acc scaled = sum * alpha;
            if (beta == acc(0)) {
                E::st(C, ldc * i + j, scaled);
            } else {
                acc cin = E::ld(C, ldc * i + j) * beta;
                E::st(C, ldc * i + j, scaled + cin);
            }
        }
    }
}

// ---- index helpers for C-order tensors ------------------------------------------------
struct ReduceGeom {
    std::vector<int64_t> kept_dims, kept_strides, red_dims, red_strides;
    int64_t n_kept = 1, n_red = 1, total = 1;
};
ReduceGeom make_geom(int rank, const int64_t* shape, int naxes, const int64_t* axes) {
    ReduceGeom g;
    std::vector<int64_t> strides(rank, 1);
    for (int d = rank - 2; d >= 0; d--) strides[d] = strides[d + 1] * shape[d + 1];
    std::vector<bool> is_red(rank, false);
    for (int a = 0; a < naxes; a++) {
        int64_t ax = axes[a] < 0 ? axes[a] + rank : axes[a];
        is_red[ax] = true;
    }
    for (int d = 0; d < rank; d++) {
        g.total *= shape[d];
        if (is_red[d]) {
            g.red_dims.push_back(shape[d]);
            g.red_strides.push_back(strides[d]);
            g.n_red *= shape[d];
        } else {
            g.kept_dims.push_back(shape[d]);
            g.kept_strides.push_back(strides[d]);
            g.n_kept *= shape[d];
        }
    }
    return g;
}
inline int64_t offset_of(int64_t lin, const std::vector<int64_t>& dims, const std::vector<int64_t>& strides) {
    int64_t off = 0;
    for (int d = int(dims.size()) - 1; d >= 0; d--) {
        off += (lin % dims[d]) * strides[d];
        lin /= dims[d];
    }
    return off;
}

// ---- Reduce: reduce_node.cpp:187-333 ----------------------------------------------------
// An init loop writes the identity, then maps over the kept dims surround a *sequential*
// for-nest over the reduced dims (outer-to-inner in axis order), accumulating in element
// precision: out = in + out (sum_node.cpp:30-48), out = fmax(in, out) (max_node.cpp:51-71).
enum { RED_SUM = 0, RED_MAX = 1, RED_MIN = 2, RED_MEAN = 3, RED_STD = 4 };

template <typename T>
void reduce_basic(int op, const ReduceGeom& g, const T* X, T* out) {
#pragma omp parallel for schedule(static)
    for (int64_t o = 0; o < g.n_kept; o++) {
        const int64_t base = offset_of(o, g.kept_dims, g.kept_strides);
        T acc = op == RED_SUM ? T(0) : (op == RED_MAX ? -std::numeric_limits<T>::infinity() : std::numeric_limits<T>::infinity());
        for (int64_t r = 0; r < g.n_red; r++) {
            T v = X[base + offset_of(r, g.red_dims, g.red_strides)];
            if (op == RED_SUM) acc = v + acc;
            else if (op == RED_MAX) acc = std::fmax(v, acc);
            else acc = std::fmin(v, acc);
        }
        out[o] = acc;
    }
}

// Mean = Sum then Div by the element count (mean_node.cpp:77-118).
// Std = sqrt(mean(x*x) - mean(x)^2), population (std_node.cpp:147-222).
template <typename T>
void reduce_t(int op, int rank, const int64_t* shape, int naxes, const int64_t* axes, const T* X, T* Y) {
    ReduceGeom g = make_geom(rank, shape, naxes, axes);
    if (op == RED_SUM || op == RED_MAX || op == RED_MIN) {
        reduce_basic<T>(op, g, X, Y);
    } else if (op == RED_MEAN) {
        reduce_basic<T>(RED_SUM, g, X, Y);
        for (int64_t o = 0; o < g.n_kept; o++) Y[o] = Y[o] / T(g.n_red);
    } else {
        std::vector<T> sq(size_t(g.total));
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < g.total; i++) sq[i] = X[i] * X[i];
        std::vector<T> m2(size_t(g.n_kept));
        reduce_basic<T>(RED_SUM, g, sq.data(), m2.data());
        reduce_basic<T>(RED_SUM, g, X, Y);
        for (int64_t o = 0; o < g.n_kept; o++) {
            T mean = Y[o] / T(g.n_red);
            T msq = m2[o] / T(g.n_red);
            Y[o] = std::sqrt(msq - mean * mean);
        }
    }
}

// ---- Softmax: softmax_node.cpp:92-252 ---------------------------------------------------
// Six temporaries (max, max_bcast, sub, exp, sum, sum_bcast) and seven loop nests:
//   max = Max(X); max_b = Broadcast(max); sub = X - max_b; e = exp(sub);
//   sum = Sum(e); sum_b = Broadcast(sum); Y = e / sum_b
// kept literally, including the full-size temporaries, because this function is also the
// timed CPU baseline.
template <typename T>
void softmax_t(int rank, const int64_t* shape, int naxes, const int64_t* axes, const T* X, T* Y) {
    ReduceGeom g = make_geom(rank, shape, naxes, axes);
    const int64_t total = g.total;
    T* t_max = static_cast<T*>(std::malloc(sizeof(T) * size_t(std::max<int64_t>(g.n_kept, 1))));
    T* t_max_b = static_cast<T*>(std::malloc(sizeof(T) * size_t(std::max<int64_t>(total, 1))));
    T* t_sub = static_cast<T*>(std::malloc(sizeof(T) * size_t(std::max<int64_t>(total, 1))));
    T* t_exp = static_cast<T*>(std::malloc(sizeof(T) * size_t(std::max<int64_t>(total, 1))));
    T* t_sum = static_cast<T*>(std::malloc(sizeof(T) * size_t(std::max<int64_t>(g.n_kept, 1))));
    T* t_sum_b = static_cast<T*>(std::malloc(sizeof(T) * size_t(std::max<int64_t>(total, 1))));

    reduce_basic<T>(RED_MAX, g, X, t_max);
    auto bcast = [&](const T* small, T* full) {
#pragma omp parallel for schedule(static)
        for (int64_t o = 0; o < g.n_kept; o++) {
            const int64_t base = offset_of(o, g.kept_dims, g.kept_strides);
            for (int64_t r = 0; r < g.n_red; r++) full[base + offset_of(r, g.red_dims, g.red_strides)] = small[o];
        }
    };
    bcast(t_max, t_max_b);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < total; i++) t_sub[i] = X[i] - t_max_b[i];
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < total; i++) t_exp[i] = std::exp(t_sub[i]);
    reduce_basic<T>(RED_SUM, g, t_exp, t_sum);
    bcast(t_sum, t_sum_b);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < total; i++) Y[i] = t_exp[i] / t_sum_b[i];

    std::free(t_max); std::free(t_max_b); std::free(t_sub); std::free(t_exp); std::free(t_sum); std::free(t_sum_b);
}

// ---- Conv: conv_node.cpp:225-437 ----------------------------------------------------------
// Output dims (:225-233): (D + pb + pe - d*(k-1) - 1)/s + 1. Maps n, oc, o0.. (:243-295);
// sequential reduction ic, k0, k1.. with accum = fma(x, w, accum) (:309-399); bias added
// after accumulation (:412-437). The expansion indexes X at o*s - pb + k*d without a bounds
// guard; this restatement adds the guard (taps outside the input contribute nothing), which
// is the zero-padding contract of the ONNX Conv operator the node documents
// (sdfg/include/sdfg/data_flow/library_nodes/math/tensor/conv_node.h:9-22). Weight index
// follows the documented [C_out, C_in/group, k..] shape.
template <typename TS, typename TA, typename LD, typename ST>
void conv_t(int sr, const int64_t* xs, const int64_t* ks, const int64_t* st, const int64_t* pads, const int64_t* dil,
            int64_t c_out, int64_t group, const TS* X, const TS* W, const void* Bias, bool bias_is_acc_type, void* Y,
            bool out_is_acc_type, LD ld, ST store16) {
    const int64_t N = xs[0], C = xs[1];
    int64_t in_d[3] = {1, 1, 1}, k_d[3] = {1, 1, 1}, s_d[3] = {1, 1, 1}, pb[3] = {0, 0, 0}, d_d[3] = {1, 1, 1},
            o_d[3] = {1, 1, 1};
    // right-align the spatial dims into 3 slots
    for (int i = 0; i < sr; i++) {
        int s = 3 - sr + i;
        in_d[s] = xs[2 + i]; k_d[s] = ks[i]; s_d[s] = st[i]; pb[s] = pads[i]; d_d[s] = dil[i];
        o_d[s] = (xs[2 + i] + pads[i] + pads[sr + i] - dil[i] * (ks[i] - 1) - 1) / st[i] + 1;
    }
    const int64_t cg = C / group, og = c_out / group;
    const int64_t in_sp = in_d[0] * in_d[1] * in_d[2], k_sp = k_d[0] * k_d[1] * k_d[2];
    const int64_t o_sp = o_d[0] * o_d[1] * o_d[2];
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; n++) {
        for (int64_t oc = 0; oc < c_out; oc++) {
            const int64_t g = oc / og;
            for (int64_t o0 = 0; o0 < o_d[0]; o0++)
                for (int64_t o1 = 0; o1 < o_d[1]; o1++)
                    for (int64_t o2 = 0; o2 < o_d[2]; o2++) {
                        TA accum = TA(0);
                        for (int64_t ic = 0; ic < cg; ic++)
                            for (int64_t k0 = 0; k0 < k_d[0]; k0++)
                                for (int64_t k1 = 0; k1 < k_d[1]; k1++)
                                    for (int64_t k2 = 0; k2 < k_d[2]; k2++) {
                                        int64_t i0 = o0 * s_d[0] - pb[0] + k0 * d_d[0];
                                        int64_t i1 = o1 * s_d[1] - pb[1] + k1 * d_d[1];
                                        int64_t i2 = o2 * s_d[2] - pb[2] + k2 * d_d[2];
                                        if (i0 < 0 || i0 >= in_d[0] || i1 < 0 || i1 >= in_d[1] || i2 < 0 || i2 >= in_d[2])
                                            continue;
                                        TA x = ld(X, (n * C + g * cg + ic) * in_sp + (i0 * in_d[1] + i1) * in_d[2] + i2);
                                        TA w = ld(W, (oc * cg + ic) * k_sp + (k0 * k_d[1] + k1) * k_d[2] + k2);
                                        accum = fma_t(x, w, accum);
                                    }
                        if (Bias) {
                            TA b = bias_is_acc_type ? static_cast<const TA*>(Bias)[oc] : ld(static_cast<const TS*>(Bias), oc);
                            accum = accum + b;
                        }
                        const int64_t yi = (n * c_out + oc) * o_sp + (o0 * o_d[1] + o1) * o_d[2] + o2;
                        if (out_is_acc_type) static_cast<TA*>(Y)[yi] = accum;
                        else store16(static_cast<TS*>(Y), yi, accum);
                    }
        }
    }
}

inline float gelu_erf(float x) { return 0.5f * x * (1.0f + std::erf(x * 0.70710678118654752440f)); }
inline double gelu_erf(double x) { return 0.5 * x * (1.0 + std::erf(x * 0.70710678118654752440)); }

template <typename T>
T act_t(int act, T x) {
    switch (act) {
        case 1: return gelu_erf(x);
        case 2: return x > T(0) ? x : T(0);
        case 3: return std::tanh(x);
        case 4: return T(1) / (T(1) + std::exp(-x));
        case 5: return std::exp(x);
        case 6: return std::erf(x);
        case 7: return std::sqrt(x);
        case 8: return std::fabs(x);
        default: return x;
    }
}

}  // namespace

extern "C" {

int oracle_num_threads() {
#if defined(_OPENMP)
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// Launchers such as torch.distributed.run export OMP_NUM_THREADS=1; the timed baseline asks for the cores it may use.
void oracle_set_num_threads(int n) {
#if defined(_OPENMP)
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

// alpha/beta as doubles; converted to the accumulate type inside.
int oracle_gemm(int prec, int layout, int transa, int transb, int64_t m, int64_t n, int64_t k, double alpha,
                const void* A, int64_t lda, const void* B, int64_t ldb, double beta, void* C, int64_t ldc) {
    switch (prec) {
        case 'd': gemm_t<'d'>(layout, transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc); return 0;
        case 's': gemm_t<'s'>(layout, transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc); return 0;
        case 'b': gemm_t<'b'>(layout, transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc); return 0;
        case 'h': gemm_t<'h'>(layout, transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc); return 0;
    }
    return 1;
}

// MatMulNode::expand (matmul_node.cpp:353-489): batch maps around GEMM(RowMajor, NN, alpha=1, beta=0).
int oracle_matmul(int prec, int64_t batch, int64_t m, int64_t n, int64_t k, const void* A, int64_t lda, int64_t sa,
                  const void* B, int64_t ldb, int64_t sb, void* Y, int64_t ldy, int64_t sy) {
    const int64_t es = prec == 'd' ? 8 : (prec == 's' ? 4 : 2);
    for (int64_t b = 0; b < batch; b++) {
        int rc = oracle_gemm(prec, 101, 111, 111, m, n, k, 1.0, static_cast<const char*>(A) + b * sa * es, lda,
                             static_cast<const char*>(B) + b * sb * es, ldb, 0.0, static_cast<char*>(Y) + b * sy * es, ldy);
        if (rc) return rc;
    }
    return 0;
}

int oracle_softmax(int prec, int rank, const int64_t* shape, int naxes, const int64_t* axes, const void* X, void* Y) {
    if (prec == 's') softmax_t<float>(rank, shape, naxes, axes, static_cast<const float*>(X), static_cast<float*>(Y));
    else if (prec == 'd') softmax_t<double>(rank, shape, naxes, axes, static_cast<const double*>(X), static_cast<double*>(Y));
    else return 1;
    return 0;
}

int oracle_reduce(int op, int prec, int rank, const int64_t* shape, int naxes, const int64_t* axes, const void* X, void* Y) {
    if (prec == 's') reduce_t<float>(op, rank, shape, naxes, axes, static_cast<const float*>(X), static_cast<float*>(Y));
    else if (prec == 'd') reduce_t<double>(op, rank, shape, naxes, axes, static_cast<const double*>(X), static_cast<double*>(Y));
    else return 1;
    return 0;
}

// prec_in: 's','d','b','h'; prec_out: 's' (fp32), 'd' or the 16-bit input type. Bias has the output type.
int oracle_conv(int prec_in, int prec_out, int sr, const int64_t* xs, const int64_t* ks, const int64_t* st,
                const int64_t* pads, const int64_t* dil, int64_t c_out, int64_t group, const void* X, const void* W,
                const void* Bias, void* Y) {
    if (sr < 1 || sr > 3) return 1;
    if (prec_in == 'd') {
        conv_t<double, double>(sr, xs, ks, st, pads, dil, c_out, group, static_cast<const double*>(X),
                               static_cast<const double*>(W), Bias, true, Y, true,
                               [](const double* p, int64_t i) { return p[i]; }, [](double*, int64_t, double) {});
    } else if (prec_in == 's') {
        conv_t<float, float>(sr, xs, ks, st, pads, dil, c_out, group, static_cast<const float*>(X),
                             static_cast<const float*>(W), Bias, true, Y, true,
                             [](const float* p, int64_t i) { return p[i]; }, [](float*, int64_t, float) {});
    } else if (prec_in == 'b') {
        conv_t<uint16_t, float>(sr, xs, ks, st, pads, dil, c_out, group, static_cast<const uint16_t*>(X),
                                static_cast<const uint16_t*>(W), Bias, prec_out == 's', Y, prec_out == 's',
                                [](const uint16_t* p, int64_t i) { return bf16_to_f32(p[i]); },
                                [](uint16_t* p, int64_t i, float v) { p[i] = f32_to_bf16(v); });
    } else if (prec_in == 'h') {
        conv_t<uint16_t, float>(sr, xs, ks, st, pads, dil, c_out, group, static_cast<const uint16_t*>(X),
                                static_cast<const uint16_t*>(W), Bias, prec_out == 's', Y, prec_out == 's',
                                [](const uint16_t* p, int64_t i) { return f16_to_f32(p[i]); },
                                [](uint16_t* p, int64_t i, float v) { p[i] = f32_to_f16(v); });
    } else {
        return 1;
    }
    return 0;
}

// Attention has no docc node. Composition of the restated primitives, per (b,h):
//   S = Q K^T (GEMM loop order, fp32 fma, k-sequential), S *= scale (Mul node),
//   causal: keys j > i + Skv - Sq are excluded from max, sum and PV,
//   P = softmax(S, axis -1) (max, sub, exp, left-to-right sum, div), O = P V (GEMM loop).
// 16-bit inputs are widened to fp32 on load and the result is rounded once on store.
int oracle_attention(int prec, int64_t Bn, int64_t H, int64_t Sq, int64_t Skv, int64_t D, float scale, int causal,
                     const void* Q, const int64_t* qs, const void* K, const int64_t* ks, const void* V, const int64_t* vs,
                     void* O, const int64_t* os) {
    auto ldf = [prec](const void* p, int64_t i) -> float {
        if (prec == 's') return static_cast<const float*>(p)[i];
        if (prec == 'b') return bf16_to_f32(static_cast<const uint16_t*>(p)[i]);
        return f16_to_f32(static_cast<const uint16_t*>(p)[i]);
    };
    auto stf = [prec](void* p, int64_t i, float v) {
        if (prec == 's') static_cast<float*>(p)[i] = v;
        else if (prec == 'b') static_cast<uint16_t*>(p)[i] = f32_to_bf16(v);
        else static_cast<uint16_t*>(p)[i] = f32_to_f16(v);
    };
    if (prec != 's' && prec != 'b' && prec != 'h') return 1;
    int64_t dq[3] = {H * Sq * D, Sq * D, D}, dk[3] = {H * Skv * D, Skv * D, D};
    if (!qs) qs = dq;
    if (!os) os = dq;
    if (!ks) ks = dk;
    if (!vs) vs = dk;
#pragma omp parallel for schedule(static) collapse(2)
    for (int64_t b = 0; b < Bn; b++)
        for (int64_t h = 0; h < H; h++) {
            std::vector<float> s(static_cast<size_t>(Skv)), e(static_cast<size_t>(Skv));
            for (int64_t i = 0; i < Sq; i++) {
                const int64_t lim = causal ? std::min<int64_t>(Skv, i + Skv - Sq + 1) : Skv;
                const int64_t qo = b * qs[0] + h * qs[1] + i * qs[2];
                float mx = -std::numeric_limits<float>::infinity();
                for (int64_t j = 0; j < lim; j++) {
                    const int64_t ko = b * ks[0] + h * ks[1] + j * ks[2];
                    float sum = 0.f;
                    for (int64_t d = 0; d < D; d++) sum = std::fmaf(ldf(Q, qo + d), ldf(K, ko + d), sum);
                    s[j] = sum * scale;
                    mx = std::fmax(s[j], mx);
                }
                float den = 0.f;
                for (int64_t j = 0; j < lim; j++) {
                    e[j] = std::exp(s[j] - mx);
                    den = e[j] + den;
                }
                const int64_t oo = b * os[0] + h * os[1] + i * os[2];
                for (int64_t d = 0; d < D; d++) {
                    float acc = 0.f;
                    for (int64_t j = 0; j < lim; j++) {
                        const int64_t vo = b * vs[0] + h * vs[1] + j * vs[2];
                        acc = std::fmaf(e[j] / den, ldf(V, vo + d), acc);
                    }
                    stf(O, oo + d, lim > 0 ? acc : 0.f);
                }
            }
        }
    return 0;
}

// LayerNorm has no docc node: (x - mean) / sqrt(var + eps) * gamma + beta, population variance,
// built from the Sum/Mean primitives (left-to-right sums in fp32; 16-bit inputs widened on load).
int oracle_layernorm(int prec, int64_t rows, int64_t cols, const void* X, const float* gamma, const float* beta,
                     double eps, void* Y) {
    if (prec != 's' && prec != 'b' && prec != 'd') return 1;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; r++) {
        if (prec == 'd') {
            const double* x = static_cast<const double*>(X) + r * cols;
            double* y = static_cast<double*>(Y) + r * cols;
            double s = 0;
            for (int64_t c = 0; c < cols; c++) s = x[c] + s;
            double mean = s / double(cols), v = 0;
            for (int64_t c = 0; c < cols; c++) v = (x[c] - mean) * (x[c] - mean) + v;
            double rstd = 1.0 / std::sqrt(v / double(cols) + eps);
            for (int64_t c = 0; c < cols; c++)
                y[c] = (x[c] - mean) * rstd * (gamma ? double(gamma[c]) : 1.0) + (beta ? double(beta[c]) : 0.0);
            continue;
        }
        auto ld = [&](int64_t c) -> float {
            return prec == 's' ? static_cast<const float*>(X)[r * cols + c]
                               : bf16_to_f32(static_cast<const uint16_t*>(X)[r * cols + c]);
        };
        float s = 0.f;
        for (int64_t c = 0; c < cols; c++) s = ld(c) + s;
        float mean = s / float(cols), v = 0.f;
        for (int64_t c = 0; c < cols; c++) v = (ld(c) - mean) * (ld(c) - mean) + v;
        float rstd = 1.0f / std::sqrt(v / float(cols) + float(eps));
        for (int64_t c = 0; c < cols; c++) {
            float o = (ld(c) - mean) * rstd * (gamma ? gamma[c] : 1.f) + (beta ? beta[c] : 0.f);
            if (prec == 's') static_cast<float*>(Y)[r * cols + c] = o;
            else static_cast<uint16_t*>(Y)[r * cols + c] = f32_to_bf16(o);
        }
    }
    return 0;
}

// Y = act(scale*X + bias[col]) + residual: chain of element-wise tensor nodes
// (elementwise_node.cpp:86-339), each one libm call per element on the CPU targets.
int oracle_bias_act(int prec, int64_t rows, int64_t cols, const void* X, float scale, const float* bias, int act,
                    const void* residual, void* Y) {
    if (prec != 's' && prec != 'b' && prec != 'd') return 1;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; r++)
        for (int64_t c = 0; c < cols; c++) {
            const int64_t i = r * cols + c;
            if (prec == 'd') {
                double v = static_cast<const double*>(X)[i] * double(scale) + (bias ? double(bias[c]) : 0.0);
                v = act_t<double>(act, v);
                if (residual) v += static_cast<const double*>(residual)[i];
                static_cast<double*>(Y)[i] = v;
            } else {
                float x = prec == 's' ? static_cast<const float*>(X)[i] : bf16_to_f32(static_cast<const uint16_t*>(X)[i]);
                float v = act_t<float>(act, x * scale + (bias ? bias[c] : 0.f));
                if (residual)
                    v += prec == 's' ? static_cast<const float*>(residual)[i]
                                     : bf16_to_f32(static_cast<const uint16_t*>(residual)[i]);
                if (prec == 's') static_cast<float*>(Y)[i] = v;
                else static_cast<uint16_t*>(Y)[i] = f32_to_bf16(v);
            }
        }
    return 0;
}

int oracle_binary(int op, int prec, int64_t n, const void* A, const void* B, void* Y) {
    if (prec != 's' && prec != 'd') return 1;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; i++) {
        if (prec == 's') {
            float a = static_cast<const float*>(A)[i], b = static_cast<const float*>(B)[i], y;
            switch (op) { case 0: y = a + b; break; case 1: y = a - b; break; case 2: y = a * b; break;
                          case 3: y = a / b; break; case 4: y = std::fmax(a, b); break; default: y = std::fmin(a, b); }
            static_cast<float*>(Y)[i] = y;
        } else {
            double a = static_cast<const double*>(A)[i], b = static_cast<const double*>(B)[i], y;
            switch (op) { case 0: y = a + b; break; case 1: y = a - b; break; case 2: y = a * b; break;
                          case 3: y = a / b; break; case 4: y = std::fmax(a, b); break; default: y = std::fmin(a, b); }
            static_cast<double*>(Y)[i] = y;
        }
    }
    return 0;
}

void oracle_f32_to_bf16(const float* src, uint16_t* dst, int64_t n) {
    for (int64_t i = 0; i < n; i++) dst[i] = f32_to_bf16(src[i]);
}
void oracle_bf16_to_f32(const uint16_t* src, float* dst, int64_t n) {
    for (int64_t i = 0; i < n; i++) dst[i] = bf16_to_f32(src[i]);
}

}  // extern "C"
