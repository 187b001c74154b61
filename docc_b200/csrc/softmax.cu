// Softmax and the Sum/Max/Min/Mean/Std reductions as single fused bandwidth kernels.
//
// docc expands SoftmaxNode into seven loop nests over six temporaries
// (softmax_node.cpp:92-252: Max, Broadcast, Sub, Exp, Sum, Broadcast, Div), i.e. 7 reads and
// 5 writes of the tensor. Here a row is read once into registers, reduced with warp shuffles,
// and written once: 2 * rows * cols * sizeof(T) bytes of HBM traffic.
#include <cfloat>

#include <cstdlib>

#include "common.cuh"
#include "device_math.cuh"
#include "ptx.cuh"

namespace docc_b200 {
namespace {

constexpr int kMaxRank = 8;

// ---- storage <-> compute conversion ----------------------------------------------------
template <typename T> struct Cvt;
template <> struct Cvt<float> { using acc = float;
    __device__ static float ld(float v) { return v; } __device__ static float st(float v) { return v; } };
template <> struct Cvt<double> { using acc = double;
    __device__ static double ld(double v) { return v; } __device__ static double st(double v) { return v; } };
template <> struct Cvt<__half> { using acc = float;
    __device__ static float ld(__half v) { return __half2float(v); } __device__ static __half st(float v) { return __float2half_rn(v); } };
template <> struct Cvt<__nv_bfloat16> { using acc = float;
    __device__ static float ld(__nv_bfloat16 v) { return __bfloat162float(v); }
    __device__ static __nv_bfloat16 st(float v) { return __float2bfloat16_rn(v); } };

__device__ __forceinline__ float fast_exp(float d) {
    // exp(d) = 2^(d*log2(e)) on the SFU; d <= 0 here, relative error ~ |d| * 2^-23
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(d * 1.4426950408889634f));
    return r;
}
__device__ __forceinline__ double fast_exp(double d) { return exp(d); }

template <typename A> __device__ __forceinline__ A neg_inf();
template <> __device__ __forceinline__ float neg_inf<float>() { return -INFINITY; }
template <> __device__ __forceinline__ double neg_inf<double>() { return -INFINITY; }

template <typename A> __device__ __forceinline__ A warp_max(A v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmax(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
template <typename A> __device__ __forceinline__ A warp_sum(A v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---- row kernel ------------------------------------------------------------------------------
// TPR threads cooperate on one row; each holds VPT packs of VEC elements (pack index
// p = i*TPR + t, so a warp reads 32 consecutive packs = 512 contiguous bytes). A block of
// BLOCK threads works on BLOCK/TPR rows at once and strides over row groups.
template <typename T, int VEC, int VPT, int TPR, int BLOCK>
__global__ void __launch_bounds__(BLOCK) softmax_rows_kernel(const T* __restrict__ X, T* __restrict__ Y, int64_t rows,
                                                             int64_t cols) {
    using A = typename Cvt<T>::acc;
    using P = Pack<T, VEC>;
    constexpr int ROWS_PER_BLOCK = BLOCK / TPR;
    constexpr int WARPS_PER_ROW = TPR / 32;
    __shared__ A red[2][ROWS_PER_BLOCK][WARPS_PER_ROW > 0 ? WARPS_PER_ROW : 1];

    const int t = threadIdx.x % TPR;
    const int r_in_block = threadIdx.x / TPR;
    const int warp_in_row = t / 32;
    const int64_t packs_per_row = cols / VEC;  // cols % VEC == 0 is guaranteed by the dispatcher
    const int64_t n_groups = (rows + ROWS_PER_BLOCK - 1) / ROWS_PER_BLOCK;
    // launched with programmatic stream serialization: blocks become resident while the launch before this one drains,
    // and touch no global memory before it has completed
    ptx::griddep_wait();
    ptx::griddep_launch_dependents();

    for (int64_t g = blockIdx.x; g < n_groups; g += gridDim.x) {
        const int64_t row = g * ROWS_PER_BLOCK + r_in_block;
        const bool row_ok = row < rows;
        const P* xrow = reinterpret_cast<const P*>(X + row * cols);
        P* yrow = reinterpret_cast<P*>(Y + row * cols);

        A vals[VPT][VEC];
        A mx = neg_inf<A>();
#pragma unroll
        for (int i = 0; i < VPT; i++) {
            const int64_t p = int64_t(i) * TPR + t;
            if (row_ok && p < packs_per_row) {
                const P pk = load_pack(xrow + p);
#pragma unroll
                for (int e = 0; e < VEC; e++) {
                    vals[i][e] = Cvt<T>::ld(pk.v[e]);
                    mx = fmax(mx, vals[i][e]);
                }
            } else {
#pragma unroll
                for (int e = 0; e < VEC; e++) vals[i][e] = neg_inf<A>();
            }
        }
        mx = warp_max(mx);
        if (WARPS_PER_ROW > 1) {
            if ((t & 31) == 0) red[0][r_in_block][warp_in_row] = mx;
            __syncthreads();
            mx = red[0][r_in_block][0];
#pragma unroll
            for (int w = 1; w < WARPS_PER_ROW; w++) mx = fmax(mx, red[0][r_in_block][w]);
        }
        // a row of -inf (or an empty row) would give inf - inf: keep exp argument finite
        const A mref = (mx == neg_inf<A>()) ? A(0) : mx;
        A sum = A(0);
#pragma unroll
        for (int i = 0; i < VPT; i++)
#pragma unroll
            for (int e = 0; e < VEC; e++) {
                vals[i][e] = fast_exp(vals[i][e] - mref);
                sum += vals[i][e];
            }
        sum = warp_sum(sum);
        if (WARPS_PER_ROW > 1) {
            if ((t & 31) == 0) red[1][r_in_block][warp_in_row] = sum;
            __syncthreads();
            sum = red[1][r_in_block][0];
#pragma unroll
            for (int w = 1; w < WARPS_PER_ROW; w++) sum += red[1][r_in_block][w];
        }
        const A inv = A(1) / sum;
#pragma unroll
        for (int i = 0; i < VPT; i++) {
            const int64_t p = int64_t(i) * TPR + t;
            if (row_ok && p < packs_per_row) {
                P pk;
#pragma unroll
                for (int e = 0; e < VEC; e++) pk.v[e] = Cvt<T>::st(vals[i][e] * inv);
                store_pack(yrow + p, pk);
            }
        }
        if (WARPS_PER_ROW > 1) __syncthreads();  // red[] is reused by the next row group
    }
}

// ---- generic kernel --------------------------------------------------------------------------
// Any set of reduced axes of a C-order tensor. One block per kept index; threads stride over
// the reduced index space, three passes (max, sum, write). Used for non-trailing axes and for
// rows too long for the register kernel.
struct Geom {
    int n_kept, n_red;
    int64_t kept_dims[kMaxRank], kept_strides[kMaxRank];
    int64_t red_dims[kMaxRank], red_strides[kMaxRank];
    int64_t kept_total, red_total;
};

__device__ __forceinline__ int64_t decompose(int64_t lin, const int64_t* dims, const int64_t* strides, int n) {
    int64_t off = 0;
    for (int d = n - 1; d >= 0; d--) {
        const int64_t q = lin / dims[d];
        off += (lin - q * dims[d]) * strides[d];
        lin = q;
    }
    return off;
}

template <typename A, bool IS_MAX> __device__ A block_reduce(A v, A* smem) {
    v = IS_MAX ? warp_max(v) : warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    A r = smem[0];
    for (int w = 1; w < nwarps; w++) r = IS_MAX ? fmax(r, smem[w]) : r + smem[w];
    return r;
}

template <typename T>
__global__ void __launch_bounds__(256) softmax_generic_kernel(const T* __restrict__ X, T* __restrict__ Y, Geom g) {
    using A = typename Cvt<T>::acc;
    __shared__ A smem[8];
    for (int64_t o = blockIdx.x; o < g.kept_total; o += gridDim.x) {
        const int64_t base = decompose(o, g.kept_dims, g.kept_strides, g.n_kept);
        A mx = neg_inf<A>();
        for (int64_t r = threadIdx.x; r < g.red_total; r += blockDim.x)
            mx = fmax(mx, Cvt<T>::ld(X[base + decompose(r, g.red_dims, g.red_strides, g.n_red)]));
        mx = block_reduce<A, true>(mx, smem);
        const A mref = (mx == neg_inf<A>()) ? A(0) : mx;
        A sum = A(0);
        for (int64_t r = threadIdx.x; r < g.red_total; r += blockDim.x)
            sum += fast_exp(Cvt<T>::ld(X[base + decompose(r, g.red_dims, g.red_strides, g.n_red)]) - mref);
        sum = block_reduce<A, false>(sum, smem);
        const A inv = A(1) / sum;
        for (int64_t r = threadIdx.x; r < g.red_total; r += blockDim.x) {
            const int64_t off = base + decompose(r, g.red_dims, g.red_strides, g.n_red);
            Y[off] = Cvt<T>::st(fast_exp(Cvt<T>::ld(X[off]) - mref) * inv);
        }
    }
}

// Thread-per-kept-index variant for many short reductions over a strided axis (e.g. axis 0):
// consecutive threads take consecutive kept indices, so accesses stay coalesced when the
// innermost tensor dimension is kept.
template <typename T>
__global__ void __launch_bounds__(256) softmax_strided_kernel(const T* __restrict__ X, T* __restrict__ Y, Geom g) {
    using A = typename Cvt<T>::acc;
    for (int64_t o = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; o < g.kept_total; o += int64_t(gridDim.x) * blockDim.x) {
        const int64_t base = decompose(o, g.kept_dims, g.kept_strides, g.n_kept);
        A mx = neg_inf<A>();
        for (int64_t r = 0; r < g.red_total; r++)
            mx = fmax(mx, Cvt<T>::ld(X[base + decompose(r, g.red_dims, g.red_strides, g.n_red)]));
        const A mref = (mx == neg_inf<A>()) ? A(0) : mx;
        A sum = A(0);
        for (int64_t r = 0; r < g.red_total; r++)
            sum += fast_exp(Cvt<T>::ld(X[base + decompose(r, g.red_dims, g.red_strides, g.n_red)]) - mref);
        const A inv = A(1) / sum;
        for (int64_t r = 0; r < g.red_total; r++) {
            const int64_t off = base + decompose(r, g.red_dims, g.red_strides, g.n_red);
            Y[off] = Cvt<T>::st(fast_exp(Cvt<T>::ld(X[off]) - mref) * inv);
        }
    }
}

// ---- reductions ---------------------------------------------------------------------------------
// op: DOCC_B200_RED_*. One block per kept index (block_mode) or one thread per kept index.
template <typename T, bool BLOCK_MODE>
__global__ void __launch_bounds__(256) reduce_kernel(int op, const T* __restrict__ X, T* __restrict__ Y, Geom g) {
    using A = typename Cvt<T>::acc;
    __shared__ A smem[8];
    const int64_t start = BLOCK_MODE ? blockIdx.x : blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
    const int64_t step = BLOCK_MODE ? gridDim.x : int64_t(gridDim.x) * blockDim.x;
    const int64_t rstart = BLOCK_MODE ? threadIdx.x : 0;
    const int64_t rstep = BLOCK_MODE ? blockDim.x : 1;
    for (int64_t o = start; o < g.kept_total; o += step) {
        const int64_t base = decompose(o, g.kept_dims, g.kept_strides, g.n_kept);
        A acc = (op == DOCC_B200_RED_MAX) ? neg_inf<A>() : (op == DOCC_B200_RED_MIN ? -neg_inf<A>() : A(0));
        A acc2 = A(0);
        for (int64_t r = rstart; r < g.red_total; r += rstep) {
            const A v = Cvt<T>::ld(X[base + decompose(r, g.red_dims, g.red_strides, g.n_red)]);
            if (op == DOCC_B200_RED_MAX) acc = fmax(acc, v);
            else if (op == DOCC_B200_RED_MIN) acc = fmin(acc, v);
            else {
                acc += v;
                if (op == DOCC_B200_RED_STD) acc2 += v * v;
            }
        }
        if (BLOCK_MODE) {
            if (op == DOCC_B200_RED_MAX) acc = block_reduce<A, true>(acc, smem);
            else if (op == DOCC_B200_RED_MIN) acc = -block_reduce<A, true>(-acc, smem);
            else {
                acc = block_reduce<A, false>(acc, smem);
                if (op == DOCC_B200_RED_STD) acc2 = block_reduce<A, false>(acc2, smem);
            }
        }
        if (!BLOCK_MODE || threadIdx.x == 0) {
            A out = acc;
            if (op == DOCC_B200_RED_MEAN) out = acc / A(g.red_total);
            if (op == DOCC_B200_RED_STD) {
                const A mean = acc / A(g.red_total);
                out = sqrt(fmax(acc2 / A(g.red_total) - mean * mean, A(0)));
            }
            Y[o] = Cvt<T>::st(out);
        }
    }
}

// ---- host side -------------------------------------------------------------------------------------
int build_geom(int rank, const int64_t* shape, int naxes, const int64_t* axes, Geom* g, bool* trailing) {
    DOCC_REQUIRE(rank >= 0 && rank <= kMaxRank, "rank %d outside [0,%d]", rank, kMaxRank);
    DOCC_REQUIRE(naxes >= 0 && naxes <= rank, "naxes %d outside [0,%d]", naxes, rank);
    DOCC_REQUIRE(rank == 0 || shape != nullptr, "shape is NULL");
    DOCC_REQUIRE(naxes == 0 || axes != nullptr, "axes is NULL");
    bool is_red[kMaxRank] = {false};
    for (int a = 0; a < naxes; a++) {
        int64_t ax = axes[a] < 0 ? axes[a] + rank : axes[a];
        // same bounds rule as SoftmaxNode::expand (softmax_node.cpp:60-70)
        DOCC_REQUIRE(ax >= 0 && ax < rank, "Axis value out of bounds. Axis: %lld Shape size: %d", (long long)axes[a], rank);
        DOCC_REQUIRE(!is_red[ax], "axis %lld listed twice", (long long)ax);
        is_red[ax] = true;
    }
    int64_t strides[kMaxRank];
    int64_t s = 1;
    for (int d = rank - 1; d >= 0; d--) {
        DOCC_REQUIRE(shape[d] >= 0, "negative extent in shape[%d]", d);
        strides[d] = s;
        s *= shape[d];
    }
    g->n_kept = g->n_red = 0;
    g->kept_total = g->red_total = 1;
    for (int d = 0; d < rank; d++) {
        if (is_red[d]) {
            g->red_dims[g->n_red] = shape[d];
            g->red_strides[g->n_red++] = strides[d];
            g->red_total *= shape[d];
        } else {
            g->kept_dims[g->n_kept] = shape[d];
            g->kept_strides[g->n_kept++] = strides[d];
            g->kept_total *= shape[d];
        }
    }
    // reduced axes are exactly the trailing dims -> [kept_total x red_total] row problem
    bool tr = true;
    for (int d = 0; d < rank; d++)
        if (is_red[d] != (d >= rank - naxes)) tr = false;
    *trailing = tr;
    return DOCC_B200_OK;
}

template <typename T, int VEC, int VPT, int TPR>
int launch_rows(Ctx* ctx, const T* X, T* Y, int64_t rows, int64_t cols) {
    constexpr int BLOCK = TPR > 256 ? TPR : 256;
    constexpr int RPB = BLOCK / TPR;
    const int64_t groups = ceil_div(rows, RPB);
    // One row group per block: the hardware block scheduler then balances the SMs dynamically. A grid capped at the
    // resident block count (grid-stride inside the kernel) left part of the SMs idle during the last, partly filled
    // round of groups (5740 -> 5920 GB/s on fp32 [8192,4096]).
    const int64_t max_blocks = 0x7fffffff;
    const int grid = int(groups < max_blocks ? groups : max_blocks);
    DOCC_CUDA_TRY(launch_pdl(softmax_rows_kernel<T, VEC, VPT, TPR, BLOCK>, dim3(unsigned(grid)), dim3(BLOCK), 0, ctx->stream, X, Y, rows, cols));
    return after_launch(ctx, "softmax_rows_kernel");
}

template <typename T, int VEC>
int dispatch_rows(Ctx* ctx, const T* X, T* Y, int64_t rows, int64_t cols, bool* handled) {
    const int64_t packs = cols / VEC;
    *handled = true;
    if (packs <= 32) return launch_rows<T, VEC, 1, 32>(ctx, X, Y, rows, cols);
    if (packs <= 64) return launch_rows<T, VEC, 2, 32>(ctx, X, Y, rows, cols);
    if (packs <= 128) return launch_rows<T, VEC, 4, 32>(ctx, X, Y, rows, cols);
    if (packs <= 256) return launch_rows<T, VEC, 8, 32>(ctx, X, Y, rows, cols);
    if (packs <= 512) return launch_rows<T, VEC, 4, 128>(ctx, X, Y, rows, cols);
    if (packs <= 1024) return launch_rows<T, VEC, 4, 256>(ctx, X, Y, rows, cols);  // 16 values per thread instead of 32: more resident blocks
    if (packs <= 2048) return launch_rows<T, VEC, 8, 256>(ctx, X, Y, rows, cols);
    if (packs <= 8192) return launch_rows<T, VEC, 8, 1024>(ctx, X, Y, rows, cols);
    *handled = false;
    return DOCC_B200_OK;
}

template <typename T>
int softmax_device(Ctx* ctx, int rank, const int64_t* shape, int naxes, const int64_t* axes, const T* X, T* Y) {
    Geom g;
    bool trailing;
    DOCC_TRY(build_geom(rank, shape, naxes, axes, &g, &trailing));
    if (g.kept_total == 0 || g.red_total == 0) return DOCC_B200_OK;  // empty tensor: nothing to write
    if (trailing) {
        const int64_t rows = g.kept_total, cols = g.red_total;
        constexpr int VEC = 16 / sizeof(T);
        const bool aligned = (reinterpret_cast<uintptr_t>(X) % 16 == 0) && (reinterpret_cast<uintptr_t>(Y) % 16 == 0) &&
                             (cols % VEC == 0);
        bool handled = false;
        if (aligned) {
            DOCC_TRY((dispatch_rows<T, VEC>(ctx, X, Y, rows, cols, &handled)));
        } else if (cols <= 1024) {
            DOCC_TRY((dispatch_rows<T, 1>(ctx, X, Y, rows, cols, &handled)));
        }
        if (handled) return DOCC_B200_OK;
    }
    const bool block_mode = g.red_total >= 512 || g.kept_total < int64_t(ctx->sm_count) * 64;
    if (block_mode) {
        const int64_t cap = int64_t(ctx->sm_count) * 8;
        softmax_generic_kernel<T><<<int(g.kept_total < cap ? g.kept_total : cap), 256, 0, ctx->stream>>>(X, Y, g);
        return after_launch(ctx, "softmax_generic_kernel");
    }
    const int64_t blocks = ceil_div(g.kept_total, 256);
    const int64_t cap = int64_t(ctx->sm_count) * 8;
    softmax_strided_kernel<T><<<int(blocks < cap ? blocks : cap), 256, 0, ctx->stream>>>(X, Y, g);
    return after_launch(ctx, "softmax_strided_kernel");
}

template <typename T>
int reduce_device(Ctx* ctx, int op, int rank, const int64_t* shape, int naxes, const int64_t* axes, const T* X, T* Y) {
    Geom g;
    bool trailing;
    DOCC_TRY(build_geom(rank, shape, naxes, axes, &g, &trailing));
    if (g.kept_total == 0) return DOCC_B200_OK;
    const int64_t cap = int64_t(ctx->sm_count) * 8;
    const bool block_mode = g.red_total >= 512 || g.kept_total < int64_t(ctx->sm_count) * 64;
    if (block_mode) {
        reduce_kernel<T, true><<<int(g.kept_total < cap ? g.kept_total : cap), 256, 0, ctx->stream>>>(op, X, Y, g);
    } else {
        const int64_t blocks = ceil_div(g.kept_total, 256);
        reduce_kernel<T, false><<<int(blocks < cap ? blocks : cap), 256, 0, ctx->stream>>>(op, X, Y, g);
    }
    return after_launch(ctx, "reduce_kernel");
}

int64_t numel(int rank, const int64_t* shape) {
    int64_t n = 1;
    for (int d = 0; d < rank; d++) n *= shape[d];
    return n;
}

// Host-pointer softmax over trailing axes: rows are cut into chunks that flow through
// H2D -> kernel -> D2H on two streams so that both PCIe directions and the SMs overlap.
template <typename T>
int softmax_host_pipelined(Ctx* ctx, int64_t rows, int64_t cols, const T* hX, T* hY) {
    const size_t row_bytes = size_t(cols) * sizeof(T);
    int64_t chunk_rows = (size_t(16) << 20) / (row_bytes ? row_bytes : 1);
    if (chunk_rows < 1) chunk_rows = 1;
    if (chunk_rows > rows) chunk_rows = rows;
    const int64_t n_chunks = ceil_div(rows, chunk_rows);
    const int depth = n_chunks < 3 ? int(n_chunks) : 3;
    TempBuffers tmp;
    T* dX[3];
    T* dY[3];
    for (int i = 0; i < depth; i++) {
        DOCC_TRY(tmp.alloc(reinterpret_cast<void**>(&dX[i]), size_t(chunk_rows) * row_bytes));
        DOCC_TRY(tmp.alloc(reinterpret_cast<void**>(&dY[i]), size_t(chunk_rows) * row_bytes));
    }
    cudaStream_t user = ctx->stream;
    cudaStream_t lanes[3] = {ctx->copy_streams[0], ctx->copy_streams[1], ctx->own_stream};
    int status = DOCC_B200_OK;
    for (int64_t c = 0; c < n_chunks && status == DOCC_B200_OK; c++) {
        const int slot = int(c % depth);
        cudaStream_t s = lanes[slot];
        const int64_t r0 = c * chunk_rows;
        const int64_t nr = (rows - r0) < chunk_rows ? (rows - r0) : chunk_rows;
        // stream order on `s` protects the reuse of dX[slot] / dY[slot]
        cudaError_t e = cudaMemcpyAsync(dX[slot], hX + r0 * cols, size_t(nr) * row_bytes, cudaMemcpyHostToDevice, s);
        if (e != cudaSuccess) { status = set_error(DOCC_B200_ERR_CUDA, "H2D: %s", cudaGetErrorString(e)); break; }
        ctx->stream = s;
        const int64_t shp[2] = {nr, cols};
        const int64_t ax[1] = {1};
        status = softmax_device<T>(ctx, 2, shp, 1, ax, dX[slot], dY[slot]);
        ctx->stream = user;
        if (status != DOCC_B200_OK) break;
        e = cudaMemcpyAsync(hY + r0 * cols, dY[slot], size_t(nr) * row_bytes, cudaMemcpyDeviceToHost, s);
        if (e != cudaSuccess) { status = set_error(DOCC_B200_ERR_CUDA, "D2H: %s", cudaGetErrorString(e)); break; }
    }
    for (int i = 0; i < 3; i++) {
        cudaError_t e = cudaStreamSynchronize(lanes[i]);
        if (e != cudaSuccess && status == DOCC_B200_OK) status = set_error(DOCC_B200_ERR_CUDA, "sync: %s", cudaGetErrorString(e));
    }
    return status;
}

template <typename T>
int softmax_entry(Ctx* ctx, int rank, const int64_t* shape, int naxes, const int64_t* axes, const void* X, void* Y, int flags) {
    if (!(flags & DOCC_B200_FLAG_HOST_PTRS))
        return softmax_device<T>(ctx, rank, shape, naxes, axes, static_cast<const T*>(X), static_cast<T*>(Y));
    Geom g;
    bool trailing;
    DOCC_TRY(build_geom(rank, shape, naxes, axes, &g, &trailing));
    const int64_t n = numel(rank, shape);
    if (n == 0) return DOCC_B200_OK;
    if (trailing && g.red_total * int64_t(sizeof(T)) <= (int64_t(8) << 20))
        return softmax_host_pipelined<T>(ctx, g.kept_total, g.red_total, static_cast<const T*>(X), static_cast<T*>(Y));
    TempBuffers tmp;
    void *dX, *dY;
    DOCC_TRY(tmp.alloc(&dX, size_t(n) * sizeof(T)));
    DOCC_TRY(tmp.alloc(&dY, size_t(n) * sizeof(T)));
    DOCC_CUDA_TRY(cudaMemcpyAsync(dX, X, size_t(n) * sizeof(T), cudaMemcpyHostToDevice, ctx->stream));
    DOCC_TRY(softmax_device<T>(ctx, rank, shape, naxes, axes, static_cast<const T*>(dX), static_cast<T*>(dY)));
    DOCC_CUDA_TRY(cudaMemcpyAsync(Y, dY, size_t(n) * sizeof(T), cudaMemcpyDeviceToHost, ctx->stream));
    DOCC_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    return DOCC_B200_OK;
}

template <typename T>
int reduce_entry(Ctx* ctx, int op, int rank, const int64_t* shape, int naxes, const int64_t* axes, const void* X, void* Y,
                 int flags) {
    if (!(flags & DOCC_B200_FLAG_HOST_PTRS))
        return reduce_device<T>(ctx, op, rank, shape, naxes, axes, static_cast<const T*>(X), static_cast<T*>(Y));
    Geom g;
    bool trailing;
    DOCC_TRY(build_geom(rank, shape, naxes, axes, &g, &trailing));
    const int64_t n = numel(rank, shape);
    TempBuffers tmp;
    void *dX, *dY;
    DOCC_TRY(tmp.alloc(&dX, size_t(n) * sizeof(T)));
    DOCC_TRY(tmp.alloc(&dY, size_t(g.kept_total) * sizeof(T)));
    DOCC_CUDA_TRY(cudaMemcpyAsync(dX, X, size_t(n) * sizeof(T), cudaMemcpyHostToDevice, ctx->stream));
    DOCC_TRY(reduce_device<T>(ctx, op, rank, shape, naxes, axes, static_cast<const T*>(dX), static_cast<T*>(dY)));
    DOCC_CUDA_TRY(cudaMemcpyAsync(Y, dY, size_t(g.kept_total) * sizeof(T), cudaMemcpyDeviceToHost, ctx->stream));
    DOCC_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    return DOCC_B200_OK;
}

}  // namespace
}  // namespace docc_b200

using namespace docc_b200;

extern "C" int docc_b200_softmax(int prec, int rank, const int64_t* shape, int naxes, const int64_t* axes, const void* X,
                                 void* Y, int flags) {
    Ctx* ctx;
    DOCC_TRY(get_ctx(&ctx));
    DOCC_REQUIRE(rank >= 0 && rank <= kMaxRank, "softmax: rank %d outside [0,%d]", rank, kMaxRank);
    const int64_t n = rank > 0 && shape ? numel(rank, shape) : (rank == 0 ? 1 : 0);
    DOCC_REQUIRE(n == 0 || (X && Y), "softmax: NULL data pointer");
    switch (prec) {
        case DOCC_B200_PREC_S: return softmax_entry<float>(ctx, rank, shape, naxes, axes, X, Y, flags);
        case DOCC_B200_PREC_D: return softmax_entry<double>(ctx, rank, shape, naxes, axes, X, Y, flags);
        case DOCC_B200_PREC_H: return softmax_entry<__half>(ctx, rank, shape, naxes, axes, X, Y, flags);
        case DOCC_B200_PREC_B: return softmax_entry<__nv_bfloat16>(ctx, rank, shape, naxes, axes, X, Y, flags);
    }
    return set_error(DOCC_B200_ERR_INVALID_ARG, "softmax: unknown precision code %d", prec);
}

extern "C" int docc_b200_reduce(int op, int prec, int rank, const int64_t* shape, int naxes, const int64_t* axes,
                                const void* X, void* Y, int flags) {
    Ctx* ctx;
    DOCC_TRY(get_ctx(&ctx));
    DOCC_REQUIRE(op >= DOCC_B200_RED_SUM && op <= DOCC_B200_RED_STD, "reduce: unknown op %d", op);
    DOCC_REQUIRE(X && Y, "reduce: NULL data pointer");
    switch (prec) {
        case DOCC_B200_PREC_S: return reduce_entry<float>(ctx, op, rank, shape, naxes, axes, X, Y, flags);
        case DOCC_B200_PREC_D: return reduce_entry<double>(ctx, op, rank, shape, naxes, axes, X, Y, flags);
    }
    return set_error(DOCC_B200_ERR_INVALID_ARG, "reduce: precision code %d not supported (use 's' or 'd')", prec);
}
