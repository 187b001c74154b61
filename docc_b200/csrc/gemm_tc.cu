// tcgen05 contraction engine: D = epilogue(sum_p A_p * B_p) with 16-bit operands and fp32
// accumulation in tensor memory.
//
// Replaces the cublas{S,D}gemm call sequence of docc's CUDA target
// (opt/src/targets/cuda/blas/gemm.cpp:131-185) for everything except fp64.
//
// Structure (one persistent CTA per SM, 320 threads; two kernels share it):
//   warp 0      TMA producer: cp.async.bulk.tensor loads of A and B tiles (64 deep) into a ring of
//               128-byte-swizzled shared-memory stages, completion on mbarriers.
//   warp 1      UMMA issuer: one lane issues tcgen05.mma (K=16) four times per stage and tile half;
//               tcgen05.commit releases the stage and, after the last k-block, publishes the
//               accumulator. It also owns the tensor-memory allocation.
//   warps 2-9   epilogue: tcgen05.ld the fp32 accumulator (each warp its own 32-lane quadrant),
//               apply alpha/beta/bias/activation/residual, stage and TMA-store.
// tc_gemm_kernel (cta_group::1): tiles are 256xBN (two M=128 UMMAs per k-step sharing the B tile; both
// 256-column TMEM regions belong to one tile and each epilogue warp group drains one of them) or
// 128xBN (the two TMEM regions are alternating accumulator buffers, so the epilogue of tile i
// overlaps the main loop of tile i+1); operands may be K-major or MN-major.
// tc_gemm_pair_kernel (cta_group::2, K-major operands, large problems): a cluster of two CTAs owns a
// 256x256 or 256x512 tile; each CTA loads its half of the rows of A and of B.
// fp32 operands are handled as split bf16 (hi + lo): the kernels run up to three passes (hi*hi, hi*lo,
// lo*hi) into the same accumulator, which keeps fp32-level accuracy (~2^-16 relative per product)
// at a third of the bf16 rate. Every wait is bounded. Producer and issuer are single lanes: their
// loops carry the ring position and the descriptors incrementally, because every scalar instruction
// between two UMMAs is issue latency the tensor pipe has to absorb.
#include <cstdio>
#include <cstdlib>
#include <mutex>

#include "device_math.cuh"
#include "gemm_tc.h"
#include "ptx.cuh"

namespace docc_b200 {
namespace {

using namespace ptx;

constexpr int kBK = 64;  // 64 bf16 = one 128-byte swizzle row
constexpr int kThreads = 320;  // TMA warp, UMMA warp, eight epilogue warps
constexpr int kMaxStages = 8;
constexpr uint32_t kTmemCols = 512;
constexpr int kSmemBudget = 227 * 1024;
constexpr uint32_t kStagingBytes = 8 * 4096;

struct TcKernelParams {
    int M, N, K, batch;
    int npass;
    int pa[3], pb[3];
    int bm, bn;  // tile: bm is 128 or 256 rows
    int group_m;  // row tiles per group of the tile order
    uint32_t a_bytes;
    int a_kmajor, b_kmajor;
    int a_bcast, b_bcast;  // operand shared by all batch items
    int tiles_m, tiles_n;
    int num_kb;
    int stages;
    uint32_t b_bytes;
    uint32_t idesc;
    float alpha, beta;
    const float* bias;
    int bias_mode;
    int act;
    const void* residual;
    long long ldr, res_bs;
    void* out;
    long long ldo, out_bs;
    int out_prec;
    int vec_out, vec_res, vec_bias;
    int tma_out;  // epilogue goes through swizzled staging tiles and TMA stores
    DeviceStatus* status;
};

__device__ __forceinline__ void report_timeout(DeviceStatus* st, unsigned where) {
    // plain stores into mapped host memory (system-scope atomics over PCIe are not guaranteed)
    volatile unsigned int* f = &st->timeout_flag;
    volatile unsigned int* w = &st->timeout_where;
    if (*w == 0u) *w = where;
    *f = 1u;
    __threadfence_system();
}

// Epilogue arithmetic for 16 consecutive columns of one accumulator row:
// v = act(alpha*acc + beta*C + bias) + residual. Columns at or beyond N are left untouched.
// ACT is the activation code, or -1 to select it at run time (rare codes only).
// `pre`: the residual's 16 columns were fetched by the caller (`res_pre`, 16-byte vectors) instead of being read here.
template <typename OutT, int ACT>
__device__ __forceinline__ void epilogue_values(const TcKernelParams& p, const uint32_t (&r)[16], long long row, int col0, int b,
                                                bool row_ok, float (&v)[16], bool pre, const uint4 (&res_pre)[16 / (16 / int(sizeof(OutT)))]) {
    int ncols = p.N - col0 < 16 ? p.N - col0 : 16;
    if (ncols < 0 || !row_ok) ncols = 0;
#pragma unroll
    for (int j = 0; j < 16; j++) v[j] = __uint_as_float(r[j]) * p.alpha;
    constexpr int EPV = 16 / sizeof(OutT);  // elements per 16-byte vector
    const bool full = ncols == 16;
    if (p.beta != 0.f && ncols > 0) {
        const OutT* orow = static_cast<const OutT*>(p.out) + b * p.out_bs + row * p.ldo + col0;
        if (full && p.vec_out) {
#pragma unroll
            for (int q = 0; q < 16 / EPV; q++) {
                const Pack<OutT, EPV> c = *reinterpret_cast<const Pack<OutT, EPV>*>(orow + q * EPV);
#pragma unroll
                for (int e = 0; e < EPV; e++) v[q * EPV + e] += p.beta * to_float(c.v[e]);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 16; j++)
                if (j < ncols) v[j] += p.beta * to_float(orow[j]);
        }
    }
    if (p.bias_mode == 1 && ncols > 0) {
        if (full && p.vec_bias) {
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const float4 bv = __ldg(reinterpret_cast<const float4*>(p.bias + col0) + q);
                v[q * 4 + 0] += bv.x; v[q * 4 + 1] += bv.y; v[q * 4 + 2] += bv.z; v[q * 4 + 3] += bv.w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 16; j++)
                if (j < ncols) v[j] += __ldg(p.bias + col0 + j);
        }
    } else if (p.bias_mode == 2 && row_ok) {
        const float bv = __ldg(p.bias + row);
#pragma unroll
        for (int j = 0; j < 16; j++) v[j] += bv;
    }
    if constexpr (ACT == DOCC_B200_ACT_GELU_ERF) {
#pragma unroll
        for (int j = 0; j < 16; j++) {
            if constexpr (sizeof(OutT) == 2) v[j] = gelu_erf_16bit(v[j]);
            else v[j] = 0.5f * v[j] * (1.0f + erf_fast(v[j] * 0.70710678118654752440f));
        }
    } else if constexpr (ACT == DOCC_B200_ACT_RELU) {
#pragma unroll
        for (int j = 0; j < 16; j++) v[j] = fmaxf(v[j], 0.f);
    } else if constexpr (ACT == -1) {
#pragma unroll
        for (int j = 0; j < 16; j++) v[j] = apply_act_fast(p.act, v[j]);
    }
    if (pre) {
#pragma unroll
        for (int q = 0; q < 16 / EPV; q++) {
            const Pack<OutT, EPV> c = *reinterpret_cast<const Pack<OutT, EPV>*>(&res_pre[q]);
#pragma unroll
            for (int e = 0; e < EPV; e++) v[q * EPV + e] += to_float(c.v[e]);
        }
    } else if (p.residual && ncols > 0) {
        const OutT* rrow = static_cast<const OutT*>(p.residual) + b * p.res_bs + row * p.ldr + col0;
        if (full && p.vec_res) {
#pragma unroll
            for (int q = 0; q < 16 / EPV; q++) {
                const Pack<OutT, EPV> c = *reinterpret_cast<const Pack<OutT, EPV>*>(rrow + q * EPV);
#pragma unroll
                for (int e = 0; e < EPV; e++) v[q * EPV + e] += to_float(c.v[e]);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 16; j++)
                if (j < ncols) v[j] += to_float(rrow[j]);
        }
    }
}

// Direct store of 16 columns (used when the output is not 16-byte aligned for TMA).
template <typename OutT>
__device__ __forceinline__ void epilogue_store_direct(const TcKernelParams& p, const float (&v)[16], long long row, int col0, int b) {
    const int ncols = p.N - col0 < 16 ? p.N - col0 : 16;
    if (ncols <= 0) return;
    OutT* orow = static_cast<OutT*>(p.out) + b * p.out_bs + row * p.ldo + col0;
    constexpr int EPV = 16 / sizeof(OutT);
    if (ncols == 16 && p.vec_out) {
#pragma unroll
        for (int q = 0; q < 16 / EPV; q++) {
            Pack<OutT, EPV> o;
#pragma unroll
            for (int e = 0; e < EPV; e++) o.v[e] = from_float<OutT>(v[q * EPV + e]);
            *reinterpret_cast<Pack<OutT, EPV>*>(orow + q * EPV) = o;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 16; j++)
            if (j < ncols) orow[j] = from_float<OutT>(v[j]);
    }
}

// 16 columns of this lane's row into the warp's staging tile: 32 rows x 128 bytes, 128-byte swizzle
// (16-byte chunk c of row r sits at chunk c ^ (r & 7)), the layout a SWIZZLE_128B TMA store reads.
// `sub` is the index of the 16-column group inside the 128-byte row.
template <typename OutT>
__device__ __forceinline__ void epilogue_stage(uint32_t stage_base, int lane, int sub, const float (&v)[16]) {
    constexpr int EPV = 16 / sizeof(OutT);
    constexpr int CHUNKS = 16 / EPV;  // 16-byte chunks per 16 columns: 4 (fp32) or 2 (16-bit)
#pragma unroll
    for (int q = 0; q < CHUNKS; q++) {
        Pack<OutT, EPV> o;
#pragma unroll
        for (int e = 0; e < EPV; e++) o.v[e] = from_float<OutT>(v[q * EPV + e]);
        const uint4 w = *reinterpret_cast<const uint4*>(&o);
        const int chunk = sub * CHUNKS + q;
        const uint32_t dst = stage_base + uint32_t(lane) * 128u + uint32_t((chunk ^ (lane & 7)) * 16);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w.x), "r"(w.y), "r"(w.z), "r"(w.w) : "memory");
    }
}

// Fetches a 32-row x 128-byte residual tile with coalesced requests (all eight in flight together) and parks it in the
// warp's staging tile in the swizzled layout, once the previous TMA store has finished reading that tile. Kept out of
// line: inlined, its eight vectors push the epilogue's register allocation over the limit.
template <typename OutT>
__device__ __noinline__ void stage_residual_tile(const OutT* rbase, long long ldr, uint32_t stage_base, int lane) {
    constexpr int EPV = 16 / int(sizeof(OutT));
    uint4 rt[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int id = i * 32 + lane;  // 16-byte chunk (id & 7) of tile row (id >> 3)
        rt[i] = __ldg(reinterpret_cast<const uint4*>(rbase + (long long)(id >> 3) * ldr + (id & 7) * EPV));
    }
    if (lane == 0) tma_store_wait_read<0>();
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int id = i * 32 + lane;
        const int rr = id >> 3, ch = id & 7;
        const uint32_t dst = stage_base + uint32_t(rr) * 128u + uint32_t((ch ^ (rr & 7)) * 16);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(rt[i].x), "r"(rt[i].y), "r"(rt[i].z), "r"(rt[i].w) : "memory");
    }
    __syncwarp();
}

template <typename OutT, int ACT>
__device__ __forceinline__ void epilogue_tile(const TcKernelParams& p, const CUtensorMap* tm_out, uint32_t stage_base, uint32_t t_addr,
                                              int c_begin, int c_end, long long row, int row0, int n0, int b, int lane) {
    const bool row_ok = row < p.M;
    if (p.tma_out) {
        constexpr int BOX = 128 / sizeof(OutT);  // columns per 128-byte staging row
        constexpr int EPV = 16 / int(sizeof(OutT));  // elements per 16-byte vector
        constexpr int CHUNKS = 16 / EPV;             // vectors per 16 columns
        for (int c0 = c_begin; c0 < c_end; c0 += BOX) {
            // Residual: a thread owns an accumulator row, so reading "its" residual means 32 lanes touching 32 different
            // lines, 16 bytes at a time. When the whole 32 x 128-byte tile is in range the warp fetches it the other way
            // round instead, as eight coalesced 512-byte requests that are all in flight together, parks it in the staging
            // tile (same swizzled layout the result will have) and every lane then picks its row up from shared memory.
            // (16-bit results with the plain or the GELU / ReLU epilogue: the other instantiations have no registers to spare)
            const bool res_tile = sizeof(OutT) == 2 && ACT >= 0 && p.residual != nullptr && p.vec_res && row0 + 32 <= p.M && n0 + c0 + BOX <= p.N;
            if (res_tile) {
                stage_residual_tile<OutT>(static_cast<const OutT*>(p.residual) + b * p.res_bs + (long long)row0 * p.ldr + n0 + c0, p.ldr, stage_base, lane);
            } else {
                // the previous TMA store must have finished reading the staging tile
                if (lane == 0) tma_store_wait_read<0>();
                __syncwarp();
            }
            // 32 accumulator columns per tensor-memory load: half as many load/wait round trips per staging tile
#pragma unroll
            for (int sub = 0; sub < BOX / 16; sub += 2) {
                uint32_t r[32];
                tmem_ld_x32(t_addr + uint32_t(c0 + sub * 16), r);
                tmem_ld_wait();
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    uint32_t rh[16];
#pragma unroll
                    for (int j = 0; j < 16; j++) rh[j] = r[h * 16 + j];
                    float v[16];
                    uint4 rp[CHUNKS];
                    if (res_tile) {  // this lane's own row: the same addresses epilogue_stage overwrites right after
#pragma unroll
                        for (int q = 0; q < CHUNKS; q++) {
                            const int chunk = (sub + h) * CHUNKS + q;
                            const uint32_t src = stage_base + uint32_t(lane) * 128u + uint32_t((chunk ^ (lane & 7)) * 16);
                            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(rp[q].x), "=r"(rp[q].y), "=r"(rp[q].z), "=r"(rp[q].w) : "r"(src) : "memory");
                        }
                    }
                    epilogue_values<OutT, ACT>(p, rh, row, n0 + c0 + (sub + h) * 16, b, row_ok, v, res_tile, rp);
                    epilogue_stage<OutT>(stage_base, lane, sub + h, v);
                }
            }
            fence_proxy_async_smem();
            __syncwarp();
            // rows >= M and columns >= N are clipped by the tensor map
            if (lane == 0 && n0 + c0 < p.N && row0 < p.M) {
                tma_store_3d(tm_out, stage_base, n0 + c0, row0, b);
                tma_store_commit();
            }
        }
    } else {
        for (int c = c_begin; c < c_end; c += 16) {
            uint32_t r[16];
            tmem_ld_x16(t_addr + uint32_t(c), r);
            tmem_ld_wait();
            float v[16];
            const uint4 none[16 / (16 / int(sizeof(OutT)))] = {};
            epilogue_values<OutT, ACT>(p, r, row, n0 + c, b, row_ok, v, false, none);
            if (row_ok) epilogue_store_direct<OutT>(p, v, row, n0 + c, b);
        }
    }
}

// Tile coordinates of linear tile index t. Tiles are walked in groups of `group_m` row tiles
// (m fastest inside a group), so that the ~148 tiles in flight cover a near-square patch of C and
// the operand panels they share stay in L2.
__device__ __forceinline__ void tile_coords(const TcKernelParams& p, int t, int& b, int& m0, int& n0) {
    const int tiles_per_batch = p.tiles_m * p.tiles_n;
    b = t / tiles_per_batch;
    const int rem = t - b * tiles_per_batch;
    const int per_group = p.group_m * p.tiles_n;
    const int g = rem / per_group;
    const int first_m = g * p.group_m;
    const int gm = p.tiles_m - first_m < p.group_m ? p.tiles_m - first_m : p.group_m;
    const int in_group = rem - g * per_group;
    m0 = (first_m + in_group % gm) * p.bm;
    n0 = (in_group / gm) * p.bn;
}

__global__ void __launch_bounds__(kThreads, 1)
    tc_gemm_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmA1,
                   const __grid_constant__ CUtensorMap tmB0, const __grid_constant__ CUtensorMap tmB1,
                   const __grid_constant__ CUtensorMap tmOut, const TcKernelParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    const uint32_t sA = base;
    const uint32_t sB = sA + uint32_t(p.stages) * p.a_bytes;
    const uint32_t sStage = sB + uint32_t(p.stages) * p.b_bytes;  // eight 4 KB staging tiles for the TMA-store epilogue
    const uint32_t bars = sStage + kStagingBytes;
    auto full_bar = [&](int i) { return bars + 8u * uint32_t(i); };
    auto empty_bar = [&](int i) { return bars + 64u + 8u * uint32_t(i); };
    auto tfull_bar = [&](int i) { return bars + 128u + 8u * uint32_t(i); };
    auto tempty_bar = [&](int i) { return bars + 144u + 8u * uint32_t(i); };
    volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem_raw + (bars + 160u - raw_addr));

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // bm == 256: one tile owns both TMEM regions (rows 0-127 in columns [0,256), rows 128-255 in
    // [256,512)); bm == 128: the regions are two accumulator buffers used by alternate tiles.
    const bool tall = p.bm == 256;

    if (warp == 0 && lane == 0) {
        for (int i = 0; i < p.stages; i++) {
            mbar_init(full_bar(i), 1);
            mbar_init(empty_bar(i), 1);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(tfull_bar(i), 1);
            mbar_init(tempty_bar(i), tall ? 4 : 8);  // one arrival per epilogue warp that drains the region
        }
        fence_barrier_init();
        prefetch_tensormap(&tmA0);
        prefetch_tensormap(&tmB0);
        if (p.npass > 1) {
            prefetch_tensormap(&tmA1);
            prefetch_tensormap(&tmB1);
        }
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_holder)), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_holder;
    // everything before this point touches no global memory: under programmatic stream serialization it overlaps
    // the tail of the kernel launched before this one
    griddep_wait();
    griddep_launch_dependents();

    const int total_tiles = p.tiles_m * p.tiles_n * p.batch;
    const uint32_t stage_tx = p.a_bytes + uint32_t(p.bn) * 128u;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        // One lane issues everything, so the loop keeps its ring position incrementally (no division per
        // k-block): slot index, phase and destination addresses.
        if (lane == 0) {
            bool ok = true;
            uint32_t s = 0, ph = 0;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                int b, m0, n0;
                tile_coords(p, t, b, m0, n0);
                const int ba = p.a_bcast ? 0 : b, bb = p.b_bcast ? 0 : b;
                for (int pass = 0; pass < p.npass && ok; pass++) {
                    const CUtensorMap* ma = p.pa[pass] ? &tmA1 : &tmA0;
                    const CUtensorMap* mb = p.pb[pass] ? &tmB1 : &tmB0;
                    for (int k0 = 0; k0 < p.num_kb * kBK; k0 += kBK) {
                        const uint32_t full = full_bar(0) + 8u * s;
                        if (!mbar_wait(empty_bar(0) + 8u * s, ph ^ 1u)) {
                            report_timeout(p.status, 1);
                            ok = false;
                            break;
                        }
                        mbar_arrive_expect_tx(full, stage_tx);
                        const uint32_t a_dst = sA + s * p.a_bytes;
                        const uint32_t b_dst = sB + s * p.b_bytes;
                        if (p.a_kmajor) {
                            tma_load_3d(a_dst, ma, full, k0, m0, ba);
                        } else {
                            for (int j = 0; j < p.bm / 64; j++) tma_load_3d(a_dst + uint32_t(j) * 8192u, ma, full, m0 + 64 * j, k0, ba);
                        }
                        if (p.b_kmajor) {
                            tma_load_3d(b_dst, mb, full, k0, n0, bb);
                        } else {
                            for (int j = 0; j < p.bn / 64; j++) tma_load_3d(b_dst + uint32_t(j) * 8192u, mb, full, n0 + 64 * j, k0, bb);
                        }
                        if (++s == uint32_t(p.stages)) {
                            s = 0;
                            ph ^= 1u;
                        }
                    }
                }
            }
            if (!ok) {
                // let copies already in flight land before the CTA retires
                const long long t0 = clock64();
                while (clock64() - t0 < 200000) {
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- UMMA issuer ----------------
        // Also a single lane: descriptors advance by adds, the four 16-deep k-steps of a k-block go out in one asm block.
        if (lane == 0) {
            uint32_t lt = 0;
            bool ok = true;
            const int k_iters = p.npass * p.num_kb;
            // K-major tiles advance 32 bytes per k-step, MN-major tiles 2048 (16 rows of 128 bytes)
            const uint64_t a_desc0 = p.a_kmajor ? make_smem_desc(sA, 16u, 1024u) : make_smem_desc(sA, 8192u, 1024u);
            const uint64_t b_desc0 = p.b_kmajor ? make_smem_desc(sB, 16u, 1024u) : make_smem_desc(sB, 8192u, 1024u);
            const uint64_t a_step = p.a_kmajor ? 2 : 128, b_step = p.b_kmajor ? 2 : 128;
            const uint64_t a_stride = p.a_bytes >> 4, b_stride = p.b_bytes >> 4;  // per ring slot, in descriptor address units
            uint64_t a_desc = a_desc0, b_desc = b_desc0;
            uint32_t s = 0, ph = 0;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, lt++) {
                // the epilogue must have drained the accumulator region(s) this tile overwrites
                const uint32_t buf = tall ? 0u : (lt & 1u);
                const uint32_t wait_parity = tall ? ((lt & 1u) ^ 1u) : (((lt >> 1) & 1u) ^ 1u);
                if (!mbar_wait(tempty_bar(int(buf)), wait_parity) || (tall && !mbar_wait(tempty_bar(1), wait_parity))) {
                    report_timeout(p.status, 2);
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * 256u;
                uint32_t acc = 0;
                for (int k = 0; k < k_iters; k++) {
                    if (!mbar_wait(full_bar(0) + 8u * s, ph)) {
                        report_timeout(p.status, 3);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    umma_f16_ss_x4<1>(d_tmem, a_desc, b_desc, p.idesc, acc, a_step, b_step);
                    // tall: rows 128..255 of the A tile (16 KB further on in either layout) into the second region
                    if (tall) umma_f16_ss_x4<1>(d_tmem + 256u, a_desc + (16384u >> 4), b_desc, p.idesc, acc, a_step, b_step);
                    acc = 1;
                    umma_commit(empty_bar(0) + 8u * s);  // frees the slot once these MMAs have read it
                    a_desc += a_stride;
                    b_desc += b_stride;
                    if (++s == uint32_t(p.stages)) {
                        s = 0;
                        ph ^= 1u;
                        a_desc = a_desc0;
                        b_desc = b_desc0;
                    }
                }
                if (!ok) break;
                umma_commit(tfull_bar(int(buf)));  // accumulator complete
                if (tall) umma_commit(tfull_bar(1));
            }
        }
    } else {
        // ---------------- epilogue warps (two groups of four) ----------------
        const int q = warp & 3;          // tensor-memory lane quadrant this warp may read
        const int wg = (warp - 2) >> 2;  // 0 or 1
        uint32_t lt = 0;
        for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, lt++) {
            int b, m0, n0;
            tile_coords(p, t, b, m0, n0);
            const uint32_t region = tall ? uint32_t(wg) : (lt & 1u);
            const uint32_t parity = tall ? (lt & 1u) : ((lt >> 1) & 1u);
            if (!mbar_wait(tfull_bar(int(region)), parity)) {
                if (lane == 0) report_timeout(p.status, 4);
                break;
            }
            tc_fence_after();
            const int row0 = m0 + (tall ? wg * 128 : 0) + q * 32;
            const long long row = row0 + lane;
            const uint32_t t_addr = tmem_base + (uint32_t(q * 32) << 16) + region * 256u;
            // tall tiles: each group drains its own 128 rows; otherwise the groups split the columns
            // (at a multiple of 64 so that both halves are whole staging rows for every output type)
            const int half_cols = ((p.bn / 2) + 63) / 64 * 64;
            const int c_begin = tall ? 0 : (wg == 0 ? 0 : half_cols);
            const int c_end = tall ? p.bn : (wg == 0 ? (half_cols < p.bn ? half_cols : p.bn) : p.bn);
            const uint32_t stage_base = sStage + uint32_t(warp - 2) * 4096u;
#define DOCC_EPI(T, A) epilogue_tile<T, A>(p, &tmOut, stage_base, t_addr, c_begin, c_end, row, row0, n0, b, lane)
#define DOCC_EPI_ACT(T)                                                  \
    do {                                                                 \
        if (p.act == DOCC_B200_ACT_NONE) DOCC_EPI(T, 0);                 \
        else if (p.act == DOCC_B200_ACT_GELU_ERF) DOCC_EPI(T, 1);        \
        else if (p.act == DOCC_B200_ACT_RELU) DOCC_EPI(T, 2);            \
        else DOCC_EPI(T, -1);                                            \
    } while (0)
            if (p.out_prec == DOCC_B200_PREC_S) DOCC_EPI_ACT(float);
            else if (p.out_prec == DOCC_B200_PREC_B) DOCC_EPI_ACT(__nv_bfloat16);
            else DOCC_EPI_ACT(__half);
#undef DOCC_EPI_ACT
#undef DOCC_EPI
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(int(region)));
        }
        if (p.tma_out && lane == 0) tma_store_wait<0>();  // staging tiles must outlive the bulk stores that read them
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---- CTA-pair variant (cta_group::2) ------------------------------------------------------------------
// A cluster of two CTAs owns a 256 x bn tile, bn = 256 or 512. Per k-block rank r loads rows
// [128r, 128r+128) of the A tile and, for each 256-column block of the tile, rows [128r, 128r+128) of
// that block of B: 32 KB (bn = 256) or 48 KB (bn = 512) per CTA, against 64 KB for a single-CTA 256x256
// tile of the same arithmetic, which is what relieves the L2 -> SM fabric. The leader's UMMA thread issues
// M = 256, N = 256 instructions for both CTAs; its commits release the stage in both and publish both
// accumulator halves. Each CTA drains its own 128 accumulator rows through the same epilogue as the
// single-CTA kernel and reports the drain to the leader. bn = 256 double-buffers the accumulator so the
// drain overlaps the next main loop; bn = 512 fills tensor memory (no overlap: long K only).
// Operands must be K-major.
__global__ void __launch_bounds__(kThreads, 1)
    tc_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmA1,
                        const __grid_constant__ CUtensorMap tmB0, const __grid_constant__ CUtensorMap tmB1,
                        const __grid_constant__ CUtensorMap tmOut, const TcKernelParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    constexpr uint32_t kHalf = 128u * 128u;  // 128 rows x 64 bf16
    const bool wide = p.bn == 512;
    const int nh = wide ? 2 : 1;  // 256-column blocks per tile
    const uint32_t b_stage = uint32_t(nh) * kHalf;
    const uint32_t sA = base;
    const uint32_t sB = sA + uint32_t(p.stages) * kHalf;
    const uint32_t sStage = sB + uint32_t(p.stages) * b_stage;
    const uint32_t bars = sStage + kStagingBytes;
    auto full_bar = [&](int i) { return bars + 8u * uint32_t(i); };
    auto empty_bar = [&](int i) { return bars + 64u + 8u * uint32_t(i); };
    auto tfull_bar = [&](int i) { return bars + 128u + 8u * uint32_t(i); };
    auto tempty_bar = [&](int i) { return bars + 144u + 8u * uint32_t(i); };
    volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem_raw + (bars + 160u - raw_addr));

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1;
    const int n_pairs = gridDim.x >> 1;

    if (warp == 0 && lane == 0) {
        for (int i = 0; i < p.stages; i++) {
            mbar_init(full_bar(i), 1);   // waited on in the leader only: its producer's arrive + both CTAs' bytes
            mbar_init(empty_bar(i), 1);  // one multicast commit per use
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(tfull_bar(i), 1);
            // the leader's copy collects the drains of both CTAs: all eight epilogue warps of each for a
            // double-buffered 256-column accumulator, one group of four per 256-column block when wide
            mbar_init(tempty_bar(i), wide ? 8 : 16);
        }
        fence_barrier_init();
        prefetch_tensormap(&tmA0);
        prefetch_tensormap(&tmB0);
        if (p.npass > 1) {
            prefetch_tensormap(&tmA1);
            prefetch_tensormap(&tmB1);
        }
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_holder)), kTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();  // the peer's barriers are initialised before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_holder;
    // everything before this point touches no global memory: under programmatic stream serialization it overlaps
    // the tail of the kernel launched before this one
    griddep_wait();
    griddep_launch_dependents();

    const int total_tiles = p.tiles_m * p.tiles_n * p.batch;

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        // One lane issues everything, so the loop keeps its ring position incrementally (no division per
        // k-block): slot index, phase, destination addresses and the leader's barrier address.
        if (lane == 0) {
            bool ok = true;
            const uint32_t stage_tx = 2u * (kHalf + b_stage);  // both CTAs' A and B parts
            const uint32_t lead_full0 = map_to_cta(full_bar(0), 0);
            const int row_off = 128 * int(rank);
            uint32_t s = 0, ph = 0;
            for (int t = pair; t < total_tiles && ok; t += n_pairs) {
                int b, m0, n0;
                tile_coords(p, t, b, m0, n0);
                const int ba = p.a_bcast ? 0 : b, bb = p.b_bcast ? 0 : b;
                m0 += row_off;
                n0 += row_off;
                for (int pass = 0; pass < p.npass && ok; pass++) {
                    const CUtensorMap* ma = p.pa[pass] ? &tmA1 : &tmA0;
                    const CUtensorMap* mb = p.pb[pass] ? &tmB1 : &tmB0;
                    for (int k0 = 0; k0 < p.num_kb * kBK; k0 += kBK) {
                        if (!mbar_wait(empty_bar(0) + 8u * s, ph ^ 1u)) {
                            report_timeout(p.status, 41);
                            ok = false;
                            break;
                        }
                        const uint32_t lead_full = lead_full0 + 8u * s;
                        if (leader) mbar_arrive_expect_tx(full_bar(0) + 8u * s, stage_tx);
                        tma_load_3d_pair(sA + s * kHalf, ma, lead_full, k0, m0, ba);
                        tma_load_3d_pair(sB + s * b_stage, mb, lead_full, k0, n0, bb);
                        if (wide) tma_load_3d_pair(sB + s * b_stage + kHalf, mb, lead_full, k0, n0 + 256, bb);
                        if (++s == uint32_t(p.stages)) {
                            s = 0;
                            ph ^= 1u;
                        }
                    }
                }
            }
            if (!ok) {
                // let copies already in flight land before the CTA retires
                const long long t0 = clock64();
                while (clock64() - t0 < 200000) {
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- UMMA issuer (leader only) ----------------
        if (leader && lane == 0) {
            uint32_t lt = 0;
            bool ok = true;
            const int k_iters = p.npass * p.num_kb;
            const uint64_t a_desc0 = make_smem_desc(sA, 16u, 1024u), b_desc0 = make_smem_desc(sB, 16u, 1024u);
            const uint64_t a_stride = kHalf >> 4, b_stride = b_stage >> 4;  // per ring slot, in descriptor address units
            uint64_t a_desc = a_desc0, b_desc = b_desc0;
            uint32_t s = 0, ph = 0;
            for (int t = pair; t < total_tiles && ok; t += n_pairs, lt++) {
                // both CTAs must have drained the accumulator region(s) this tile overwrites
                const uint32_t buf = wide ? 0u : (lt & 1u);
                const uint32_t wait_parity = wide ? ((lt & 1u) ^ 1u) : (((lt >> 1) & 1u) ^ 1u);
                if (!mbar_wait(tempty_bar(int(buf)), wait_parity) || (wide && !mbar_wait(tempty_bar(1), wait_parity))) {
                    report_timeout(p.status, 42);
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * 256u;
                uint32_t acc = 0;
                for (int k = 0; k < k_iters; k++) {
                    if (!mbar_wait(full_bar(0) + 8u * s, ph)) {
                        report_timeout(p.status, 43);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    umma_f16_ss_x4<2>(d_tmem, a_desc, b_desc, p.idesc, acc, 2, 2);  // +32 bytes per 16-deep k-step
                    if (wide) umma_f16_ss_x4<2>(d_tmem + 256u, a_desc, b_desc + (kHalf >> 4), p.idesc, acc, 2, 2);
                    acc = 1;
                    umma_commit_pair(empty_bar(0) + 8u * s, 3);  // both CTAs may refill the slot
                    a_desc += a_stride;
                    b_desc += b_stride;
                    if (++s == uint32_t(p.stages)) {
                        s = 0;
                        ph ^= 1u;
                        a_desc = a_desc0;
                        b_desc = b_desc0;
                    }
                }
                if (!ok) break;
                umma_commit_pair(tfull_bar(int(buf)), 3);  // accumulator complete in both CTAs
                if (wide) umma_commit_pair(tfull_bar(1), 3);
            }
        }
    } else {
        // ---------------- epilogue warps: this CTA's 128 rows of the tile ----------------
        const int q = warp & 3;
        const int wg = (warp - 2) >> 2;
        uint32_t lt = 0;
        for (int t = pair; t < total_tiles; t += n_pairs, lt++) {
            int b, m0, n0;
            tile_coords(p, t, b, m0, n0);
            const uint32_t region = wide ? uint32_t(wg) : (lt & 1u);
            const uint32_t parity = wide ? (lt & 1u) : ((lt >> 1) & 1u);
            if (!mbar_wait(tfull_bar(int(region)), parity)) {
                if (lane == 0) report_timeout(p.status, 44);
                break;
            }
            tc_fence_after();
            const int row0 = m0 + 128 * int(rank) + q * 32;
            const long long row = row0 + lane;
            // wide: accumulator column c is tile column c and group wg drains block wg; otherwise the
            // groups split the 256 columns of the current buffer
            const uint32_t t_addr = tmem_base + (uint32_t(q * 32) << 16) + (wide ? 0u : region * 256u);
            const int c_begin = wide ? 256 * wg : (wg == 0 ? 0 : 128);
            const int c_end = wide ? 256 * wg + 256 : (wg == 0 ? 128 : 256);
            const uint32_t stage_base = sStage + uint32_t(warp - 2) * 4096u;
#define DOCC_EPI(T, A) epilogue_tile<T, A>(p, &tmOut, stage_base, t_addr, c_begin, c_end, row, row0, n0, b, lane)
#define DOCC_EPI_ACT(T)                                                  \
    do {                                                                 \
        if (p.act == DOCC_B200_ACT_NONE) DOCC_EPI(T, 0);                 \
        else if (p.act == DOCC_B200_ACT_GELU_ERF) DOCC_EPI(T, 1);        \
        else if (p.act == DOCC_B200_ACT_RELU) DOCC_EPI(T, 2);            \
        else DOCC_EPI(T, -1);                                            \
    } while (0)
            if (p.out_prec == DOCC_B200_PREC_S) DOCC_EPI_ACT(float);
            else if (p.out_prec == DOCC_B200_PREC_B) DOCC_EPI_ACT(__nv_bfloat16);
            else DOCC_EPI_ACT(__half);
#undef DOCC_EPI_ACT
#undef DOCC_EPI
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(tempty_bar(int(region)), 0));
        }
        if (p.tma_out && lane == 0) tma_store_wait<0>();
    }

    tc_fence_before();
    __syncthreads();
    cluster_sync();  // neither CTA retires while the other may still signal its barriers or read its tiles
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, kTmemCols);
    }
}

// ---- fp32 -> bf16 hi/lo split ---------------------------------------------------------------------
__device__ __forceinline__ void split1(float x, __nv_bfloat16& hi, __nv_bfloat16& lo) {
    hi = __float2bfloat16_rn(x);
    lo = __float2bfloat16_rn(x - __bfloat162float(hi));
}

__global__ void __launch_bounds__(256) split_rows_kernel(const float* __restrict__ X, int64_t rows, int64_t cols, int64_t ld,
                                                         int64_t bs, __nv_bfloat16* __restrict__ hi,
                                                         __nv_bfloat16* __restrict__ lo, int64_t ldo, int64_t obs, int vec) {
    ptx::griddep_wait();
    ptx::griddep_launch_dependents();
    const int64_t b = blockIdx.z;
    X += b * bs;
    hi += b * obs;
    lo += b * obs;
    if (vec) {
        const int64_t cpr = cols / 4;
        const int64_t total = rows * cpr;
        for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x) {
            const int64_t r = i / cpr, c = (i - r * cpr) * 4;
            const float4 x = *reinterpret_cast<const float4*>(X + r * ld + c);
            Pack<__nv_bfloat16, 4> h, l;
            split1(x.x, h.v[0], l.v[0]);
            split1(x.y, h.v[1], l.v[1]);
            split1(x.z, h.v[2], l.v[2]);
            split1(x.w, h.v[3], l.v[3]);
            *reinterpret_cast<Pack<__nv_bfloat16, 4>*>(hi + r * ldo + c) = h;
            *reinterpret_cast<Pack<__nv_bfloat16, 4>*>(lo + r * ldo + c) = l;
        }
    } else {
        const int64_t total = rows * cols;
        for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x) {
            const int64_t r = i / cols, c = i - r * cols;
            split1(X[r * ld + c], hi[r * ldo + c], lo[r * ldo + c]);
        }
    }
}

// out[c][r] = split(X[r][c]); 32x32 tiles through shared memory keep both sides coalesced.
__global__ void __launch_bounds__(256) split_transpose_kernel(const float* __restrict__ X, int64_t rows, int64_t cols,
                                                              int64_t ld, int64_t bs, __nv_bfloat16* __restrict__ hi,
                                                              __nv_bfloat16* __restrict__ lo, int64_t ldo, int64_t obs) {
    ptx::griddep_wait();
    ptx::griddep_launch_dependents();
    __shared__ float tile[32][33];
    const int64_t b = blockIdx.z;
    X += b * bs;
    hi += b * obs;
    lo += b * obs;
    const int64_t tiles_c = (cols + 31) / 32, tiles_r = (rows + 31) / 32;
    for (int64_t t = blockIdx.x; t < tiles_c * tiles_r; t += gridDim.x) {
        const int64_t r0 = (t / tiles_c) * 32, c0 = (t % tiles_c) * 32;
        const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
        for (int j = ty; j < 32; j += 8) {
            const int64_t r = r0 + j, c = c0 + tx;
            tile[j][tx] = (r < rows && c < cols) ? X[r * ld + c] : 0.f;
        }
        __syncthreads();
        for (int j = ty; j < 32; j += 8) {
            const int64_t c = c0 + j, r = r0 + tx;
            if (c < cols && r < rows) split1(tile[tx][j], hi[c * ldo + r], lo[c * ldo + r]);
        }
        __syncthreads();
    }
}

// ---- tensor map encoding --------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn g_encode = nullptr;
std::once_flag g_encode_once;

int get_encode(EncodeFn* fn) {
    std::call_once(g_encode_once, [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            g_encode = reinterpret_cast<EncodeFn>(f);
        else
            (void)cudaGetLastError();
    });
    if (!g_encode) return set_error(DOCC_B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    *fn = g_encode;
    return DOCC_B200_OK;
}

bool g_attr_set[16] = {false};
bool g_attr_pair_set[16] = {false};

}  // namespace

int encode_tmap(CUtensorMap* map, CUtensorMapDataType dtype, size_t elem_size, CUtensorMapSwizzle swizzle, const void* base,
                int rank, const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box) {
    EncodeFn fn;
    DOCC_TRY(get_encode(&fn));
    cuuint64_t gd[5], gs[5];
    cuuint32_t bx[5], es[5];
    for (int i = 0; i < rank; i++) {
        gd[i] = dims[i];
        bx[i] = box[i];
        es[i] = 1;
        if (i > 0) gs[i - 1] = strides_bytes[i - 1];
    }
    (void)elem_size;
    CUresult r = fn(map, dtype, cuuint32_t(rank), const_cast<void*>(base), gd, gs, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        return set_error(DOCC_B200_ERR_CUDA,
                         "cuTensorMapEncodeTiled failed (%d): rank %d dims [%llu,%llu,%llu,%llu] strides [%llu,%llu,%llu] box "
                         "[%u,%u,%u,%u] base %p",
                         int(r), rank, (unsigned long long)gd[0], (unsigned long long)(rank > 1 ? gd[1] : 0),
                         (unsigned long long)(rank > 2 ? gd[2] : 0), (unsigned long long)(rank > 3 ? gd[3] : 0),
                         (unsigned long long)(rank > 1 ? gs[0] : 0), (unsigned long long)(rank > 2 ? gs[1] : 0),
                         (unsigned long long)(rank > 3 ? gs[2] : 0), bx[0], rank > 1 ? bx[1] : 0, rank > 2 ? bx[2] : 0,
                         rank > 3 ? bx[3] : 0, base);
    }
    return DOCC_B200_OK;
}

int encode_tmap_16bit(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                      const uint32_t* box) {
    return encode_tmap(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, CU_TENSOR_MAP_SWIZZLE_128B, base, rank, dims, strides_bytes, box);
}

int split_f32_to_bf16x2(Ctx* ctx, const float* X, int64_t rows, int64_t cols, int64_t ld, int64_t batch, int64_t batch_stride,
                        bool transpose, __nv_bfloat16* hi, __nv_bfloat16* lo, int64_t ld_out, int64_t out_batch_stride) {
    if (rows == 0 || cols == 0 || batch == 0) return DOCC_B200_OK;
    const int64_t cap = int64_t(ctx->sm_count) * 8;
    if (!transpose) {
        const int vec = (cols % 4 == 0 && ld % 4 == 0 && ld_out % 4 == 0 && batch_stride % 4 == 0 && out_batch_stride % 4 == 0 &&
                         reinterpret_cast<uintptr_t>(X) % 16 == 0 && reinterpret_cast<uintptr_t>(hi) % 8 == 0 &&
                         reinterpret_cast<uintptr_t>(lo) % 8 == 0)
                            ? 1
                            : 0;
        const int64_t items = vec ? rows * cols / 4 : rows * cols;
        int64_t blocks = ceil_div(items, 256);
        if (blocks > cap) blocks = cap;
        dim3 grid(unsigned(blocks), 1, unsigned(batch));
        DOCC_CUDA_TRY(launch_pdl(split_rows_kernel, grid, dim3(256), 0, ctx->stream, X, rows, cols, ld, batch_stride, hi, lo, ld_out, out_batch_stride, vec));
        return after_launch(ctx, "split_rows_kernel");
    }
    int64_t blocks = ceil_div(rows, 32) * ceil_div(cols, 32);
    if (blocks > cap) blocks = cap;
    dim3 grid(unsigned(blocks), 1, unsigned(batch));
    DOCC_CUDA_TRY(launch_pdl(split_transpose_kernel, grid, dim3(256), 0, ctx->stream, X, rows, cols, ld, batch_stride, hi, lo, ld_out, out_batch_stride));
    return after_launch(ctx, "split_transpose_kernel");
}

int tc_gemm(Ctx* ctx, int ab_format, int64_t M, int64_t N, int64_t K, int64_t batch, int npass, const TcOperand* A, const int* pa,
            const TcOperand* B, const int* pb, const TcEpilogue& ep) {
    if (M == 0 || N == 0 || batch == 0) return DOCC_B200_OK;
    if (K <= 0) return set_error(DOCC_B200_ERR_UNSUPPORTED, "tc_gemm: K must be positive");
    if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX || batch > 65535 * 64) return set_error(DOCC_B200_ERR_UNSUPPORTED, "tc_gemm: extent too large");
    if (npass < 1 || npass > 3) return set_error(DOCC_B200_ERR_INVALID_ARG, "tc_gemm: npass %d", npass);
    int n_a = 0, n_b = 0;
    for (int i = 0; i < npass; i++) {
        if (pa[i] + 1 > n_a) n_a = pa[i] + 1;
        if (pb[i] + 1 > n_b) n_b = pb[i] + 1;
    }
    auto aligned = [](const TcOperand& o) {
        return reinterpret_cast<uintptr_t>(o.ptr) % 16 == 0 && o.ld % 8 == 0 && o.batch_stride % 8 == 0;
    };
    for (int i = 0; i < n_a; i++)
        if (!aligned(A[i]) || A[i].k_major != A[0].k_major) return set_error(DOCC_B200_ERR_UNSUPPORTED, "tc_gemm: A operand not 16-byte aligned");
    for (int i = 0; i < n_b; i++)
        if (!aligned(B[i]) || B[i].k_major != B[0].k_major) return set_error(DOCC_B200_ERR_UNSUPPORTED, "tc_gemm: B operand not 16-byte aligned");

    TcKernelParams p;
    memset(&p, 0, sizeof(p));
    p.M = int(M); p.N = int(N); p.K = int(K); p.batch = int(batch);
    p.npass = npass;
    for (int i = 0; i < npass; i++) { p.pa[i] = pa[i]; p.pb[i] = pb[i]; }
    p.a_kmajor = A[0].k_major ? 1 : 0;
    p.b_kmajor = B[0].k_major ? 1 : 0;
    p.a_bcast = (batch > 1 && A[0].batch_stride == 0) ? 1 : 0;
    p.b_bcast = (batch > 1 && B[0].batch_stride == 0) ? 1 : 0;

    // Tile shape. L2 feeds an SM at most ~64 B/clk, so the tensor pipe only stays busy when a
    // k-block's flops per loaded byte are high: 256x256 tiles (131 flop/B) run at full rate,
    // 128x256 at ~0.68, 128x128 at ~0.5. Small problems prefer more, smaller tiles. Pick the
    // candidate with the lowest (waves x tile area / efficiency).
    const bool heavy_epilogue = ep.bias || ep.act != DOCC_B200_ACT_NONE || ep.residual || ep.beta != 0.f;
    int bm = 128, bn;
    if (N <= 64) {
        bn = p.b_kmajor ? int(ceil_div(N, 16) * 16) : 64;
    } else {
        static const struct { int bm, bn; double eff; } cand[] = {{256, 256, 1.0}, {128, 256, 0.68}, {128, 128, 0.5}, {128, 64, 0.33}};
        double best = 0;
        bn = 64;
        for (const auto& c : cand) {
            if (c.bm == 256 && M <= 128) continue;
            // a 256-row tile owns all of TMEM, so its epilogue does not overlap the next main loop:
            // only worth it when the main loop is long (longer still when the drain also has to load
            // bias / residual or evaluate an activation)
            if (c.bm == 256 && K * npass < (heavy_epilogue ? 2048 : 1024)) continue;
            if (c.bn > 64 && c.bn / 2 >= N) continue;
            const int64_t tiles = ceil_div(M, c.bm) * ceil_div(N, c.bn) * batch;
            const double cost = double(ceil_div(tiles, ctx->sm_count)) * c.bm * c.bn / c.eff;
            if (best == 0 || cost < best) {
                best = cost;
                bm = c.bm;
                bn = c.bn;
            }
        }
    }
    // CTA pairs (cta_group::2) for large K-major problems: 256x256 tiles at half the shared-memory and, with
    // 256x512 tiles on a long K, three quarters of the L2 -> SM traffic of the single-CTA kernel
    static const int pair_mode = [] { const char* e = getenv("DOCC_B200_GEMM_PAIR"); return e ? atoi(e) : 1; }();
    bool use_pair = pair_mode && p.a_kmajor && p.b_kmajor && M >= 256 && N >= 256 && ctx->sm_count % 2 == 0 && K * npass >= 512;
    if (use_pair) {
        const int pairs = ctx->sm_count / 2;
        const int64_t t256 = ceil_div(M, 256) * ceil_div(N, 256) * batch, t512 = ceil_div(M, 256) * ceil_div(N, 512) * batch;
        if (t256 < pairs) use_pair = false;
        else {
            bm = 256;
            bn = 256;
            const bool wide_ok = pair_mode == 2 || (pair_mode == 1 && K * npass >= 4096);  // pair_mode 3: never
            if (wide_ok && t512 >= pairs && double(ceil_div(t512, pairs)) * 512 <= double(ceil_div(t256, pairs)) * 256 * 1.05) bn = 512;
        }
    }
    p.bm = bm;
    p.bn = bn;
    p.a_bytes = uint32_t(bm) * 128u;
    p.tiles_m = int(ceil_div(M, bm));
    p.tiles_n = int(ceil_div(N, bn));
    p.group_m = bm == 256 ? 12 : 16;
    p.num_kb = int(ceil_div(K, kBK));
    p.b_bytes = uint32_t((bn * 128 + 1023) / 1024 * 1024);
    int stages = (kSmemBudget - 2048 - int(kStagingBytes)) / int(p.a_bytes + p.b_bytes);
    if (stages > kMaxStages) stages = kMaxStages;
    const int64_t k_iters = int64_t(p.num_kb) * npass;
    if (stages > k_iters && k_iters >= 2) stages = int(k_iters);
    if (stages < 2) stages = 2;
    p.stages = stages;
    p.idesc = make_idesc(128, bn, ab_format, p.a_kmajor ? 0 : 1, p.b_kmajor ? 0 : 1);
    if (use_pair) {
        stages = (kSmemBudget - 2048 - int(kStagingBytes)) / ((1 + bn / 256) * 128 * 128);
        if (stages > kMaxStages) stages = kMaxStages;
        if (stages > k_iters && k_iters >= 2) stages = int(k_iters);
        if (stages < 2) stages = 2;
        p.stages = stages;
        p.idesc = make_idesc(256, 256, ab_format, 0, 0);
    }

    p.alpha = ep.alpha; p.beta = ep.beta;
    p.bias = ep.bias; p.bias_mode = ep.bias ? ep.bias_mode : 0;
    p.act = ep.act;
    p.residual = ep.residual; p.ldr = ep.ldr; p.res_bs = ep.residual_batch_stride;
    p.out = ep.out; p.ldo = ep.ldo; p.out_bs = ep.out_batch_stride; p.out_prec = ep.out_prec;
    const size_t oes = prec_size(ep.out_prec);
    if (oes != 2 && oes != 4) return set_error(DOCC_B200_ERR_INVALID_ARG, "tc_gemm: output precision %d", ep.out_prec);
    const int64_t epv = 16 / int64_t(oes);
    p.vec_out = (reinterpret_cast<uintptr_t>(ep.out) % 16 == 0 && ep.ldo % epv == 0 && ep.out_batch_stride % epv == 0) ? 1 : 0;
    p.vec_res = (ep.residual && reinterpret_cast<uintptr_t>(ep.residual) % 16 == 0 && ep.ldr % epv == 0 &&
                 ep.residual_batch_stride % epv == 0)
                    ? 1
                    : 0;
    p.vec_bias = (ep.bias && reinterpret_cast<uintptr_t>(ep.bias) % 16 == 0) ? 1 : 0;
    p.tma_out = p.vec_out;
    p.status = ctx->status_dev;

    CUtensorMap maps[5];
    memset(maps, 0, sizeof(maps));
    if (p.tma_out) {
        // output as [batch][M][N] with 32-row x 128-byte boxes; the map clips the M and N tails
        const uint64_t od[3] = {uint64_t(N), uint64_t(M), uint64_t(batch)};
        uint64_t obs = uint64_t(ep.out_batch_stride) * oes;
        if (batch == 1 || obs == 0) obs = uint64_t(ep.ldo) * oes * uint64_t(M);
        const uint64_t os[2] = {uint64_t(ep.ldo) * oes, obs};
        const uint32_t ob[3] = {uint32_t(128 / oes), 32, 1};
        const CUtensorMapDataType odt = ep.out_prec == DOCC_B200_PREC_S ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                        : ep.out_prec == DOCC_B200_PREC_B ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                                          : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
        DOCC_TRY(encode_tmap(&maps[4], odt, oes, CU_TENSOR_MAP_SWIZZLE_128B, ep.out, 3, od, os, ob));
    }
    auto encode_operand = [&](CUtensorMap* m, const TcOperand& o, int64_t mn, uint32_t mn_box, bool bcast) -> int {
        const uint64_t nb = bcast ? 1 : uint64_t(batch);
        uint64_t bs_bytes = uint64_t(o.batch_stride) * 2;
        if (nb == 1 || bs_bytes == 0) bs_bytes = uint64_t(o.ld) * 2 * uint64_t(o.k_major ? mn : K);
        if (o.k_major) {
            const uint64_t dims[3] = {uint64_t(K), uint64_t(mn), nb};
            const uint64_t strides[2] = {uint64_t(o.ld) * 2, bs_bytes};
            const uint32_t box[3] = {uint32_t(kBK), mn_box, 1};
            return encode_tmap_16bit(m, o.ptr, 3, dims, strides, box);
        }
        const uint64_t dims[3] = {uint64_t(mn), uint64_t(K), nb};
        const uint64_t strides[2] = {uint64_t(o.ld) * 2, bs_bytes};
        const uint32_t box[3] = {64, uint32_t(kBK), 1};
        return encode_tmap_16bit(m, o.ptr, 3, dims, strides, box);
    };
    for (int i = 0; i < 2; i++) {
        DOCC_TRY(encode_operand(&maps[i], A[i < n_a ? i : 0], M, use_pair ? 128u : uint32_t(bm), p.a_bcast || batch == 1));
        DOCC_TRY(encode_operand(&maps[2 + i], B[i < n_b ? i : 0], N, use_pair ? 128u : uint32_t(bn), p.b_bcast || batch == 1));
    }
    if (use_pair) {
        const size_t smem2 = size_t(stages) * ((1 + bn / 256) * 128 * 128) + kStagingBytes + 1024 + 256;
        if (!g_attr_pair_set[ctx->device & 15]) {
            DOCC_CUDA_TRY(cudaFuncSetAttribute(tc_gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget));
            g_attr_pair_set[ctx->device & 15] = true;
        }
        const int64_t tiles = int64_t(p.tiles_m) * p.tiles_n * batch;
        const int64_t pairs = tiles < ctx->sm_count / 2 ? tiles : ctx->sm_count / 2;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(unsigned(2 * pairs), 1, 1);
        cfg.blockDim = dim3(kThreads, 1, 1);
        cfg.dynamicSmemBytes = smem2;
        cfg.stream = ctx->stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // the kernel waits (griddepcontrol.wait) after its set-up
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 2;
        DOCC_CUDA_TRY(cudaLaunchKernelEx(&cfg, tc_gemm_pair_kernel, maps[0], maps[1], maps[2], maps[3], maps[4], p));
        return after_launch(ctx, "tc_gemm_pair_kernel");
    }

    const size_t smem = size_t(stages) * (p.a_bytes + p.b_bytes) + kStagingBytes + 1024 + 256;
    if (!g_attr_set[ctx->device & 15]) {
        DOCC_CUDA_TRY(cudaFuncSetAttribute(tc_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget));
        g_attr_set[ctx->device & 15] = true;
    }
    const int64_t total_tiles = int64_t(p.tiles_m) * p.tiles_n * batch;
    const int grid = int(total_tiles < ctx->sm_count ? total_tiles : ctx->sm_count);
    DOCC_CUDA_TRY(launch_pdl(tc_gemm_kernel, dim3(unsigned(grid)), dim3(kThreads), smem, ctx->stream, maps[0], maps[1], maps[2], maps[3], maps[4], p));
    return after_launch(ctx, "tc_gemm_kernel");
}

}  // namespace docc_b200
