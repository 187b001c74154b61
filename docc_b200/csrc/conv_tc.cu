// Implicit-GEMM 2-D convolution (stride 1, dilation 1, one group) on tcgen05.
//
// docc's expansion of ConvNode (conv_node.cpp:243-399) gives every output element its own
// sequential C_in*kh*kw FMA chain. Here, per image,  Y_n[oc, pixel] = sum_{tap, c} W[oc, tap, c] *
// X_n[pixel + tap, c]  is a GEMM with M = C_out, N = output pixels, K = kh*kw*C_in:
//   1. fp32 inputs: one launch re-lays X from NCHW to NHWC 16-bit (bf16 hi and lo planes) and W from
//      [oc][c][kh][kw] to [oc][kh][kw][c], so that K is contiguous for both operands. 16-bit inputs of narrow images
//      skip this: conv_nchw_kernel reads the NCHW input in place and transposes it in shared memory (and, for 3x3
//      filters over one channel block, takes the weights as they lie and keeps them on the SM);
//   2. a persistent warp-specialised kernel (same skeleton as the GEMM engine: TMA producer warp,
//      UMMA issuer warp, epilogue warps, two TMEM accumulators) walks tiles of 128 output channels
//      x up to four output rows. Narrow images (conv_halo_kernel): the tile's input neighbourhood is
//      loaded once per 64-channel block and every tap reads it through a shifted descriptor. Wide
//      images (conv_tc_kernel): for each filter tap the producer issues one TMA load per output row
//      with the tap's (kh - pad, kw - pad) shift in the *outer* coordinates. Rows and columns that
//      fall outside the image are zero-filled by TMA, which is the zero padding;
//   3. the accumulator tile is [oc lanes x pixel columns], i.e. already NCHW: it leaves through
//      swizzled staging tiles and TMA stores with the bias added.
// fp32 inputs run three passes (w_lo*x_hi, w_hi*x_lo, w_hi*x_hi) into the same accumulator.
#include <cstdlib>
#include <type_traits>

#include "conv.h"
#include "device_math.cuh"
#include "gemm_tc.h"
#include "ptx.cuh"

namespace docc_b200 {
namespace {

using namespace ptx;

constexpr int kThreads = 192;
constexpr uint32_t kABytes = 128 * 64 * 2;
constexpr uint32_t kBBytes = 256 * 64 * 2;
constexpr int kStages = 4;
constexpr uint32_t kTmemCols = 512;

struct ConvKernelParams {
    int N, C, H, W, c_out, kh, kw, pad_h, pad_w, Ho, Wo;
    int npass;
    int pw[3], px[3];  // weight / input plane used by each pass
    int r_max;         // output rows per tile (r_max * Wo <= 256)
    int tiles_m;
    long long total_units;  // tiles_m * N * Ho output-row units
    int w_stages;  // halo variant: depth of the weight ring
    int x_chunks;  // fused variant: depth of the input staging ring
    int tma_out;  // Y rows are 16-byte aligned: full 32-pixel groups go out through TMA stores
    int even_rows;  // tiles of an even number of rows where the range allows it (two-row accumulators)
    int paired;  // halo variant, split operands: three halo slots, the high weight plane streamed once for both input planes
    const float* bias;
    float* Y;
    DeviceStatus* status;
};

__device__ __forceinline__ void conv_timeout(DeviceStatus* st, unsigned where) {
    volatile unsigned int* f = &st->timeout_flag;
    volatile unsigned int* w = &st->timeout_where;
    if (*w == 0u) *w = where;
    *f = 1u;
    __threadfence_system();
}

struct Tile {
    int m0, n, oh0, rows;
};

// Work is the list of (channel tile, image, output row) units; CTA i owns the contiguous range
// [i*U/G, (i+1)*U/G) and cuts it into tiles of at most r_max rows inside one image.
__device__ __forceinline__ bool next_tile(const ConvKernelParams& p, long long& u, long long u_end, Tile& t) {
    if (u >= u_end) return false;
    if (p.total_units <= 0x7fffffffLL) {
        // the usual case in 32-bit arithmetic: the 64-bit divisions below cost the one thread that issues the tensor-core
        // work about a thousand clocks between two tiles
        const uint32_t u32 = uint32_t(u), rows_total = uint32_t(p.N) * uint32_t(p.Ho);
        const uint32_t mt = u32 / rows_total, row = u32 - mt * rows_total;
        const uint32_t n = row / uint32_t(p.Ho), oh0 = row - n * uint32_t(p.Ho);
        t.m0 = int(mt) * 128;
        t.n = int(n);
        t.oh0 = int(oh0);
        uint32_t rem = uint32_t(p.Ho) - oh0;
        if (rem > uint32_t(u_end - u)) rem = uint32_t(u_end - u);
        const uint32_t rmax = uint32_t(p.r_max);
        const uint32_t nt = (rem + rmax - 1) / rmax;
        uint32_t r = (rem + nt - 1) / nt;
        if (p.even_rows && (r & 1u) && r < rem && r < rmax) r++;
        t.rows = int(r);
        u += r;
        return true;
    }
    const long long rows_total = (long long)p.N * p.Ho;
    const long long mt = u / rows_total;
    const long long row = u - mt * rows_total;
    t.m0 = int(mt) * 128;
    t.n = int(row / p.Ho);
    t.oh0 = int(row - (long long)t.n * p.Ho);
    // rows still to do in this image and range, cut into equal tiles of at most r_max rows
    long long rem = p.Ho - t.oh0;
    if (rem > u_end - u) rem = u_end - u;
    const long long nt = (rem + p.r_max - 1) / p.r_max;
    long long r = (rem + nt - 1) / nt;
    if (p.even_rows && (r & 1) && r < rem && r < p.r_max) r++;
    t.rows = int(r);
    u += r;
    return true;
}

__global__ void __launch_bounds__(kThreads, 1)
    conv_tc_kernel(const __grid_constant__ CUtensorMap tmW0, const __grid_constant__ CUtensorMap tmW1,
                   const __grid_constant__ CUtensorMap tmX0, const __grid_constant__ CUtensorMap tmX1,
                   const __grid_constant__ CUtensorMap tmY, const ConvKernelParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    const uint32_t sA = base;
    const uint32_t sB = sA + kStages * kABytes;
    const uint32_t sStage = sB + kStages * kBBytes;  // four 4 KB staging tiles (one per epilogue warp)
    const uint32_t bars = sStage + 4 * 4096u;
    auto full_bar = [&](int i) { return bars + 8u * uint32_t(i); };
    auto empty_bar = [&](int i) { return bars + 64u + 8u * uint32_t(i); };
    auto tfull_bar = [&](int i) { return bars + 128u + 8u * uint32_t(i); };
    auto tempty_bar = [&](int i) { return bars + 144u + 8u * uint32_t(i); };
    volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem_raw + (bars + 160u - raw_addr));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (warp == 0 && lane == 0) {
        for (int i = 0; i < kStages; i++) {
            mbar_init(full_bar(i), 1);
            mbar_init(empty_bar(i), 1);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(tfull_bar(i), 1);
            mbar_init(tempty_bar(i), 4);
        }
        fence_barrier_init();
        prefetch_tensormap(&tmW0);
        prefetch_tensormap(&tmX0);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_holder)), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_holder;

    const long long u_begin = p.total_units * blockIdx.x / gridDim.x;
    const long long u_end = p.total_units * (blockIdx.x + 1) / gridDim.x;
    const int cblocks = p.C / 64;
    const int kb_per_pass = p.kh * p.kw * cblocks;

    if (warp == 0) {
        // TMA producer. A single lane issues, so the k-block loop is a (tap row, tap column, channel block) nest with
        // an incrementally kept ring position: no division between two loads.
        if (lane == 0) {
            uint32_t s = 0, ph = 0;
            long long u = u_begin;
            Tile t;
            bool ok = true;
            const uint32_t row_bytes = uint32_t(p.Wo) * 128u;
            while (ok && next_tile(p, u, u_end, t)) {
                const uint32_t tx = kABytes + uint32_t(t.rows) * row_bytes;
                for (int pass = 0; pass < p.npass && ok; pass++) {
                    const CUtensorMap* mw = p.pw[pass] ? &tmW1 : &tmW0;
                    const CUtensorMap* mx = p.px[pass] ? &tmX1 : &tmX0;
                    int k_col = 0;  // column of this k-block in the re-laid weights: (tap * cblocks + cb) * 64
                    for (int ky = 0; ky < p.kh && ok; ky++) {
                        const int ih0 = t.oh0 + ky - p.pad_h;
                        for (int kx = 0; kx < p.kw && ok; kx++) {
                            const int iw0 = kx - p.pad_w;
                            for (int c0 = 0; c0 < p.C; c0 += 64, k_col += 64) {
                                const uint32_t full = full_bar(0) + 8u * s;
                                if (!mbar_wait(empty_bar(0) + 8u * s, ph ^ 1u)) {
                                    conv_timeout(p.status, 21);
                                    ok = false;
                                    break;
                                }
                                mbar_arrive_expect_tx(full, tx);
                                tma_load_2d(sA + s * kABytes, mw, full, k_col, t.m0);
                                uint32_t b_dst = sB + s * kBBytes;
                                for (int r = 0; r < t.rows; r++, b_dst += row_bytes) tma_load_4d(b_dst, mx, full, c0, iw0, ih0 + r, t.n);
                                if (++s == uint32_t(kStages)) {
                                    s = 0;
                                    ph ^= 1u;
                                }
                            }
                        }
                    }
                }
            }
            if (!ok) {
                const long long t0 = clock64();
                while (clock64() - t0 < 200000) {
                }
            }
        }
    } else if (warp == 1) {
        // UMMA issuer: descriptors advance by adds, four k-steps per asm block.
        if (lane == 0) {
            uint32_t lt = 0;
            long long u = u_begin;
            Tile t;
            bool ok = true;
            const int k_iters = p.npass * kb_per_pass;
            const uint64_t a_desc0 = make_smem_desc(sA, 16u, 1024u), b_desc0 = make_smem_desc(sB, 16u, 1024u);
            uint64_t a_desc = a_desc0, b_desc = b_desc0;
            uint32_t s = 0, ph = 0;
            while (ok && next_tile(p, u, u_end, t)) {
                const uint32_t buf = lt & 1u, use = lt >> 1;
                lt++;
                if (!mbar_wait(tempty_bar(int(buf)), (use & 1u) ^ 1u)) {
                    conv_timeout(p.status, 22);
                    break;
                }
                tc_fence_after();
                const int n_mma = (t.rows * p.Wo + 15) / 16 * 16;
                const uint32_t idesc = make_idesc(128, n_mma, 1, 0, 0);
                const uint32_t d_tmem = tmem_base + buf * 256u;
                uint32_t acc = 0;
                for (int k = 0; k < k_iters; k++) {
                    if (!mbar_wait(full_bar(0) + 8u * s, ph)) {
                        conv_timeout(p.status, 23);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    umma_f16_ss_x4<1>(d_tmem, a_desc, b_desc, idesc, acc, 2, 2);  // +32 bytes per 16-deep k-step
                    acc = 1;
                    umma_commit(empty_bar(0) + 8u * s);
                    a_desc += kABytes >> 4;
                    b_desc += kBBytes >> 4;
                    if (++s == uint32_t(kStages)) {
                        s = 0;
                        ph ^= 1u;
                        a_desc = a_desc0;
                        b_desc = b_desc0;
                    }
                }
                if (ok) umma_commit(tfull_bar(int(buf)));
            }
        }
    } else {
        const int q = warp & 3;
        uint32_t lt = 0;
        long long u = u_begin;
        Tile t;
        const long long plane = (long long)p.Ho * p.Wo;
        while (next_tile(p, u, u_end, t)) {
            const uint32_t buf = lt & 1u, use = lt >> 1;
            lt++;
            if (!mbar_wait(tfull_bar(int(buf)), use & 1u)) {
                if (lane == 0) conv_timeout(p.status, 24);
                break;
            }
            tc_fence_after();
            const int oc = t.m0 + q * 32 + lane;
            const int ncols = t.rows * p.Wo;
            const uint32_t t_addr = tmem_base + (uint32_t(q * 32) << 16) + buf * 256u;
            const bool row_ok = oc < p.c_out;
            const float bv = (row_ok && p.bias) ? __ldg(p.bias + oc) : 0.f;
            float* yrow = p.Y + ((long long)t.n * p.c_out + (row_ok ? oc : 0)) * plane + (long long)t.oh0 * p.Wo;
            const bool vec = (reinterpret_cast<uintptr_t>(yrow) & 15) == 0;
            const uint32_t stage_base = sStage + uint32_t(warp - 2) * 4096u;
            const int pix0 = t.oh0 * p.Wo;
            int c = 0;
            if (p.tma_out) {
                // whole 32-pixel groups leave through a swizzled staging tile and one TMA store per warp:
                // 32 channels x 32 pixels, every row a full 128-byte line of Y
                for (; c + 32 <= ncols; c += 32) {
                    if (lane == 0) tma_store_wait_read<0>();
                    __syncwarp();
#pragma unroll
                    for (int sub = 0; sub < 2; sub++) {
                        uint32_t r[16];
                        tmem_ld_x16(t_addr + uint32_t(c + sub * 16), r);
                        tmem_ld_wait();
#pragma unroll
                        for (int v4 = 0; v4 < 4; v4++) {
                            const int chunk = sub * 4 + v4;
                            const uint32_t dst = stage_base + uint32_t(lane) * 128u + uint32_t((chunk ^ (lane & 7)) * 16);
                            const uint32_t w0 = __float_as_uint(__uint_as_float(r[v4 * 4 + 0]) + bv);
                            const uint32_t w1 = __float_as_uint(__uint_as_float(r[v4 * 4 + 1]) + bv);
                            const uint32_t w2 = __float_as_uint(__uint_as_float(r[v4 * 4 + 2]) + bv);
                            const uint32_t w3 = __float_as_uint(__uint_as_float(r[v4 * 4 + 3]) + bv);
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w0), "r"(w1), "r"(w2), "r"(w3) : "memory");
                        }
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0 && t.m0 + q * 32 < p.c_out) {
                        tma_store_3d(&tmY, stage_base, pix0 + c, t.m0 + q * 32, t.n);  // channels >= C_out are clipped
                        tma_store_commit();
                    }
                }
            }
            for (; c < ncols; c += 16) {
                uint32_t r[16];
                tmem_ld_x16(t_addr + uint32_t(c), r);
                tmem_ld_wait();
                if (!row_ok) continue;
                if (vec && c + 16 <= ncols) {
#pragma unroll
                    for (int v4 = 0; v4 < 4; v4++) {
                        float4 o;
                        o.x = __uint_as_float(r[v4 * 4 + 0]) + bv;
                        o.y = __uint_as_float(r[v4 * 4 + 1]) + bv;
                        o.z = __uint_as_float(r[v4 * 4 + 2]) + bv;
                        o.w = __uint_as_float(r[v4 * 4 + 3]) + bv;
                        __stcs(reinterpret_cast<float4*>(yrow + c) + v4, o);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 16; j++)
                        if (c + j < ncols) yrow[c + j] = __uint_as_float(r[j]) + bv;
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(int(buf)));
        }
        if (p.tma_out && lane == 0) tma_store_wait<0>();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---- halo variant ---------------------------------------------------------------------------------
// For images at most 64 - kw + 1 output pixels wide, the tile's input neighbourhood is loaded once and all
// kh*kw taps read it in place. The halo of a tile of r output rows is (r + kh - 1) input rows of 64 pixel
// slots (input columns -pad_w .. 63 - pad_w; slots outside the image are zero-filled by TMA), 128 bytes of
// channels each: one 4-D TMA box per 64-channel block. The accumulator has 64 columns per output row
// (column = row * 64 + ow, the columns ow >= Wo hold garbage and are never stored); tap (ky, kx) is the
// same shared-memory tile read from a start address (ky * 64 + kx) * 128 bytes further on, which works
// because the 128-byte swizzle is a function of the absolute shared-memory address. Against the per-tap
// loads of the kernel above this cuts the L2 -> SM traffic of the input by kh*kw (weights still stream
// through their own ring, one 128 x 64 block per tap).
constexpr int kHaloSlots = 2;
constexpr int kMaxWStages = 8;  // the weight ring takes what the halo slots leave: its depth has to cover the TMA latency

constexpr int kHaloThreads = 320;  // TMA warp, UMMA warp, eight epilogue warps (two per tensor-memory lane quadrant)

__global__ void __launch_bounds__(kHaloThreads, 1)
    conv_halo_kernel(const __grid_constant__ CUtensorMap tmW0, const __grid_constant__ CUtensorMap tmW1,
                     const __grid_constant__ CUtensorMap tmX0, const __grid_constant__ CUtensorMap tmX1,
                     const __grid_constant__ CUtensorMap tmY, const ConvKernelParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    const uint32_t halo_bytes = uint32_t(p.r_max + p.kh - 1) * 8192u;
    const uint32_t w_stages = uint32_t(p.w_stages);
    const uint32_t n_slots = p.paired == 1 ? 3u : uint32_t(kHaloSlots);
    const uint32_t sH = base;                           // halo slots; reads past a slot's end land in the next region
    const uint32_t sA = sH + n_slots * halo_bytes;      // weight ring
    const uint32_t sStage = sA + w_stages * kABytes;    // eight 4 KB staging tiles (one per epilogue warp)
    const uint32_t bars = sStage + 8 * 4096u;
    auto full_a = [&](uint32_t i) { return bars + 8u * i; };
    auto empty_a = [&](uint32_t i) { return bars + 64u + 8u * i; };
    auto full_h = [&](uint32_t i) { return bars + 128u + 8u * i; };   // up to three halo slots
    auto empty_h = [&](uint32_t i) { return bars + 200u + 8u * i; };
    auto tfull_bar = [&](uint32_t i) { return bars + 160u + 8u * i; };
    auto tempty_bar = [&](uint32_t i) { return bars + 176u + 8u * i; };
    volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem_raw + (bars + 192u - raw_addr));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (warp == 0 && lane == 0) {
        for (uint32_t i = 0; i < w_stages; i++) {
            mbar_init(full_a(i), 1);
            mbar_init(empty_a(i), 1);
        }
        for (uint32_t i = 0; i < 3; i++) {
            mbar_init(full_h(i), 1);
            mbar_init(empty_h(i), 1);
        }
        for (uint32_t i = 0; i < 2; i++) {
            mbar_init(tfull_bar(i), 1);
            mbar_init(tempty_bar(i), 8);
        }
        fence_barrier_init();
        prefetch_tensormap(&tmW0);
        prefetch_tensormap(&tmX0);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_holder)), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_holder;
    // launched with programmatic stream serialization behind the re-layout launch: everything above overlaps its tail
    griddep_wait();
    griddep_launch_dependents();

    const long long u_begin = p.total_units * blockIdx.x / gridDim.x;
    const long long u_end = p.total_units * (blockIdx.x + 1) / gridDim.x;

    if (warp == 0) {
        // TMA producer: per (pass, channel block) one halo box, then the kh*kw weight blocks.
        if (lane == 0) {
            uint32_t s = 0, ph = 0, hs = 0, hph = 0;
            long long u = u_begin;
            Tile t;
            bool ok = true;
            while (ok && p.paired && next_tile(p, u, u_end, t)) {
                // Split operands, paired form: per channel block the high and the low plane of the input go into two
                // slots; the low weight plane runs over the high input, then every block of the high weight plane is
                // used for both input planes (18 weight blocks and two halo boxes per tile and channel block, not 27 and 3).
                for (int c0 = 0; c0 < p.C && ok; c0 += 64) {
                    for (int pl = 0; pl < 2 && ok; pl++) {
                        if (!mbar_wait(empty_h(hs), hph ^ 1u)) {
                            conv_timeout(p.status, 25);
                            ok = false;
                            break;
                        }
                        mbar_arrive_expect_tx(full_h(hs), halo_bytes);
                        tma_load_4d(sH + hs * halo_bytes, pl ? &tmX1 : &tmX0, full_h(hs), c0, -p.pad_w, t.oh0 - p.pad_h, t.n);
                        if (++hs == n_slots) {
                            hs = 0;
                            hph ^= 1u;
                        }
                    }
                    int k_col = c0;
                    for (int tap = 0; tap < p.kh * p.kw && ok; tap++, k_col += p.C) {
                        for (int wp = 1; wp >= 0; wp--) {  // per tap: the low weight plane's block, then the high one's
                            if (!mbar_wait(empty_a(s), ph ^ 1u)) {
                                conv_timeout(p.status, 21);
                                ok = false;
                                break;
                            }
                            mbar_arrive_expect_tx(full_a(s), kABytes);
                            tma_load_2d(sA + s * kABytes, wp ? &tmW1 : &tmW0, full_a(s), k_col, t.m0);
                            if (++s == w_stages) {
                                s = 0;
                                ph ^= 1u;
                            }
                        }
                    }
                }
            }
            while (ok && next_tile(p, u, u_end, t)) {
                for (int pass = 0; pass < p.npass && ok; pass++) {
                    const CUtensorMap* mw = p.pw[pass] ? &tmW1 : &tmW0;
                    const CUtensorMap* mx = p.px[pass] ? &tmX1 : &tmX0;
                    for (int c0 = 0; c0 < p.C && ok; c0 += 64) {
                        if (!mbar_wait(empty_h(hs), hph ^ 1u)) {
                            conv_timeout(p.status, 25);
                            ok = false;
                            break;
                        }
                        mbar_arrive_expect_tx(full_h(hs), halo_bytes);
                        tma_load_4d(sH + hs * halo_bytes, mx, full_h(hs), c0, -p.pad_w, t.oh0 - p.pad_h, t.n);
                        if (++hs == n_slots) {
                            hs = 0;
                            hph ^= 1u;
                        }
                        int k_col = c0;  // column of (tap, channel block) in the re-laid weights: tap * C + c0
                        for (int tap = 0; tap < p.kh * p.kw; tap++, k_col += p.C) {
                            if (!mbar_wait(empty_a(s), ph ^ 1u)) {
                                conv_timeout(p.status, 21);
                                ok = false;
                                break;
                            }
                            mbar_arrive_expect_tx(full_a(s), kABytes);
                            tma_load_2d(sA + s * kABytes, mw, full_a(s), k_col, t.m0);
                            if (++s == w_stages) {
                                s = 0;
                                ph ^= 1u;
                            }
                        }
                    }
                }
            }
            if (!ok) {
                const long long t0 = clock64();
                while (clock64() - t0 < 200000) {
                }
            }
        }
    } else if (warp == 1) {
        // UMMA issuer
        if (lane == 0) {
            uint32_t lt = 0;
            long long u = u_begin;
            Tile t;
            bool ok = true;
            const uint64_t a_desc0 = make_smem_desc(sA, 16u, 1024u), h_desc0 = make_smem_desc(sH, 16u, 1024u);
            const int cblocks = p.npass * (p.C / 64);
            uint32_t s = 0, ph = 0, hs = 0, hph = 0;
            uint64_t a_desc = a_desc0;
            while (ok && next_tile(p, u, u_end, t)) {
                const uint32_t buf = lt & 1u, use = lt >> 1;
                lt++;
                if (!mbar_wait(tempty_bar(buf), (use & 1u) ^ 1u)) {
                    conv_timeout(p.status, 22);
                    break;
                }
                tc_fence_after();
                const uint32_t idesc = make_idesc(128, t.rows * 64, 1, 0, 0);
                const uint32_t d_tmem = tmem_base + buf * 256u;
                uint32_t acc = 0;
                for (int cb = 0; p.paired && cb < p.C / 64 && ok; cb++) {
                    // slots: hs holds the high plane of the input, the one after it the low plane
                    const uint32_t hs_lo = hs + 1u == n_slots ? 0u : hs + 1u;
                    const uint32_t hph_lo = hs + 1u == n_slots ? hph ^ 1u : hph;
                    for (int wp = 1; wp >= 0 && ok; wp--) {
                        if (!mbar_wait(wp ? full_h(hs) : full_h(hs_lo), wp ? hph : hph_lo)) {
                            conv_timeout(p.status, 26);
                            ok = false;
                        }
                    }
                    if (!ok) break;
                    tc_fence_after();
                    uint64_t row_hi = h_desc0 + uint64_t(hs * (halo_bytes >> 4)), row_lo = h_desc0 + uint64_t(hs_lo * (halo_bytes >> 4));
                    for (int ky = 0; ky < p.kh && ok; ky++, row_hi += (64 * 128) >> 4, row_lo += (64 * 128) >> 4) {
                        uint64_t b_hi = row_hi, b_lo = row_lo;
                        for (int kx = 0; kx < p.kw && ok; kx++, b_hi += 128 >> 4, b_lo += 128 >> 4) {
                            for (int wp = 1; wp >= 0; wp--) {
                                if (!mbar_wait(full_a(s), ph)) {
                                    conv_timeout(p.status, 23);
                                    ok = false;
                                    break;
                                }
                                tc_fence_after();
                                if (wp) {
                                    umma_f16_ss_x4<1>(d_tmem, a_desc, b_hi, idesc, acc, 2, 2);  // W_lo * X_hi
                                } else {
                                    umma_f16_ss_x4<1>(d_tmem, a_desc, b_lo, idesc, 1u, 2, 2);   // W_hi * X_lo
                                    umma_f16_ss_x4<1>(d_tmem, a_desc, b_hi, idesc, 1u, 2, 2);   // W_hi * X_hi
                                }
                                acc = 1;
                                umma_commit(empty_a(s));
                                a_desc += kABytes >> 4;
                                if (++s == w_stages) {
                                    s = 0;
                                    ph ^= 1u;
                                    a_desc = a_desc0;
                                }
                            }
                        }
                    }
                    if (!ok) break;
                    umma_commit(empty_h(hs));
                    umma_commit(empty_h(hs_lo));
                    for (int i = 0; i < 2; i++) {
                        if (++hs == n_slots) {
                            hs = 0;
                            hph ^= 1u;
                        }
                    }
                }
                for (int cb = 0; !p.paired && cb < cblocks && ok; cb++) {
                    if (!mbar_wait(full_h(hs), hph)) {
                        conv_timeout(p.status, 26);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    uint64_t row_desc = h_desc0 + uint64_t(hs * (halo_bytes >> 4));
                    for (int ky = 0; ky < p.kh && ok; ky++, row_desc += (64 * 128) >> 4) {
                        uint64_t b_desc = row_desc;
                        for (int kx = 0; kx < p.kw; kx++, b_desc += 128 >> 4) {
                            if (!mbar_wait(full_a(s), ph)) {
                                conv_timeout(p.status, 23);
                                ok = false;
                                break;
                            }
                            tc_fence_after();
                            umma_f16_ss_x4<1>(d_tmem, a_desc, b_desc, idesc, acc, 2, 2);  // +32 bytes per 16-deep k-step
                            acc = 1;
                            umma_commit(empty_a(s));
                            a_desc += kABytes >> 4;
                            if (++s == w_stages) {
                                s = 0;
                                ph ^= 1u;
                                a_desc = a_desc0;
                            }
                        }
                    }
                    if (!ok) break;
                    umma_commit(empty_h(hs));
                    if (++hs == n_slots) {
                        hs = 0;
                        hph ^= 1u;
                    }
                }
                if (ok) umma_commit(tfull_bar(buf));
            }
        }
    } else {
        const int q = warp & 3;
        const int wg = (warp - 2) >> 2;
        uint32_t lt = 0;
        long long u = u_begin;
        Tile t;
        const long long plane = (long long)p.Ho * p.Wo;
        const uint32_t stage_base = sStage + uint32_t(warp - 2) * 4096u;
        while (next_tile(p, u, u_end, t)) {
            const uint32_t buf = lt & 1u, use = lt >> 1;
            lt++;
            if (!mbar_wait(tfull_bar(buf), use & 1u)) {
                if (lane == 0) conv_timeout(p.status, 24);
                break;
            }
            tc_fence_after();
            const int oc = t.m0 + q * 32 + lane;
            const uint32_t t_addr = tmem_base + (uint32_t(q * 32) << 16) + buf * 256u;
            const bool row_ok = oc < p.c_out;
            const float bv = (row_ok && p.bias) ? __ldg(p.bias + oc) : 0.f;
            // the two warps of a quadrant take alternate groups of 32 output pixels
            int gi = 0;
            for (int rr = 0; rr < t.rows; rr++) {
                float* yrow = p.Y + ((long long)t.n * p.c_out + (row_ok ? oc : 0)) * plane + (long long)(t.oh0 + rr) * p.Wo;
                for (int c = 0; c < p.Wo; c += 32, gi++) {
                    if ((gi & 1) != wg) continue;
                    const uint32_t col = uint32_t(rr * 64 + c);
                    if (p.tma_out) {
                        // a swizzled staging tile of 32 channels x 32 pixels and one TMA store per warp; the tensor map
                        // clips pixels >= Wo and channels >= C_out
                        uint32_t r0[16], r1[16];
                        tmem_ld_x16(t_addr + col, r0);
                        tmem_ld_x16(t_addr + col + 16u, r1);
                        if (lane == 0) tma_store_wait_read<0>();  // the previous store has finished reading the staging tile
                        tmem_ld_wait();
                        __syncwarp();
#pragma unroll
                        for (int sub = 0; sub < 2; sub++) {
                            const uint32_t (&r)[16] = sub ? r1 : r0;
#pragma unroll
                            for (int v4 = 0; v4 < 4; v4++) {
                                const int chunk = sub * 4 + v4;
                                const uint32_t dst = stage_base + uint32_t(lane) * 128u + uint32_t((chunk ^ (lane & 7)) * 16);
                                const uint32_t w0 = __float_as_uint(__uint_as_float(r[v4 * 4 + 0]) + bv);
                                const uint32_t w1 = __float_as_uint(__uint_as_float(r[v4 * 4 + 1]) + bv);
                                const uint32_t w2 = __float_as_uint(__uint_as_float(r[v4 * 4 + 2]) + bv);
                                const uint32_t w3 = __float_as_uint(__uint_as_float(r[v4 * 4 + 3]) + bv);
                                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w0), "r"(w1), "r"(w2), "r"(w3) : "memory");
                            }
                        }
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0 && t.m0 + q * 32 < p.c_out) {
                            tma_store_4d(&tmY, stage_base, c, t.oh0 + rr, t.m0 + q * 32, t.n);
                            tma_store_commit();
                        }
                    } else {
#pragma unroll
                        for (int sub = 0; sub < 2; sub++) {
                            uint32_t r[16];
                            tmem_ld_x16(t_addr + col + uint32_t(sub * 16), r);
                            tmem_ld_wait();
                            if (!row_ok) continue;
#pragma unroll
                            for (int j = 0; j < 16; j++)
                                if (c + sub * 16 + j < p.Wo) yrow[c + sub * 16 + j] = __uint_as_float(r[j]) + bv;
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(buf));
        }
        if (p.tma_out && lane == 0) tma_store_wait<0>();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---- layout pre-passes ---------------------------------------------------------------------------
template <typename TIn> __device__ __forceinline__ float ld_f(const TIn* p) { return to_float(*p); }

// W [oc][c][taps] -> hi (and lo) [oc][taps][c]; `part` of `parts` cooperating blocks
template <typename TIn, bool SPLIT>
__device__ __forceinline__ void weight_relayout(const TIn* __restrict__ Wt, __nv_bfloat16* __restrict__ hi, __nv_bfloat16* __restrict__ lo,
                                                int c_out, int C, int taps, long long part, long long parts) {
    const long long total = (long long)c_out * C * taps;
    for (long long i = part * blockDim.x + threadIdx.x; i < total; i += parts * blockDim.x) {
        const int c = int(i % C);
        const int tap = int((i / C) % taps);
        const long long oc = i / ((long long)C * taps);
        const float v = ld_f(Wt + (oc * C + c) * taps + tap);
        const __nv_bfloat16 h = __float2bfloat16_rn(v);
        hi[i] = h;
        if (SPLIT) lo[i] = __float2bfloat16_rn(v - __bfloat162float(h));
    }
}

// ---- fused variant: 16-bit NCHW input read in place ----------------------------------------------------
// Same tiling, tap addressing, weight ring and epilogue as conv_halo_kernel, but the input never takes a trip through an
// NHWC copy in HBM. NCHW keeps the pixels of one channel contiguous, whereas the tensor cores want, per pixel slot,
// the 64 channels of a block contiguous (K-major rows of 128 bytes, 128-byte swizzle). A one-pixel tap shift is 2
// bytes in NCHW, below the 16-byte granularity of TMA coordinates and shared-memory descriptors alike, so neither
// can do the transposition. It happens between two shared-memory buffers instead:
//   * a producer warp brings one input row of a 64-channel block at a time, [64 channels][64 pixels] (8 KB, 128-byte
//     swizzle), through a ring of staging chunks by TMA. The box starts 8 pixels left of the image when there is left
//     padding (x coordinate -8: 16 bytes, the TMA alignment rule); rows above / below the image and columns outside
//     it are zero-filled by TMA, which is the convolution's zero padding;
//   * four transposer warps move each chunk into the tile's halo slot with ldmatrix.trans / stmatrix: four 8x8 blocks
//     [8 channels][8 pixels] come out as [8 pixels][8 channels], and every 16-byte row is stored at the swizzled
//     position of its pixel slot (slot = staging pixel - 8 + pad_w). Both sides are bank-conflict free because both
//     layouts are 128-byte swizzled. Slots the box does not reach (the right padding) are written as zeros.
// Plain per-thread global loads were measured first (8 warps x 24-48 loads of 4 bytes in flight): the SM's load path
// could not keep enough of them outstanding, a tile's input took 8k clocks against 6k for its tensor-core work.
// The halo slots are double buffered: tile i+1 is assembled while the tensor core works on tile i.
// The weights come from the small re-laid copy ([oc][tap][c], written by conv_weights_kernel just before); this
// kernel is launched with programmatic stream serialization and only its weight producer waits for that copy
// (griddepcontrol.wait), so set-up, tensor-memory allocation and the first input rows overlap it.
// Requirements (checked by the host): 16-bit input, W % 8 == 0, X 16-byte aligned, Wo + kw - 1 <= 64,
// pad_w <= 8 and W <= 56, or pad_w == 0 and W <= 64.
// Warps: 0 weight producer, 1 UMMA issuer, 2-9 epilogue, 10-13 transposers, 14 input producer.
//
// WRES (3x3 filters, one channel block, at most 128 output channels): the weights stay on the SM for the whole kernel.
// Streaming them costs every tile nine 16 KB blocks through a ring that shared memory keeps four deep, over an L2 latency
// of about 3 k clocks: 6.8 k clocks per tile whatever its height (measured), a third of the kernel at three tiles per
// CTA. Here taps 0-7 live in tensor-memory columns 0-255 (lane = output channel, one column = two consecutive channels;
// A operand of tcgen05.mma taken from tensor memory) and tap 8 in a 16 KB shared-memory block (A from shared memory);
// columns 256-511 hold two accumulators of two output rows each ([128 oc] x [2 x 64 pixel slots]). The weights are taken
// as the caller holds them, [oc][c][3][3]: no re-laid copy, no launch before this one. At start-up the weight producer
// brings every output channel's 1152-byte row in eight pieces of 144 bytes (eight channels x nine taps; one TMA box of
// [128 oc][72 elements], unswizzled: the 144-byte pitch keeps a quarter warp's 16-byte reads on different banks) through
// a three-stage ring that borrows the epilogue's staging tiles (unused until the first accumulator is full) and halo
// slot 1 (unused until the second tile is assembled); warps 2-5 (thread = output channel) pick, for every tap, the eight
// channels out of their 144 bytes with byte permutes and store them as four tensor-memory columns (taps 0-7) or as
// one 16-byte chunk of the shared-memory block in the UMMA's swizzled K-major layout (tap 8).
constexpr int kFusedThreads = 480;
constexpr uint32_t kTileList = 8;  // tiles of a CTA worked out once, ahead of the roles that walk them
constexpr uint32_t kResAccCol = 256;  // first accumulator column of the resident-weights variant
constexpr uint32_t kResTmemTaps = 8;  // taps held in tensor memory; the ninth stays in shared memory
constexpr uint32_t kResPieceBytes = 128 * 144;  // one start-up piece: eight channels x nine taps of 128 output channels

// Four consecutive 16-deep k-steps of D[tmem] (+)= A[tmem] * B[smem]: A advances by 8 columns, B by `b_step`.
__device__ __forceinline__ void umma_f16_ts_x4(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate,
                                               uint64_t b_step) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        ".reg .b64 rb;\n"
        ".reg .b32 ra;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "setp.ne.b32 p, %3, 0;\n"  // the instruction descriptor is never zero: p = true
        "add.u32 ra, %1, 8;\n"
        "add.s64 rb, %2, %5;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [ra], rb, %3, p;\n"
        "add.u32 ra, ra, 8;\n"
        "add.s64 rb, rb, %5;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [ra], rb, %3, p;\n"
        "add.u32 ra, ra, 8;\n"
        "add.s64 rb, rb, %5;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [ra], rb, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "l"(b_step)
        : "memory");
}
constexpr uint32_t kChunkBytes = 64 * 64 * 2;  // one input row of a channel block

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr)
                 : "memory");
}
__device__ __forceinline__ void stmatrix_x4(uint32_t addr, const uint32_t (&r)[4]) {
    asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3])
                 : "memory");
}

template <bool IS_BF16, bool WRES>
__global__ void __launch_bounds__(kFusedThreads, 1)
    conv_nchw_kernel(const __grid_constant__ CUtensorMap tmW0, const __grid_constant__ CUtensorMap tmX,
                     const __grid_constant__ CUtensorMap tmY, const ConvKernelParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    const uint32_t halo_rows_max = uint32_t(p.r_max + p.kh - 1);
    const uint32_t halo_bytes = halo_rows_max * 8192u;
    const uint32_t w_stages = uint32_t(p.w_stages);
    const uint32_t n_chunks = uint32_t(p.x_chunks);
    const uint32_t sH = base;                           // halo slots; reads past a slot's end land in the next region
    const uint32_t sA = sH + kHaloSlots * halo_bytes;   // weight ring
    const uint32_t sX = sA + w_stages * kABytes;        // staging chunks of the input producer
    const uint32_t sStage = sX + n_chunks * kChunkBytes;  // eight 4 KB staging tiles (one per epilogue warp)
    const uint32_t sDummy = sStage + 8 * 4096u;         // 512 bytes: target of stmatrix rows that belong to no slot
    const uint32_t bars = sDummy + 512u;
    auto full_a = [&](uint32_t i) { return bars + 8u * i; };
    auto empty_a = [&](uint32_t i) { return bars + 64u + 8u * i; };
    auto full_h = [&](uint32_t i) { return bars + 128u + 8u * i; };
    auto empty_h = [&](uint32_t i) { return bars + 144u + 8u * i; };
    auto tfull_bar = [&](uint32_t i) { return bars + 160u + 8u * i; };
    auto tempty_bar = [&](uint32_t i) { return bars + 176u + 8u * i; };
    auto full_x = [&](uint32_t i) { return bars + 192u + 8u * i; };
    auto empty_x = [&](uint32_t i) { return bars + 256u + 8u * i; };
    // WRES: channels 16k..16k+15 of every tap are where the tensor core reads them (one arrival per loading warp); the
    // last of the four is also the sign that all weights are in place
    auto wres_k = [&](uint32_t k) { return bars + 96u + 8u * k; };
    const uint32_t wres_bar = wres_k(3);
    // WRES: a slot's halo rows 0-3 are assembled (what the tile's first two output rows read; one arrival per transposer warp)
    auto part_h = [&](uint32_t i) { return bars + 32u + 8u * i; };
    // WRES start-up ring: the epilogue's staging tiles (two blocks of 16 KB, unused until the first accumulator is full)
    // and as much of halo slot 1 as holds whole blocks (unused until the second tile is assembled; the transposers wait
    // for wres_bar before they write there)
    const uint32_t res_stages = 1u + (halo_bytes / kResPieceBytes < 2u ? halo_bytes / kResPieceBytes : 2u);
    auto res_stage_addr = [&](uint32_t i) { return i < 1u ? sStage : sH + halo_bytes + (i - 1u) * kResPieceBytes; };
    volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem_raw + (bars + 320u - raw_addr));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (warp == 0 && lane == 0) {
        if constexpr (WRES) {
            // start-up ring (full_a / empty_a 0..2: four loading warps release a stage)
            for (uint32_t i = 0; i < res_stages; i++) {
                mbar_init(full_a(i), 1);
                mbar_init(empty_a(i), 4);
            }
            for (uint32_t k = 0; k < 4; k++) mbar_init(wres_k(k), 4);
            for (uint32_t i = 0; i < 2; i++) mbar_init(part_h(i), 4);
        } else {
            for (uint32_t i = 0; i < w_stages; i++) {
                mbar_init(full_a(i), 1);
                mbar_init(empty_a(i), 1);
            }
        }
        for (uint32_t i = 0; i < 2; i++) {
            mbar_init(full_h(i), 4);  // one arrival per transposer warp
            mbar_init(empty_h(i), 1);
            mbar_init(tfull_bar(i), 1);
            mbar_init(tempty_bar(i), 8);
        }
        fence_barrier_init();
        prefetch_tensormap(&tmW0);
        prefetch_tensormap(&tmY);
        if constexpr (WRES) {
            // the first pieces of the weights go out before the block-wide synchronisation (the stages are free)
            griddep_wait();
            for (uint32_t st = 0; st < res_stages; st++) {
                mbar_arrive_expect_tx(full_a(st), kResPieceBytes);
                tma_load_2d(res_stage_addr(st), &tmW0, full_a(st), int(st) * 72, 0);
            }
        }
    }
    const long long u_begin = p.total_units * blockIdx.x / gridDim.x;
    const long long u_end = p.total_units * (blockIdx.x + 1) / gridDim.x;
    const int cblocks = p.C / 64;
    const int x0 = p.pad_w > 0 ? -8 : 0;  // first input column of a staging chunk
    // The CTA's first tiles, worked out once by a thread with nothing else to do before the synchronisation. Cutting the
    // range into tiles takes integer divisions, several hundred clocks on one thread, which the roles below would each
    // spend between two tiles: the thread that issues the tensor-core work on the critical path.
    const uint32_t tile_list = bars + 400u;
    volatile uint32_t* list_count = reinterpret_cast<volatile uint32_t*>(smem_raw + (bars + 384u - raw_addr));
    volatile long long* list_after = reinterpret_cast<volatile long long*>(smem_raw + (bars + 392u - raw_addr));
    if (warp == 2 && lane == 0) {
        long long u = u_begin;
        Tile t;
        uint32_t n = 0;
        while (n < kTileList && next_tile(p, u, u_end, t)) {
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(tile_list + 16u * n), "r"(t.m0), "r"(t.n), "r"(t.oh0), "r"(t.rows) : "memory");
            n++;
        }
        *list_count = n;
        *list_after = u;
    }
    // The input producer owns the barriers of its ring and fills the ring before the block-wide synchronisation: the
    // first rows (a trip to HBM) are then in flight while tensor memory is allocated and the other barriers are set up.
    uint32_t x_early = 0;
    if (warp == 14 && lane == 0) {
        for (uint32_t i = 0; i < n_chunks; i++) {
            mbar_init(full_x(i), 1);
            mbar_init(empty_x(i), 4);  // one arrival per transposer warp
        }
        fence_barrier_init();
        prefetch_tensormap(&tmX);
        // resident weights: the kernel is launched with programmatic stream serialization behind whatever ran before
        // (nothing of ours precedes it), so every first touch of global memory waits for that launch to have completed
        if constexpr (WRES) griddep_wait();
        long long u = u_begin;
        Tile t;
        if (next_tile(p, u, u_end, t)) {
            const uint32_t hrows = uint32_t(t.rows + p.kh - 1);
            x_early = hrows < n_chunks ? hrows : n_chunks;
            for (uint32_t i = 0; i < x_early; i++) {
                mbar_arrive_expect_tx(full_x(i), kChunkBytes);
                tma_load_4d(sX + i * kChunkBytes, &tmX, full_x(i), x0, t.oh0 - p.pad_h + int(i), 0, t.n);
            }
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
    const uint32_t n_list = *list_count;
    const long long u_after = *list_after;
    // tile number i of this CTA: from the list while it lasts, then cut from the rest of the range (cursor u)
    auto tile_at = [&](uint32_t& i, long long& u, Tile& t) -> bool {
        if (i < n_list) {
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(t.m0), "=r"(t.n), "=r"(t.oh0), "=r"(t.rows) : "r"(tile_list + 16u * i) : "memory");
            i++;
            return true;
        }
        return next_tile(p, u, u_end, t);
    };
    if constexpr (WRES) {
        // barrier set-up, tensor-memory allocation and descriptor prefetch above overlap the tail of the launch before;
        // the launch after this one may begin its own set-up as soon as SMs free up
        griddep_wait();
        griddep_launch_dependents();
    }

    if (warp == 0) {
        // weight producer: kh*kw blocks of 128 x 64 per (tile, channel block)
        if (WRES && lane == 0) {
            // once: the eight 144-byte pieces of every output channel's row through the borrowed stages
            uint32_t st = 0, use = 1;
            for (uint32_t piece = res_stages; piece < 8; piece++) {
                if (!mbar_wait(empty_a(st), (use & 1u) ^ 1u)) {
                    conv_timeout(p.status, 31);
                    break;
                }
                mbar_arrive_expect_tx(full_a(st), kResPieceBytes);
                tma_load_2d(res_stage_addr(st), &tmW0, full_a(st), int(piece) * 72, 0);
                if (++st == res_stages) {
                    st = 0;
                    use++;
                }
            }
        } else if (lane == 0) {
            griddep_wait();  // the re-laid weights come from the launch before this one
            uint32_t s = 0, ph = 0;
            long long u = u_begin;
            Tile t;
            bool ok = true;
            while (ok && next_tile(p, u, u_end, t)) {
                for (int c0 = 0; c0 < p.C && ok; c0 += 64) {
                    int k_col = c0;  // column of (tap, channel block) in the re-laid weights: tap * C + c0
                    for (int tap = 0; tap < p.kh * p.kw; tap++, k_col += p.C) {
                        if (!mbar_wait(empty_a(s), ph ^ 1u)) {
                            conv_timeout(p.status, 31);
                            ok = false;
                            break;
                        }
                        mbar_arrive_expect_tx(full_a(s), kABytes);
                        tma_load_2d(sA + s * kABytes, &tmW0, full_a(s), k_col, t.m0);
                        if (++s == w_stages) {
                            s = 0;
                            ph ^= 1u;
                        }
                    }
                }
            }
            if (!ok) {
                const long long t0 = clock64();
                while (clock64() - t0 < 200000) {
                }
            }
        }
    } else if (warp == 14) {
        // input producer: one staging chunk per halo row and channel block
        if (lane == 0) {
            uint32_t s = 0, ph = 0;
            long long u = u_begin;
            Tile t;
            bool ok = true;
            while (ok && next_tile(p, u, u_end, t)) {
                const int hrows = t.rows + p.kh - 1;
                for (int c0 = 0; c0 < p.C && ok; c0 += 64) {
                    for (int hr = 0; hr < hrows; hr++) {
                        if (x_early > 0) {
                            x_early--;  // issued before the block-wide synchronisation
                        } else {
                            if (!mbar_wait(empty_x(s), ph ^ 1u)) {
                                conv_timeout(p.status, 37);
                                ok = false;
                                break;
                            }
                            mbar_arrive_expect_tx(full_x(s), kChunkBytes);
                            tma_load_4d(sX + s * kChunkBytes, &tmX, full_x(s), x0, t.oh0 - p.pad_h + hr, c0, t.n);
                        }
                        if (++s == n_chunks) {
                            s = 0;
                            ph ^= 1u;
                        }
                    }
                }
            }
            if (!ok) {
                const long long t0 = clock64();
                while (clock64() - t0 < 200000) {
                }
            }
        }
    } else if (warp == 1) {
        // UMMA issuer
        if (lane == 0) {
            uint32_t lt = 0;
            long long u = u_begin;
            Tile t;
            bool ok = true;
            const uint64_t a_desc0 = make_smem_desc(sA, 16u, 1024u), h_desc0 = make_smem_desc(sH, 16u, 1024u);
            uint32_t s = 0, ph = 0, hs = 0, hph = 0;
            uint64_t a_desc = a_desc0;
            if constexpr (WRES) {
                uint32_t abuf = 0, aph = 0;
                bool first = true;
                uint32_t li = 0;
                long long ul = u_after;
                while (ok && tile_at(li, ul, t)) {
                    // a tile's first two output rows start as soon as the four halo rows they read are there
                    if (!mbar_wait(part_h(hs), hph)) {
                        conv_timeout(p.status, 36);
                        break;
                    }
                    tc_fence_after();
                    const uint64_t slot_desc = h_desc0 + uint64_t(hs * (halo_bytes >> 4));
                    if (first) {
                        // The first two output rows chase the weights: 16 channels of all nine taps at a time, as the
                        // loading warps hand them over. (Their accumulator is free: nothing has used it.)
                        const uint32_t idesc = make_idesc(128, t.rows >= 2 ? 128 : 64, 1, 0, 0);
                        const uint32_t d_tmem = tmem_base + kResAccCol;
                        for (uint32_t k = 0; k < 4 && ok; k++) {
                            if (!mbar_wait(wres_k(k), 0)) {
                                conv_timeout(p.status, 39);
                                ok = false;
                                break;
                            }
                            tc_fence_after();
#pragma unroll
                            for (int tap = 0; tap < int(kResTmemTaps); tap++)
                                umma_f16_ts(d_tmem, tmem_base + uint32_t(tap) * 32u + k * 8u,
                                            slot_desc + uint64_t(((tap / 3) * 64 + tap % 3) * 8) + uint64_t(k * 2u), idesc, (k | uint32_t(tap)) ? 1u : 0u);
                            umma_f16_ss(d_tmem, a_desc0 + uint64_t(k * 2u), slot_desc + uint64_t((2 * 64 + 2) * 8) + uint64_t(k * 2u), idesc, 1u);
                        }
                        if (!ok) break;
                        umma_commit(tfull_bar(0));
                        abuf = 1;
                    }
                    for (int rr = first ? 2 : 0; rr < t.rows && ok; rr += 2) {
                        if (rr == 2) {  // the rest of the tile reads all of its halo rows
                            if (!mbar_wait(full_h(hs), hph)) {
                                conv_timeout(p.status, 36);
                                ok = false;
                                break;
                            }
                            tc_fence_after();
                        }
                        if (!mbar_wait(tempty_bar(abuf), aph ^ 1u)) {
                            conv_timeout(p.status, 32);
                            ok = false;
                            break;
                        }
                        tc_fence_after();
                        // two output rows per accumulator (one for the last row of an odd tile): 128 or 64 pixel slots
                        const uint32_t idesc = make_idesc(128, (t.rows - rr >= 2) ? 128 : 64, 1, 0, 0);
                        const uint32_t d_tmem = tmem_base + kResAccCol + abuf * 128u;
                        const uint64_t row_desc = slot_desc + uint64_t(rr) * ((64 * 128) >> 4);
#pragma unroll
                        for (int tap = 0; tap < int(kResTmemTaps); tap++)
                            umma_f16_ts_x4(d_tmem, tmem_base + uint32_t(tap) * 32u, row_desc + uint64_t(((tap / 3) * 64 + tap % 3) * 8), idesc,
                                           tap ? 1u : 0u, 2);
                        umma_f16_ss_x4<1>(d_tmem, a_desc0, row_desc + uint64_t((2 * 64 + 2) * 8), idesc, 1u, 2, 2);
                        umma_commit(tfull_bar(abuf));
                        if (++abuf == 2u) {
                            abuf = 0;
                            aph ^= 1u;
                        }
                    }
                    if (!ok) break;
                    first = false;
                    umma_commit(empty_h(hs));
                    if (++hs == uint32_t(kHaloSlots)) {
                        hs = 0;
                        hph ^= 1u;
                    }
                }
                ok = false;  // done: the streamed-weights loop below is not for this variant
            }
            while (ok && next_tile(p, u, u_end, t)) {
                const uint32_t buf = lt & 1u, use = lt >> 1;
                lt++;
                if (!mbar_wait(tempty_bar(buf), (use & 1u) ^ 1u)) {
                    conv_timeout(p.status, 32);
                    break;
                }
                tc_fence_after();
                const uint32_t idesc = make_idesc(128, t.rows * 64, 1, 0, 0);
                const uint32_t d_tmem = tmem_base + buf * 256u;
                uint32_t acc = 0;
                for (int cb = 0; cb < cblocks && ok; cb++) {
                    if (!mbar_wait(full_h(hs), hph)) {
                        conv_timeout(p.status, 36);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    uint64_t row_desc = h_desc0 + uint64_t(hs * (halo_bytes >> 4));
                    for (int ky = 0; ky < p.kh && ok; ky++, row_desc += (64 * 128) >> 4) {
                        uint64_t b_desc = row_desc;
                        for (int kx = 0; kx < p.kw; kx++, b_desc += 128 >> 4) {
                            if (!mbar_wait(full_a(s), ph)) {
                                conv_timeout(p.status, 33);
                                ok = false;
                                break;
                            }
                            tc_fence_after();
                            umma_f16_ss_x4<1>(d_tmem, a_desc, b_desc, idesc, acc, 2, 2);  // +32 bytes per 16-deep k-step
                            acc = 1;
                            umma_commit(empty_a(s));
                            a_desc += kABytes >> 4;
                            if (++s == w_stages) {
                                s = 0;
                                ph ^= 1u;
                                a_desc = a_desc0;
                            }
                        }
                    }
                    if (!ok) break;
                    umma_commit(empty_h(hs));
                    if (++hs == uint32_t(kHaloSlots)) {
                        hs = 0;
                        hph ^= 1u;
                    }
                }
                if (ok) umma_commit(tfull_bar(buf));
            }
        }
    } else if (warp >= 10) {
        // transposers: staging chunk [channel][pixel] -> halo slot rows [pixel slot][channel]
        const int tw = warp - 10;
        const int m = lane >> 3, r = lane & 7;  // this lane supplies row r of 8x8 block m to ldmatrix / stmatrix
        const int shift = p.pad_w + x0;         // slot = staging pixel + shift (<= 0)
        uint32_t xs = 0, xph = 0, hs = 0, hph = 0;
        long long u = u_after;
        uint32_t li = 0;
        Tile t;
        bool ok = true;
        bool wres_seen = false;
        while (ok && tile_at(li, u, t)) {
            const int hrows = t.rows + p.kh - 1;
            for (int c0 = 0; c0 < p.C && ok; c0 += 64) {
                if (!mbar_wait(empty_h(hs), hph ^ 1u)) {
                    if (lane == 0) conv_timeout(p.status, 35);
                    ok = false;
                    break;
                }
                const uint32_t slot = sH + hs * halo_bytes;
                if constexpr (WRES) {
                    // halo slot 1 lends its room to the start-up weight ring: not before the weights are in tensor memory
                    if (hs == 1u && !wres_seen) {
                        if (!mbar_wait(wres_bar, 0)) {
                            if (lane == 0) conv_timeout(p.status, 41);
                            ok = false;
                            break;
                        }
                        wres_seen = true;
                    }
                }
                for (int hr = 0; hr < hrows; hr++) {
                    if (!mbar_wait(full_x(xs), xph)) {
                        if (lane == 0) conv_timeout(p.status, 38);
                        ok = false;
                        break;
                    }
                    const uint32_t chunk = sX + xs * kChunkBytes;
                    // 16 units of (8 pixels x 32 channels) per chunk, four per warp: unit = (pixel group g, channel half hf)
#pragma unroll
                    for (int it = 0; it < 4; it++) {
                        const int unit = tw * 4 + it;
                        const int g = unit >> 1, hf = unit & 1;
                        const int ch = hf * 32 + m * 8 + r;  // source row: a channel of the block
                        uint32_t v[4];
                        ldmatrix_x4_trans(chunk + uint32_t(ch) * 128u + (uint32_t(g ^ (ch & 7)) << 4), v);
                        if constexpr (!IS_BF16) {  // fp16 input: the tensor cores run in the bf16 format of the re-laid weights
#pragma unroll
                            for (int i = 0; i < 4; i++) {
                                const __half2 hv = *reinterpret_cast<const __half2*>(&v[i]);
                                const __nv_bfloat162 bv = __float22bfloat162_rn(__half22float2(hv));
                                v[i] = *reinterpret_cast<const uint32_t*>(&bv);
                            }
                        }
                        // destination row: pixel slot of staging pixel 8g + r; 16-byte chunk = channel group hf*4 + m
                        const int sl = g * 8 + r + shift;
                        const uint32_t row = uint32_t(hr * 64 + sl);
                        const uint32_t dst = sl >= 0 ? slot + row * 128u + ((uint32_t(hf * 4 + m) ^ (row & 7u)) << 4) : sDummy + uint32_t(lane) * 16u;
                        stmatrix_x4(dst, v);
                    }
                    // slots right of what the box reaches (staging pixel 64 and up) hold zeros: the right padding
                    for (int i = tw * 32 + lane; i < -shift * 8; i += 128) {
                        const uint32_t row = uint32_t(hr * 64 + 64 + shift + (i >> 3));
                        const uint32_t dst = slot + row * 128u + ((uint32_t(i & 7) ^ (row & 7u)) << 4);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0u) : "memory");
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(empty_x(xs));  // this warp has read its part of the chunk
                    if constexpr (WRES) {
                        if (hr == (hrows > 4 ? 3 : hrows - 1)) {  // what the tile's first two output rows read is in place
                            fence_proxy_async_smem();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(part_h(hs));
                        }
                    }
                    if (++xs == n_chunks) {
                        xs = 0;
                        xph ^= 1u;
                    }
                }
                if (!ok) break;
                fence_proxy_async_smem();  // the tensor core reads these generic-proxy stores through the async proxy
                __syncwarp();
                if (lane == 0) mbar_arrive(full_h(hs));
                if (++hs == uint32_t(kHaloSlots)) {
                    hs = 0;
                    hph ^= 1u;
                }
            }
        }
    } else {
        const int q = warp & 3;
        const int wg = (warp - 2) >> 2;
        uint32_t lt = 0;
        long long u = u_begin;
        Tile t;
        const long long plane = (long long)p.Ho * p.Wo;
        const uint32_t stage_base = sStage + uint32_t(warp - 2) * 4096u;
        if constexpr (WRES) {
            // warps 2-5 (one per lane quadrant): thread = output channel. A piece holds channels 8g..8g+7 of all nine taps
            // as 72 consecutive elements (element = channel * 9 + tap); channels 2j and 2j+1 of a tap are elements 18j + tap
            // and 18j + 9 + tap of the piece.
            if (wg == 0) {
                const uint32_t row = uint32_t(q * 32 + lane);
                const uint32_t w_taddr = tmem_base + (uint32_t(q * 32) << 16);
                bool wok = true;
                uint32_t st = 0, use = 0;
#pragma unroll 1
                for (uint32_t piece = 0; piece < 8 && wok; piece++) {
                    if (!mbar_wait(full_a(st), use & 1u)) {
                        if (lane == 0) conv_timeout(p.status, 40);
                        wok = false;
                        break;
                    }
                    uint32_t win[36];
                    const uint32_t rbase = res_stage_addr(st) + row * 144u;
#pragma unroll
                    for (uint32_t i = 0; i < 9; i++) {
                        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                                     : "=r"(win[4 * i + 0]), "=r"(win[4 * i + 1]), "=r"(win[4 * i + 2]), "=r"(win[4 * i + 3])
                                     : "r"(rbase + i * 16u)
                                     : "memory");
                    }
#pragma unroll
                    for (int tap = 0; tap < 9; tap++) {
                        uint32_t col[4];
#pragma unroll
                        for (int jj = 0; jj < 4; jj++) {
                            const int e0 = 18 * jj + tap, e1 = e0 + 9;
                            const uint32_t sel = ((e0 & 1) ? 0x0032u : 0x0010u) | ((e1 & 1) ? 0x7600u : 0x5400u);
                            uint32_t pair = __byte_perm(win[e0 >> 1], win[e1 >> 1], sel);
                            if constexpr (!IS_BF16) {  // fp16 weights: the tensor cores run in bf16 (as the transposers convert the input)
                                const __nv_bfloat162 bv = __float22bfloat162_rn(__half22float2(*reinterpret_cast<const __half2*>(&pair)));
                                pair = *reinterpret_cast<const uint32_t*>(&bv);
                            }
                            col[jj] = pair;
                        }
                        if (tap < int(kResTmemTaps)) {
                            tmem_st_x4(w_taddr + uint32_t(tap) * 32u + piece * 4u, col);
                        } else {
                            // tap 8: chunk `piece` of this channel's row in the block the UMMA reads (128-byte rows, 128-byte swizzle)
                            const uint32_t dst = sA + row * 128u + ((piece ^ (row & 7u)) << 4);
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(col[0]), "r"(col[1]), "r"(col[2]), "r"(col[3])
                                         : "memory");
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(empty_a(st));  // the rows of this stage have been consumed: the producer may refill it
                    if (++st == res_stages) {
                        st = 0;
                        use++;
                    }
                    if (piece & 1u) {  // 16 channels of every tap are complete: the tensor core may use them
                        tmem_st_wait();
                        fence_proxy_async_smem();  // tap 8's block was written with generic stores; the tensor core reads it through the async proxy
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(wres_k(piece >> 1));
                    }
                }
            }
        }
        uint32_t abuf = 0, aph = 0;  // WRES: accumulator of the current pair of output rows
        bool alive = true;
        uint32_t li = 0;
        u = u_after;
        while (alive && tile_at(li, u, t)) {
            const uint32_t buf = lt & 1u, use = lt >> 1;
            lt++;
            if constexpr (!WRES) {
                if (!mbar_wait(tfull_bar(buf), use & 1u)) {
                    if (lane == 0) conv_timeout(p.status, 34);
                    break;
                }
                tc_fence_after();
            }
            const int oc = t.m0 + q * 32 + lane;
            uint32_t t_addr = tmem_base + (uint32_t(q * 32) << 16) + buf * 256u;
            const bool row_ok = oc < p.c_out;
            const float bv = (row_ok && p.bias) ? __ldg(p.bias + oc) : 0.f;
            // the two warps of a quadrant take alternate groups of 32 output pixels
            int gi = 0;
            for (int rr = 0; rr < t.rows; rr++) {
                if constexpr (WRES) {
                    if ((rr & 1) == 0) {  // a new accumulator every two rows
                        if (!mbar_wait(tfull_bar(abuf), aph)) {
                            if (lane == 0) conv_timeout(p.status, 34);
                            alive = false;
                            break;
                        }
                        tc_fence_after();
                        t_addr = tmem_base + (uint32_t(q * 32) << 16) + kResAccCol + abuf * 128u;
                    }
                }
                float* yrow = p.Y + ((long long)t.n * p.c_out + (row_ok ? oc : 0)) * plane + (long long)(t.oh0 + rr) * p.Wo;
                for (int c = 0; c < p.Wo; c += 32, gi++) {
                    if ((gi & 1) != wg) continue;
                    const uint32_t col = WRES ? uint32_t((rr & 1) * 64 + c) : uint32_t(rr * 64 + c);
                    if (p.tma_out) {
                        uint32_t r0[16], r1[16];
                        tmem_ld_x16(t_addr + col, r0);
                        tmem_ld_x16(t_addr + col + 16u, r1);
                        if (lane == 0) tma_store_wait_read<0>();  // the previous store has finished reading the staging tile
                        tmem_ld_wait();
                        __syncwarp();
#pragma unroll
                        for (int sub = 0; sub < 2; sub++) {
                            const uint32_t (&r)[16] = sub ? r1 : r0;
#pragma unroll
                            for (int v4 = 0; v4 < 4; v4++) {
                                const int chunk = sub * 4 + v4;
                                const uint32_t dst = stage_base + uint32_t(lane) * 128u + uint32_t((chunk ^ (lane & 7)) * 16);
                                const uint32_t w0 = __float_as_uint(__uint_as_float(r[v4 * 4 + 0]) + bv);
                                const uint32_t w1 = __float_as_uint(__uint_as_float(r[v4 * 4 + 1]) + bv);
                                const uint32_t w2 = __float_as_uint(__uint_as_float(r[v4 * 4 + 2]) + bv);
                                const uint32_t w3 = __float_as_uint(__uint_as_float(r[v4 * 4 + 3]) + bv);
                                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w0), "r"(w1), "r"(w2), "r"(w3) : "memory");
                            }
                        }
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0 && t.m0 + q * 32 < p.c_out) {
                            tma_store_4d(&tmY, stage_base, c, t.oh0 + rr, t.m0 + q * 32, t.n);
                            tma_store_commit();
                        }
                    } else {
#pragma unroll
                        for (int sub = 0; sub < 2; sub++) {
                            uint32_t r[16];
                            tmem_ld_x16(t_addr + col + uint32_t(sub * 16), r);
                            tmem_ld_wait();
                            if (!row_ok) continue;
#pragma unroll
                            for (int j = 0; j < 16; j++)
                                if (c + sub * 16 + j < p.Wo) yrow[c + sub * 16 + j] = __uint_as_float(r[j]) + bv;
                        }
                    }
                }
                if constexpr (WRES) {
                    if ((rr & 1) == 1 || rr == t.rows - 1) {  // the accumulator's rows are read: hand it back
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(tempty_bar(abuf));
                        if (++abuf == 2u) {
                            abuf = 0;
                            aph ^= 1u;
                        }
                    }
                }
            }
            if constexpr (!WRES) {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty_bar(buf));
            }
        }
        if (p.tma_out && lane == 0) tma_store_wait<0>();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// W [oc][c][taps] -> bf16 [oc][taps][c] for the fused kernel. Every thread reads eight consecutive source elements
// (one 16-byte load when the source allows it: the whole tensor is one trip to memory) and scatters them. Lets the
// dependent launch start at once: that kernel waits for this grid (griddepcontrol.wait) only where it first reads the copy.
template <typename TIn>
__global__ void __launch_bounds__(256) conv_weights_kernel(const TIn* __restrict__ Wt, __nv_bfloat16* __restrict__ w_hi, int c_out, int C,
                                                           int taps, int vec_ok) {
    griddep_launch_dependents();
    const long long total = (long long)c_out * C * taps;
    const long long i0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (i0 >= total) return;
    TIn v[8];
    if (vec_ok && i0 + 8 <= total) {
        *reinterpret_cast<uint4*>(v) = __ldg(reinterpret_cast<const uint4*>(Wt + i0));
    } else {
#pragma unroll
        for (int e = 0; e < 8; e++) v[e] = i0 + e < total ? Wt[i0 + e] : TIn(0.f);
    }
#pragma unroll
    for (int e = 0; e < 8; e++) {
        const long long i = i0 + e;  // source index ((oc * C + c) * taps + tap)
        if (i < total) {
            const int tap = int(i % taps);
            const long long oc_c = i / taps;
            const int c = int(oc_c % C);
            const long long oc = oc_c / C;
            w_hi[(oc * taps + tap) * C + c] = __float2bfloat16_rn(to_float(v[e]));
        }
    }
}

// X [N][C][HW] -> hi (and lo) [N][HW][C] as bf16, and the weights in the same launch (the blocks of the last
// grid row, blockIdx.y == C / 64). A block moves PX pixels x 64 channels through shared memory as 32-bit
// words holding a channel pair: reads walk pixels (coalesced in NCHW), writes walk channels, so every
// pixel's 64 channels leave as one full 128-byte line. Requires C % 64 == 0.
// PAIR (16-bit input, HW even): every lane reads two neighbouring pixels as one 32-bit word and a block moves
// 128 pixels; otherwise one element per load and 64 pixels.
template <typename TIn, bool SPLIT, bool PAIR>
__global__ void __launch_bounds__(256) nchw_to_nhwc_kernel(const TIn* __restrict__ X, __nv_bfloat16* __restrict__ hi,
                                                           __nv_bfloat16* __restrict__ lo, int C, long long HW, const TIn* __restrict__ Wt,
                                                           __nv_bfloat16* __restrict__ w_hi, __nv_bfloat16* __restrict__ w_lo, int c_out, int taps) {
    constexpr int PX = PAIR ? 128 : 64;
    __shared__ uint32_t tile_hi[PX][33];
    __shared__ uint32_t tile_lo[SPLIT ? PX : 1][33];
    // may start under the launch before it (programmatic stream serialization): no global access before that one is complete
    griddep_wait();
    griddep_launch_dependents();
    if (blockIdx.y == gridDim.y - 1) {
        weight_relayout<TIn, SPLIT>(Wt, w_hi, w_lo, c_out, C, taps, (long long)blockIdx.z * gridDim.x + blockIdx.x, (long long)gridDim.x * gridDim.z);
        return;
    }
    const long long n = blockIdx.z;
    const long long p0 = (long long)blockIdx.x * PX;
    const int c0 = blockIdx.y * 64;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;  // 8 warps
    const TIn* xin = X + (n * C + c0) * HW;
    if constexpr (PAIR) {
        static_assert(sizeof(TIn) == 2 && !SPLIT, "pixel pairs are read as 32-bit words of a 16-bit type");
        // warp w, iteration i: channel pair cp = w + 8*(i/2), pixels 64*(i&1) + 2*lane, +1
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int cp = w + 8 * (i >> 1);
            const int px = (i & 1) * 64 + 2 * lane;
            const long long gp = p0 + px;
            uint32_t a = 0, b = 0;  // (pixel px, pixel px + 1) of channels 2cp and 2cp + 1
            if (gp < HW) {          // HW and gp are even: the pair is inside or outside as a whole
                a = *reinterpret_cast<const uint32_t*>(xin + (long long)(2 * cp) * HW + gp);
                b = *reinterpret_cast<const uint32_t*>(xin + (long long)(2 * cp + 1) * HW + gp);
            }
            if constexpr (!std::is_same<TIn, __nv_bfloat16>::value) {  // fp16 -> bf16
                const __half2 ha = *reinterpret_cast<const __half2*>(&a), hb = *reinterpret_cast<const __half2*>(&b);
                const __nv_bfloat162 ba = __float22bfloat162_rn(__half22float2(ha)), bb = __float22bfloat162_rn(__half22float2(hb));
                a = *reinterpret_cast<const uint32_t*>(&ba);
                b = *reinterpret_cast<const uint32_t*>(&bb);
            }
            tile_hi[px][cp] = __byte_perm(a, b, 0x5410);
            tile_hi[px + 1][cp] = __byte_perm(a, b, 0x7632);
        }
    } else {
        // warp w, iteration i: channel pair cp = w + 8*(i/2), pixel half (i&1)
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int cp = w + 8 * (i >> 1);
            const int px = (i & 1) * 32 + lane;
            const long long gp = p0 + px;
            float a = 0.f, b = 0.f;
            if (gp < HW) {
                a = ld_f(xin + (long long)(2 * cp) * HW + gp);
                b = ld_f(xin + (long long)(2 * cp + 1) * HW + gp);
            }
            const __nv_bfloat16 ah = __float2bfloat16_rn(a), bh = __float2bfloat16_rn(b);
            tile_hi[px][cp] = uint32_t(__bfloat16_as_ushort(ah)) | (uint32_t(__bfloat16_as_ushort(bh)) << 16);
            if (SPLIT) {
                const __nv_bfloat16 al = __float2bfloat16_rn(a - __bfloat162float(ah)), bl = __float2bfloat16_rn(b - __bfloat162float(bh));
                tile_lo[px][cp] = uint32_t(__bfloat16_as_ushort(al)) | (uint32_t(__bfloat16_as_ushort(bl)) << 16);
            }
        }
    }
    __syncthreads();
    uint32_t* out_hi = reinterpret_cast<uint32_t*>(hi);
    uint32_t* out_lo = reinterpret_cast<uint32_t*>(lo);
#pragma unroll
    for (int i = 0; i < PX / 8; i++) {
        const int px = w + 8 * i;
        const long long gp = p0 + px;
        if (gp < HW) {
            const long long o = ((n * HW + gp) * C + c0) / 2 + lane;
            out_hi[o] = tile_hi[px][lane];
            if (SPLIT) out_lo[o] = tile_lo[px][lane];
        }
    }
}

bool g_conv_attr[16] = {false};
bool g_halo_attr[16] = {false};
bool g_fused_attr[16][2][2] = {};

// The fused path: weights re-laid by a small launch, then conv_nchw_kernel on the NCHW input in place.
template <bool IS_BF16>
int launch_fused(Ctx* ctx, const ConvTcProblem& q, ConvKernelParams p, const void* X, const void* Wt, float* Y, bool tma_out) {
    using TIn = typename std::conditional<IS_BF16, __nv_bfloat16, __half>::type;
    const int64_t taps = q.kh * q.kw, Kt = taps * q.C;
    const size_t w_elems = size_t(q.c_out) * Kt;
    // resident weights: 3x3 filter, one channel block, one tile of output channels, weights read where they lie
    static const int wres_mode = [] { const char* e = getenv("DOCC_B200_CONV_WRES"); return e ? atoi(e) : 1; }();
    const bool wres = wres_mode && q.C == 64 && q.c_out <= 128 && q.kh == 3 && q.kw == 3 && reinterpret_cast<uintptr_t>(Wt) % 16 == 0;
    if (wres) {
        // two-row accumulators: a tile's height is not tied to one accumulator's 256 columns any more, only to the halo
        // slots' share of shared memory. Six rows (eight halo rows per slot, a six-chunk input ring) measured best on
        // [32,64,56,56]: 22.6 us at four rows, 21.7 at six, 24.3 at eight (the input ring shrinks to two chunks)
        static const int wres_rmax = [] { const char* e = getenv("DOCC_B200_CONV_WRES_RMAX"); return e ? atoi(e) : 6; }();
        if (wres_rmax >= 2 && wres_rmax <= 8) p.r_max = wres_rmax;
    }
    void* ww = nullptr;
    if (!wres) DOCC_TRY(get_workspace(ctx, 1, w_elems * 2 + 256, &ww));  // the re-laid copy of the streamed form
    __nv_bfloat16* w_hi = static_cast<__nv_bfloat16*>(ww);
    CUtensorMap tm_w, tm_x, tm_y;
    memset(&tm_y, 0, sizeof(tm_y));
    {
        const uint64_t wd[2] = {uint64_t(Kt), uint64_t(q.c_out)};
        const uint64_t ws[1] = {uint64_t(Kt) * 2};
        if (wres) {
            // the caller's [oc][c][3][3] array as rows of 576 elements; a box is 72 elements (eight channels) of 128 rows
            const uint32_t wb[2] = {72, 128};
            DOCC_TRY(encode_tmap(&tm_w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, CU_TENSOR_MAP_SWIZZLE_NONE, Wt, 2, wd, ws, wb));
        } else {
            const uint32_t wb[2] = {64, 128};
            DOCC_TRY(encode_tmap_16bit(&tm_w, w_hi, 2, wd, ws, wb));
        }
        // the input as it lies in memory: pixels, rows, channels, images; one box = one row of 64 channels
        const uint64_t xd[4] = {uint64_t(q.W), uint64_t(q.H), uint64_t(q.C), uint64_t(q.N)};
        const uint64_t xs[3] = {uint64_t(q.W) * 2, uint64_t(q.H * q.W) * 2, uint64_t(q.H * q.W) * q.C * 2};
        const uint32_t xb[4] = {64, 1, 64, 1};
        DOCC_TRY(encode_tmap_16bit(&tm_x, X, 4, xd, xs, xb));
    }
    if (tma_out) {
        const uint64_t yd[4] = {uint64_t(q.Wo), uint64_t(q.Ho), uint64_t(q.c_out), uint64_t(q.N)};
        const uint64_t ys[3] = {uint64_t(q.Wo) * 4, uint64_t(q.Ho * q.Wo) * 4, uint64_t(q.Ho * q.Wo) * q.c_out * 4};
        const uint32_t yb[4] = {32, 1, 32, 1};
        DOCC_TRY(encode_tmap(&tm_y, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, CU_TENSOR_MAP_SWIZZLE_128B, Y, 4, yd, ys, yb));
    }
    // shared memory: two halo slots, eight epilogue staging tiles, then the two rings share what is left
    const size_t halo_total = size_t(kHaloSlots) * size_t(p.r_max + p.kh - 1) * 8192;
    const size_t fixed = 8 * 4096 + 512 + 1024 + 512 + 128;  // staging tiles, dummy rows, barriers and the tile list, alignment slack
    const size_t rings = 227 * 1024 - halo_total - fixed;
    static const int x_chunks_env = [] { const char* e = getenv("DOCC_B200_CONV_XCHUNKS"); return e ? atoi(e) : 0; }();
    int x_chunks = x_chunks_env >= 2 && x_chunks_env <= 8 ? x_chunks_env : 4;
    int w_stages;
    if (wres) {
        w_stages = 1;  // the block of tap 8
        p.even_rows = 1;
        if (!(x_chunks_env >= 2 && x_chunks_env <= 8)) x_chunks = 8;  // the weight ring's room deepens the input ring
        while (x_chunks > 2 && size_t(x_chunks) * kChunkBytes + kABytes > rings) x_chunks--;
    } else {
        w_stages = int((rings - size_t(x_chunks) * kChunkBytes) / kABytes);
        if (w_stages < 3) {  // tall filters leave little room: a shallower input ring
            x_chunks = 2;
            w_stages = int((rings - size_t(x_chunks) * kChunkBytes) / kABytes);
        }
        if (w_stages > kMaxWStages) w_stages = kMaxWStages;
        if (w_stages < 2) return set_error(DOCC_B200_ERR_UNSUPPORTED, "conv_tc: filter too tall for the fused kernel");
    }
    p.w_stages = w_stages;
    p.x_chunks = x_chunks;
    const size_t smem = halo_total + size_t(w_stages) * kABytes + size_t(x_chunks) * kChunkBytes + fixed;
    auto kern = wres ? conv_nchw_kernel<IS_BF16, true> : conv_nchw_kernel<IS_BF16, false>;
    if (!g_fused_attr[ctx->device & 15][IS_BF16 ? 1 : 0][wres ? 1 : 0]) {
        DOCC_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        g_fused_attr[ctx->device & 15][IS_BF16 ? 1 : 0][wres ? 1 : 0] = true;
    }
    if (!wres) {
        const long long wblocks = ceil_div((long long)w_elems, 256 * 8);
        if (wblocks > 0x7fffffff) return set_error(DOCC_B200_ERR_UNSUPPORTED, "conv_tc: weight tensor too large");
        const int vec_ok = reinterpret_cast<uintptr_t>(Wt) % 16 == 0 ? 1 : 0;
        conv_weights_kernel<TIn><<<unsigned(wblocks), 256, 0, ctx->stream>>>(static_cast<const TIn*>(Wt), w_hi, int(q.c_out), int(q.C), int(taps), vec_ok);
        DOCC_TRY(after_launch(ctx, "conv_weights_kernel"));
    }
    long long grid = ceil_div(p.total_units, p.r_max);
    if (grid > ctx->sm_count) grid = ctx->sm_count;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(unsigned(grid));
    cfg.blockDim = dim3(kFusedThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;  // streamed weights: starts under conv_weights_kernel; resident weights: under whatever ran before (the kernel waits)
    DOCC_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, tm_w, tm_x, tm_y, p));
    return after_launch(ctx, "conv_nchw_kernel");
}

}  // namespace

int conv_tc(Ctx* ctx, const ConvTcProblem& q, const void* X, const void* Wt, const float* bias, float* Y) {
    if (q.C % 64 != 0 || q.C <= 0) return set_error(DOCC_B200_ERR_UNSUPPORTED, "conv_tc: C_in %% 64 != 0");
    if (q.Wo < 1 || q.Wo > 256 || q.Ho < 1) return set_error(DOCC_B200_ERR_UNSUPPORTED, "conv_tc: output width outside [1,256]");
    if (q.N > INT32_MAX || q.H > 65535 || q.W > 65535 || q.c_out > INT32_MAX / 2 || q.kh * q.kw * q.C > INT32_MAX / 2)
        return set_error(DOCC_B200_ERR_UNSUPPORTED, "conv_tc: extent too large");
    const bool split = q.prec_in == DOCC_B200_PREC_S;
    const int planes = split ? 2 : 1;
    const int64_t HW = q.H * q.W, taps = q.kh * q.kw, Kt = taps * q.C;
    {
        // 16-bit NCHW inputs of narrow images go through the kernel that reads them in place (TMA rules: rows of a
        // multiple of 16 bytes on a 16-byte aligned base; one 64-pixel box per row has to reach every column a tap reads)
        static const int rmax_env = [] { const char* e = getenv("DOCC_B200_CONV_RMAX"); return e ? atoi(e) : 0; }();
        int fused_rmax = int(10 - q.kh) < 4 ? int(10 - q.kh) : 4;
        if (rmax_env >= 1 && rmax_env < fused_rmax) fused_rmax = rmax_env;
        static const int fused_mode = [] { const char* e = getenv("DOCC_B200_CONV_FUSED"); return e ? atoi(e) : 1; }();
        const bool reach = q.pad_w == 0 ? q.W <= 64 : (q.pad_w <= 8 && q.W <= 56);
        if (fused_mode && !split && q.W % 8 == 0 && reinterpret_cast<uintptr_t>(X) % 16 == 0 && q.Wo + q.kw - 1 <= 64 && reach &&
            q.pad_w >= 0 && fused_rmax >= 1) {
            ConvKernelParams p;
            memset(&p, 0, sizeof(p));
            p.N = int(q.N); p.C = int(q.C); p.H = int(q.H); p.W = int(q.W); p.c_out = int(q.c_out);
            p.kh = int(q.kh); p.kw = int(q.kw); p.pad_h = int(q.pad_h); p.pad_w = int(q.pad_w); p.Ho = int(q.Ho); p.Wo = int(q.Wo);
            p.npass = 1;
            p.r_max = fused_rmax;
            p.tiles_m = int(ceil_div(q.c_out, 128));
            p.total_units = (long long)p.tiles_m * q.N * q.Ho;
            const bool tma_out = q.Wo % 4 == 0 && reinterpret_cast<uintptr_t>(Y) % 16 == 0;
            p.tma_out = tma_out ? 1 : 0;
            p.bias = bias; p.Y = Y; p.status = ctx->status_dev;
            return q.prec_in == DOCC_B200_PREC_B ? launch_fused<true>(ctx, q, p, X, Wt, Y, tma_out)
                                                 : launch_fused<false>(ctx, q, p, X, Wt, Y, tma_out);
        }
    }
    const size_t x_elems = size_t(q.N) * HW * q.C, w_elems = size_t(q.c_out) * Kt;
    void *wx, *ww;
    DOCC_TRY(get_workspace(ctx, 0, x_elems * planes * 2, &wx));
    DOCC_TRY(get_workspace(ctx, 1, w_elems * planes * 2 + 256, &ww));
    __nv_bfloat16* x_hi = static_cast<__nv_bfloat16*>(wx);
    __nv_bfloat16* x_lo = x_hi + x_elems;
    __nv_bfloat16* w_hi = static_cast<__nv_bfloat16*>(ww);
    __nv_bfloat16* w_lo = w_hi + (w_elems + 63) / 64 * 64;

    {
        // one launch re-lays the input and (in the extra grid row) the weights
        const bool pair = !split && HW % 2 == 0 && reinterpret_cast<uintptr_t>(X) % 4 == 0;
        dim3 grid(unsigned(ceil_div(HW, pair ? 128 : 64)), unsigned(q.C / 64 + 1), unsigned(q.N));
        if (grid.z > 65535) return set_error(DOCC_B200_ERR_UNSUPPORTED, "conv_tc: batch too large");
        if (split)
            DOCC_CUDA_TRY(launch_pdl(nchw_to_nhwc_kernel<float, true, false>, grid, dim3(256), 0, ctx->stream, static_cast<const float*>(X), x_hi, x_lo, int(q.C), HW,
                                                                                  static_cast<const float*>(Wt), w_hi, w_lo, int(q.c_out), int(taps)));
        else if (pair)
            DOCC_CUDA_TRY(launch_pdl(nchw_to_nhwc_kernel<__nv_bfloat16, false, true>, grid, dim3(256), 0, ctx->stream, static_cast<const __nv_bfloat16*>(X), x_hi, x_lo, int(q.C), HW,
                                                                                          static_cast<const __nv_bfloat16*>(Wt), w_hi, w_lo, int(q.c_out), int(taps)));
        else
            DOCC_CUDA_TRY(launch_pdl(nchw_to_nhwc_kernel<__nv_bfloat16, false, false>, grid, dim3(256), 0, ctx->stream, static_cast<const __nv_bfloat16*>(X), x_hi, x_lo, int(q.C), HW,
                                                                                           static_cast<const __nv_bfloat16*>(Wt), w_hi, w_lo, int(q.c_out), int(taps)));
        DOCC_TRY(after_launch(ctx, "nchw_to_nhwc_kernel"));
    }

    // narrow images: the halo variant loads each tile's input neighbourhood once for all taps
    int halo_rmax = int(10 - q.kh) < 4 ? int(10 - q.kh) : 4;  // r + kh - 1 <= 9 halo rows of 8 KB per slot (two slots, three weight stages)
    static const int halo_mode = [] { const char* e = getenv("DOCC_B200_CONV_HALO"); return e ? atoi(e) : 1; }();
    const bool halo = halo_mode && q.Wo + q.kw - 1 <= 64 && halo_rmax >= 1;

    CUtensorMap maps[5];
    memset(maps, 0, sizeof(maps));
    const bool tma_out = q.Wo % 4 == 0 && reinterpret_cast<uintptr_t>(Y) % 16 == 0;
    if (tma_out && halo) {
        const uint64_t yd[4] = {uint64_t(q.Wo), uint64_t(q.Ho), uint64_t(q.c_out), uint64_t(q.N)};
        const uint64_t ys[3] = {uint64_t(q.Wo) * 4, uint64_t(q.Ho * q.Wo) * 4, uint64_t(q.Ho * q.Wo) * q.c_out * 4};
        const uint32_t yb[4] = {32, 1, 32, 1};
        DOCC_TRY(encode_tmap(&maps[4], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, CU_TENSOR_MAP_SWIZZLE_128B, Y, 4, yd, ys, yb));
    } else if (tma_out) {
        const uint64_t yd[3] = {uint64_t(q.Ho * q.Wo), uint64_t(q.c_out), uint64_t(q.N)};
        const uint64_t ys[2] = {uint64_t(q.Ho * q.Wo) * 4, uint64_t(q.Ho * q.Wo) * q.c_out * 4};
        const uint32_t yb[3] = {32, 32, 1};
        DOCC_TRY(encode_tmap(&maps[4], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, CU_TENSOR_MAP_SWIZZLE_128B, Y, 3, yd, ys, yb));
    }
    for (int i = 0; i < 2; i++) {
        const __nv_bfloat16* wp = (i == 1 && split) ? w_lo : w_hi;
        const __nv_bfloat16* xp = (i == 1 && split) ? x_lo : x_hi;
        const uint64_t wd[2] = {uint64_t(Kt), uint64_t(q.c_out)};
        const uint64_t ws[1] = {uint64_t(Kt) * 2};
        const uint32_t wb[2] = {64, 128};
        DOCC_TRY(encode_tmap_16bit(&maps[i], wp, 2, wd, ws, wb));
        const uint64_t xd[4] = {uint64_t(q.C), uint64_t(q.W), uint64_t(q.H), uint64_t(q.N)};
        const uint64_t xs[3] = {uint64_t(q.C) * 2, uint64_t(q.W) * q.C * 2, uint64_t(HW) * q.C * 2};
        const uint32_t xb[4] = {64, halo ? 64u : uint32_t(q.Wo), halo ? uint32_t(halo_rmax + q.kh - 1) : 1u, 1};
        DOCC_TRY(encode_tmap_16bit(&maps[2 + i], xp, 4, xd, xs, xb));
    }

    ConvKernelParams p;
    memset(&p, 0, sizeof(p));
    p.N = int(q.N); p.C = int(q.C); p.H = int(q.H); p.W = int(q.W); p.c_out = int(q.c_out);
    p.kh = int(q.kh); p.kw = int(q.kw); p.pad_h = int(q.pad_h); p.pad_w = int(q.pad_w); p.Ho = int(q.Ho); p.Wo = int(q.Wo);
    if (split) {
        p.npass = 3;  // small terms first
        p.pw[0] = 1; p.px[0] = 0;
        p.pw[1] = 0; p.px[1] = 1;
        p.pw[2] = 0; p.px[2] = 0;
    } else {
        p.npass = 1;
    }
    p.r_max = int(256 / q.Wo);
    if (p.r_max > 8) p.r_max = 8;
    if (halo) p.r_max = halo_rmax;
    p.tiles_m = int(ceil_div(q.c_out, 128));
    p.total_units = (long long)p.tiles_m * q.N * q.Ho;
    p.tma_out = tma_out ? 1 : 0;
    p.bias = bias; p.Y = Y; p.status = ctx->status_dev;

    if (halo) {
        const size_t fixed = 8 * 4096 + 1024 + 256;
        const size_t slot_bytes = size_t(p.r_max + p.kh - 1) * 8192;
        // split operands: a third halo slot (both input planes of a tile resident, the next tile's first plane in flight)
        // when it leaves a weight ring of three stages
        static const int paired_mode = [] { const char* e = getenv("DOCC_B200_CONV_PAIRED"); return e ? atoi(e) : 1; }();
        p.paired = (split && paired_mode == 1 && 227 * 1024 >= 3 * slot_bytes + fixed + 3 * kABytes) ? 1 : (split && paired_mode == 2) ? 2 : 0;
        const size_t halo_total = size_t(p.paired == 1 ? 3 : kHaloSlots) * slot_bytes;
        int w_stages = int((227 * 1024 - halo_total - fixed) / kABytes);
        if (w_stages > kMaxWStages) w_stages = kMaxWStages;
        p.w_stages = w_stages;
        const size_t smem_h = halo_total + size_t(w_stages) * kABytes + fixed;
        if (!g_halo_attr[ctx->device & 15]) {
            DOCC_CUDA_TRY(cudaFuncSetAttribute(conv_halo_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
            g_halo_attr[ctx->device & 15] = true;
        }
        long long grid_h = ceil_div(p.total_units, p.r_max);
        if (grid_h > ctx->sm_count) grid_h = ctx->sm_count;
        DOCC_CUDA_TRY(launch_pdl(conv_halo_kernel, dim3(unsigned(grid_h)), dim3(kHaloThreads), smem_h, ctx->stream, maps[0], maps[1], maps[2], maps[3], maps[4], p));
        return after_launch(ctx, "conv_halo_kernel");
    }
    const size_t smem = size_t(kStages) * (kABytes + kBBytes) + 4 * 4096 + 1024 + 256;
    if (!g_conv_attr[ctx->device & 15]) {
        DOCC_CUDA_TRY(cudaFuncSetAttribute(conv_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        g_conv_attr[ctx->device & 15] = true;
    }
    // enough CTAs that each gets at least one full tile; never more than one per SM
    long long grid = ceil_div(p.total_units, p.r_max);
    if (grid > ctx->sm_count) grid = ctx->sm_count;
    conv_tc_kernel<<<unsigned(grid), kThreads, smem, ctx->stream>>>(maps[0], maps[1], maps[2], maps[3], maps[4], p);
    return after_launch(ctx, "conv_tc_kernel");
}

}  // namespace docc_b200

