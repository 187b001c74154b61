// Flash attention on tcgen05: O = softmax(scale * Q K^T [+ causal mask]) V for 16-bit inputs,
// head_dim 64 or 128, fp32 accumulation. The Sq x Skv score matrix never leaves the SM.
//
// Three kernels, all with a TMA producer warp, a UMMA issuer warp and softmax warp groups in which thread r owns
// query row r (running max / sum in the exp2 domain), and key/value blocks of 128:
//   attention_tc_kernel    one 128-row query tile per CTA (sequences of at most 128 queries): S_j = Q K_j^T and
//                          O_j = P_j V_j alternate between two TMEM buffers each, P_j goes through shared memory
//                          in the 128-byte swizzled layout UMMA reads, O is accumulated in registers.
//   attention_tc2_kernel   two query tiles per CTA, P and O resident in tensor memory (causal problems: one CTA
//                          per pair of tiles, heaviest first).
//   attention_tc2p_kernel  the same tile pair, persistent: one CTA per SM walks the (batch, head, pair) items of
//                          an unmasked problem.
// All waits are bounded.
#include <cstdlib>
#include <type_traits>

#include "attention.h"
#include "device_math.cuh"
#include "gemm_tc.h"
#include "ptx.cuh"

namespace docc_b200 {
namespace {

using namespace ptx;

constexpr int kBQ = 128;   // query rows per CTA
constexpr int kBKV = 128;  // keys per block
constexpr int kAttnThreads = 192;

struct AttnKernelParams {
    int Sq, Skv, H;
    int n_qtiles;
    int n_items;  // persistent kernel: (batch, head, tile pair) work items
    int causal;
    int causal_off;  // Skv - Sq: query i sees keys j <= i + causal_off
    float scale_log2;  // scale * log2(e)
    void* O;
    long long os_b, os_h, os_s;
    void* O_hi;  // persistent fp32 kernel: when set, O leaves as bf16 hi / lo planes (same strides) instead of fp32
    void* O_lo;
    DeviceStatus* status;
};

__device__ __forceinline__ void attn_timeout(DeviceStatus* st, unsigned where) {
    volatile unsigned int* f = &st->timeout_flag;
    volatile unsigned int* w = &st->timeout_where;
    if (*w == 0u) *w = where;
    *f = 1u;
    __threadfence_system();
}

// max of three in one instruction (sm_100): the block-maximum pass costs half an instruction per score
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// packed pairs of fp32 (sm_100): (y0, y1) = (x0, x1) * a + c, and (a0, a1) += (x0, x1), one instruction each
__device__ __forceinline__ void fma2(float& y0, float& y1, float x0, float x1, float a, float c) {
    asm("{\n.reg .b64 s, sa, sc, r;\nmov.b64 s, {%2, %3};\nmov.b64 sa, {%4, %4};\nmov.b64 sc, {%5, %5};\nfma.rn.f32x2 r, s, sa, sc;\n"
        "mov.b64 {%0, %1}, r;\n}"
        : "=f"(y0), "=f"(y1)
        : "f"(x0), "f"(x1), "f"(a), "f"(c));
}
__device__ __forceinline__ void add2(float& a0, float& a1, float x0, float x1) {
    asm("{\n.reg .b64 s, t, r;\nmov.b64 s, {%0, %1};\nmov.b64 t, {%2, %3};\nadd.rn.f32x2 r, s, t;\nmov.b64 {%0, %1}, r;\n}"
        : "+f"(a0), "+f"(a1)
        : "f"(x0), "f"(x1));
}

__device__ __forceinline__ float ex2(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

template <bool IS_BF16> __device__ __forceinline__ uint32_t pack2(float a, float b) {
    if constexpr (IS_BF16) {
        __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&v);
    } else {
        __half2 v = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&v);
    }
}

// Shared memory map (offsets from a 1024-byte aligned base):
//   Q   : D/64 chunks of [128 rows][128 B]            = 16 KB * D/64
//   K[2]: same shape per stage
//   V[2]: D/64 chunks of [128 kv rows][128 B] per stage (MN-major for the P V product)
//   P   : 2 chunks of [128 rows][128 B]                = 32 KB
template <int D, bool IS_BF16>
__global__ void __launch_bounds__(kAttnThreads, 1)
    attention_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                        const __grid_constant__ CUtensorMap tmV, const AttnKernelParams p) {
    constexpr int DC = D / 64;                      // 64-element chunks along head_dim
    constexpr uint32_t kTile = uint32_t(DC) * 16384u;  // bytes of one Q / K / V tile
    constexpr uint32_t kPBytes = 32768u;
    constexpr uint32_t kTmemCols = 512;
    constexpr uint32_t kSCol = 0;      // two score buffers of 128 columns
    constexpr uint32_t kOCol = 256;    // two output buffers, 128 columns apart
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    const uint32_t sQ = base;
    const uint32_t sK = sQ + kTile;
    const uint32_t sV = sK + 2 * kTile;
    const uint32_t sP = sV + 2 * kTile;
    const uint32_t bars = sP + kPBytes;
    const uint32_t q_full = bars;
    auto k_full = [&](int i) { return bars + 8u + 8u * uint32_t(i); };
    auto k_empty = [&](int i) { return bars + 24u + 8u * uint32_t(i); };
    auto v_full = [&](int i) { return bars + 40u + 8u * uint32_t(i); };
    auto v_empty = [&](int i) { return bars + 56u + 8u * uint32_t(i); };
    auto s_full = [&](int i) { return bars + 72u + 8u * uint32_t(i); };
    auto s_empty = [&](int i) { return bars + 88u + 8u * uint32_t(i); };
    auto o_full = [&](int i) { return bars + 104u + 8u * uint32_t(i); };
    const uint32_t p_full = bars + 120u;
    volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem_raw + (bars + 128u - raw_addr));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // heavier (later) query tiles first under a causal mask
    const int qt_raw = blockIdx.x % p.n_qtiles;
    const int qtile = p.causal ? p.n_qtiles - 1 - qt_raw : qt_raw;
    const int bh = blockIdx.x / p.n_qtiles;
    const int h = bh % p.H, b = bh / p.H;
    const int q0 = qtile * kBQ;
    // keys this tile can see
    int kv_end = p.Skv;
    if (p.causal) {
        const int last = q0 + kBQ - 1 + p.causal_off;  // last key visible to the last row of the tile
        kv_end = last + 1 < p.Skv ? last + 1 : p.Skv;
        if (kv_end < 0) kv_end = 0;
    }
    const int n_blocks = (kv_end + kBKV - 1) / kBKV;

    if (warp == 0 && lane == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; i++) {
            mbar_init(k_full(i), 1);
            mbar_init(k_empty(i), 1);
            mbar_init(v_full(i), 1);
            mbar_init(v_empty(i), 1);
            mbar_init(s_full(i), 1);
            mbar_init(s_empty(i), 4);
            mbar_init(o_full(i), 1);
        }
        mbar_init(p_full, 4);
        fence_barrier_init();
        prefetch_tensormap(&tmQ);
        prefetch_tensormap(&tmK);
        prefetch_tensormap(&tmV);
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

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0 && n_blocks > 0) {
            mbar_arrive_expect_tx(q_full, kTile);
            for (int c = 0; c < DC; c++) tma_load_4d(sQ + uint32_t(c) * 16384u, &tmQ, q_full, c * 64, q0, h, b);
            for (int j = 0; j < n_blocks; j++) {
                const int s = j & 1;
                const uint32_t ph = uint32_t(j >> 1) & 1u;
                if (!mbar_wait(k_empty(s), ph ^ 1u)) { attn_timeout(p.status, 11); break; }
                mbar_arrive_expect_tx(k_full(s), kTile);
                for (int c = 0; c < DC; c++)
                    tma_load_4d(sK + uint32_t(s) * kTile + uint32_t(c) * 16384u, &tmK, k_full(s), c * 64, j * kBKV, h, b);
                if (!mbar_wait(v_empty(s), ph ^ 1u)) { attn_timeout(p.status, 12); break; }
                mbar_arrive_expect_tx(v_full(s), kTile);
                for (int c = 0; c < DC; c++)
                    tma_load_4d(sV + uint32_t(s) * kTile + uint32_t(c) * 16384u, &tmV, v_full(s), c * 64, j * kBKV, h, b);
            }
        }
    } else if (warp == 1) {
        // ---------------- UMMA issuer ----------------
        if (lane == 0 && n_blocks > 0) {
            constexpr uint32_t idesc_qk = make_idesc(kBQ, kBKV, IS_BF16 ? 1 : 0, 0, 0);
            constexpr uint32_t idesc_pv = make_idesc(kBQ, D, IS_BF16 ? 1 : 0, 0, 1);
            bool ok = mbar_wait(q_full, 0);
            if (!ok) attn_timeout(p.status, 13);
            auto issue_qk = [&](int j) -> bool {
                const int s = j & 1;
                const uint32_t ph = uint32_t(j >> 1) & 1u;
                if (!mbar_wait(k_full(s), ph)) { attn_timeout(p.status, 14); return false; }
                if (!mbar_wait(s_empty(s), ph ^ 1u)) { attn_timeout(p.status, 15); return false; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + kSCol + uint32_t(s) * 128u;
                const uint32_t kb = sK + uint32_t(s) * kTile;
#pragma unroll
                for (int kk = 0; kk < D / 16; kk++) {
                    const uint32_t off = uint32_t(kk / 4) * 16384u + uint32_t(kk % 4) * 32u;
                    umma_f16_ss(d_tmem, make_smem_desc(sQ + off, 16u, 1024u), make_smem_desc(kb + off, 16u, 1024u), idesc_qk,
                                kk > 0 ? 1u : 0u);
                }
                umma_commit(k_empty(s));
                umma_commit(s_full(s));
                return true;
            };
            if (ok) ok = issue_qk(0);
            for (int j = 0; j < n_blocks && ok; j++) {
                if (j + 1 < n_blocks) {
                    ok = issue_qk(j + 1);
                    if (!ok) break;
                }
                const int s = j & 1;
                const uint32_t ph = uint32_t(j >> 1) & 1u;
                if (!mbar_wait(v_full(s), ph)) { attn_timeout(p.status, 16); break; }
                if (!mbar_wait(p_full, uint32_t(j) & 1u)) { attn_timeout(p.status, 17); break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + kOCol + uint32_t(s) * 128u;
                const uint32_t vb = sV + uint32_t(s) * kTile;
#pragma unroll
                for (int kk = 0; kk < kBKV / 16; kk++) {
                    // P: K-major, two 64-key chunks of 16 KB. V: MN-major, D/64 chunks of 16 KB, 16 key rows = 2 KB.
                    const uint64_t da = make_smem_desc(sP + uint32_t(kk / 4) * 16384u + uint32_t(kk % 4) * 32u, 16u, 1024u);
                    const uint64_t db = make_smem_desc(vb + uint32_t(kk) * 2048u, 16384u, 1024u);
                    umma_f16_ss(d_tmem, da, db, idesc_pv, kk > 0 ? 1u : 0u);
                }
                umma_commit(v_empty(s));
                umma_commit(o_full(s));
            }
        }
    } else {
        // ---------------- softmax / accumulate / store ----------------
        const int quad = warp & 3;
        const int r = quad * 32 + lane;  // row inside the tile == TMEM lane
        const int row = q0 + r;
        const uint32_t lane_addr = tmem_base + (uint32_t(quad * 32) << 16);
        float acc[D];
#pragma unroll
        for (int i = 0; i < D; i++) acc[i] = 0.f;
        float m = -INFINITY, l = 0.f, corr_prev = 1.f;
        bool ok = true;
        const int row_limit = p.causal ? row + p.causal_off : p.Skv - 1;  // last visible key of this row

        auto accumulate = [&](int j, float corr) -> bool {
            const int s = j & 1;
            if (!mbar_wait(o_full(s), uint32_t(j >> 1) & 1u)) {
                if (lane == 0) attn_timeout(p.status, 18);
                return false;
            }
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < D / 32; c++) {
                uint32_t o[32];
                tmem_ld_x32(lane_addr + kOCol + uint32_t(s) * 128u + uint32_t(c) * 32u, o);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; i++) acc[c * 32 + i] = fmaf(acc[c * 32 + i], corr, __uint_as_float(o[i]));
            }
            return true;
        };

        for (int j = 0; j < n_blocks && ok; j++) {
            const int s = j & 1;
            const int k0 = j * kBKV;
            if (!mbar_wait(s_full(s), uint32_t(j >> 1) & 1u)) {
                if (lane == 0) attn_timeout(p.status, 19);
                ok = false;
                break;
            }
            tc_fence_after();
            const uint32_t s_addr = lane_addr + kSCol + uint32_t(s) * 128u;
            const bool need_mask = (k0 + kBKV > p.Skv) || (p.causal && k0 + kBKV - 1 > q0 + p.causal_off);
            const int visible = (row_limit < p.Skv - 1 ? row_limit : p.Skv - 1) - k0;  // local index of the last visible key
            // pass 1: block maximum
            float bm = -INFINITY;
#pragma unroll
            for (int c = 0; c < kBKV / 32; c++) {
                uint32_t sv[32];
                tmem_ld_x32(s_addr + uint32_t(c) * 32u, sv);
                tmem_ld_wait();
                if (need_mask) {
#pragma unroll
                    for (int i = 0; i < 32; i++)
                        if (c * 32 + i <= visible) bm = fmaxf(bm, __uint_as_float(sv[i]));
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i++) bm = fmaxf(bm, __uint_as_float(sv[i]));
                }
            }
            const float m_new = fmaxf(m, bm * p.scale_log2);
            const float m_ref = (m_new == -INFINITY) ? 0.f : m_new;
            const float corr = ex2(m - m_ref);  // 0 on the first block (m = -inf)
            // P_{j-1} must have been consumed by the tensor pipe before P_j overwrites it
            if (j > 0) {
                if (!mbar_wait(o_full((j - 1) & 1), uint32_t((j - 1) >> 1) & 1u)) {
                    if (lane == 0) attn_timeout(p.status, 20);
                    ok = false;
                    break;
                }
            }
            // pass 2: exponentials, row sum, P to shared memory
            float bl = 0.f;
#pragma unroll
            for (int c = 0; c < kBKV / 32; c++) {
                uint32_t sv[32];
                tmem_ld_x32(s_addr + uint32_t(c) * 32u, sv);
                tmem_ld_wait();
                float e[32];
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    float x = ex2(fmaf(__uint_as_float(sv[i]), p.scale_log2, -m_ref));
                    if (need_mask && c * 32 + i > visible) x = 0.f;
                    e[i] = x;
                    bl += x;
                }
                // 32 keys = four 16-byte units; unit u of the row lands at (u ^ (r & 7)) in its 128-byte line
#pragma unroll
                for (int u4 = 0; u4 < 4; u4++) {
                    const int u = (c * 4 + u4) & 7;
                    const uint32_t dst = sP + uint32_t(c / 2) * 16384u + uint32_t(r) * 128u + uint32_t((u ^ (r & 7)) * 16);
                    const uint32_t w0 = pack2<IS_BF16>(e[u4 * 8 + 0], e[u4 * 8 + 1]);
                    const uint32_t w1 = pack2<IS_BF16>(e[u4 * 8 + 2], e[u4 * 8 + 3]);
                    const uint32_t w2 = pack2<IS_BF16>(e[u4 * 8 + 4], e[u4 * 8 + 5]);
                    const uint32_t w3 = pack2<IS_BF16>(e[u4 * 8 + 6], e[u4 * 8 + 7]);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w0), "r"(w1), "r"(w2), "r"(w3) : "memory");
                }
            }
            l = l * corr + bl;
            m = m_new;
            // S_j is free for Q K_{j+2}^T; P_j is ready for the tensor pipe
            tc_fence_before();
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(s_empty(s));
                mbar_arrive(p_full);
            }
            // fold in the previous block's P V while the tensor pipe works on this one
            if (j > 0) ok = accumulate(j - 1, corr_prev);
            corr_prev = corr;
        }
        if (ok && n_blocks > 0) ok = accumulate(n_blocks - 1, corr_prev);

        if (row < p.Sq) {
            const float inv = l > 0.f ? 1.f / l : 0.f;
            using T = typename std::conditional<IS_BF16, __nv_bfloat16, __half>::type;
            T* o = static_cast<T*>(p.O) + b * p.os_b + h * p.os_h + (long long)row * p.os_s;
#pragma unroll
            for (int c = 0; c < D / 8; c++) {
                uint4 w;
                w.x = pack2<IS_BF16>(acc[c * 8 + 0] * inv, acc[c * 8 + 1] * inv);
                w.y = pack2<IS_BF16>(acc[c * 8 + 2] * inv, acc[c * 8 + 3] * inv);
                w.z = pack2<IS_BF16>(acc[c * 8 + 4] * inv, acc[c * 8 + 5] * inv);
                w.w = pack2<IS_BF16>(acc[c * 8 + 6] * inv, acc[c * 8 + 7] * inv);
                *reinterpret_cast<uint4*>(o + c * 8) = w;
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}


__host__ __device__ constexpr int attn2_slots(int d, bool split) {
    const int tile = (d / 64) * 16384;
    const int n = (227 * 1024 - 2048 - 2 * (split ? 2 : 1) * tile) / tile;
    return n > 8 ? 8 : n;
}

// ---- two query tiles per CTA, P and O resident in tensor memory ------------------------------------------
// 320 threads: TMA warp, UMMA warp, and one softmax warp group per 128-row query tile. Per tile t the
// 128 score columns S_t and the 128 output columns O_t live in TMEM (2 x 256 = all 512 columns):
//   * the softmax group reads S_t, writes P_t (16-bit, two keys per 32-bit column) back over the first
//     64 columns of S_t with tcgen05.st, and the P V product takes its A operand straight from TMEM;
//   * O_t is accumulated in place by the tensor pipe (accumulate flag on from the second block). The
//     running maximum is only raised when it grew by more than 2^8; then the warp rescales its 32 rows
//     of O_t in TMEM (tcgen05.ld / st) and the row sums. Rows keep exponentials relative to a slightly
//     stale maximum otherwise, which cancels in the final division by the row sum.
// The tensor pipe alternates between the tiles: P V of tile t block j, then Q K^T of tile t block
// j+1 (S_t may only be overwritten once P_t has been consumed), so one group does softmax while the
// pipe works for the other. K_j / V_j tiles travel through one ring of shared-memory slots and are
// shared by both tiles.
// SPLIT: fp32 attention. Q, K, V arrive as bf16 hi/lo planes (x = hi + lo to ~16 bits); Q K^T and
// P V each run three products (lo*hi, hi*lo, hi*hi) into the same accumulator, P is split the same way
// (P_hi in columns 0-63 and P_lo in columns 64-127 of S_t), and O leaves as fp32.
template <int D, bool IS_BF16, bool SPLIT>
__global__ void __launch_bounds__(320, 1)
    attention_tc2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                         const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmQl,
                         const __grid_constant__ CUtensorMap tmKl, const __grid_constant__ CUtensorMap tmVl,
                         const AttnKernelParams p) {
    constexpr int DC = D / 64;
    constexpr uint32_t kTile = uint32_t(DC) * 16384u;
    constexpr int QP = SPLIT ? 2 : 1;  // planes per query tile
    constexpr int EB = SPLIT ? 4 : 2;  // ring entries per key block: K_hi, [K_lo], V_hi, [V_lo]
    constexpr int NS = attn2_slots(D, SPLIT);
    constexpr uint32_t kTmemCols = 512;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    const uint32_t sQ = base;                      // two query tiles (x hi/lo planes): tile t plane pl at (t*QP + pl)*kTile
    const uint32_t sKV = sQ + 2 * QP * kTile;      // NS ring slots
    const uint32_t bars = sKV + uint32_t(NS) * kTile;
    auto kv_full = [&](int i) { return bars + 8u * uint32_t(i); };
    auto kv_empty = [&](int i) { return bars + 64u + 8u * uint32_t(i); };
    auto q_full = [&](int t) { return bars + 128u + 8u * uint32_t(t); };
    auto s_full = [&](int t) { return bars + 144u + 8u * uint32_t(t); };
    auto p_full = [&](int t) { return bars + 160u + 8u * uint32_t(t); };
    auto o_full = [&](int t) { return bars + 176u + 8u * uint32_t(t); };
    volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem_raw + (bars + 192u - raw_addr));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_pairs = (p.n_qtiles + 1) / 2;
    const int pr_raw = blockIdx.x % n_pairs;
    const int pair = p.causal ? n_pairs - 1 - pr_raw : pr_raw;  // heavier tiles first under a causal mask
    const int bh = blockIdx.x / n_pairs;
    const int h = bh % p.H, b = bh / p.H;
    int q0[2], nb[2];
    for (int t = 0; t < 2; t++) {
        q0[t] = (pair * 2 + t) * kBQ;
        int kv_end = p.Skv;
        if (p.causal) {
            const int last = q0[t] + kBQ - 1 + p.causal_off;
            kv_end = last + 1 < p.Skv ? last + 1 : p.Skv;
            if (kv_end < 0) kv_end = 0;
        }
        nb[t] = q0[t] < p.Sq ? (kv_end + kBKV - 1) / kBKV : 0;
    }
    const int n_max = nb[0] > nb[1] ? nb[0] : nb[1];

    if (warp == 0 && lane == 0) {
        for (int i = 0; i < NS; i++) {
            mbar_init(kv_full(i), 1);
            mbar_init(kv_empty(i), 1);
        }
        for (int t = 0; t < 2; t++) {
            mbar_init(q_full(t), 1);
            mbar_init(s_full(t), 1);
            mbar_init(p_full(t), 4);
            mbar_init(o_full(t), 1);
        }
        fence_barrier_init();
        prefetch_tensormap(&tmQ);
        prefetch_tensormap(&tmK);
        prefetch_tensormap(&tmV);
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

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0 && n_max > 0) {
            for (int t = 0; t < 2; t++) {
                if (nb[t] == 0) continue;
                mbar_arrive_expect_tx(q_full(t), QP * kTile);
                for (int pl = 0; pl < QP; pl++)
                    for (int c = 0; c < DC; c++)
                        tma_load_4d(sQ + uint32_t(t * QP + pl) * kTile + uint32_t(c) * 16384u, pl ? &tmQl : &tmQ, q_full(t), c * 64, q0[t], h, b);
            }
            for (int i = 0; i < EB * n_max; i++) {  // entry e = i % EB of block j = i / EB
                const int s = i % NS;
                const uint32_t ph = uint32_t(i / NS) & 1u;
                if (!mbar_wait(kv_empty(s), ph ^ 1u)) { attn_timeout(p.status, 31); break; }
                mbar_arrive_expect_tx(kv_full(s), kTile);
                const int e = i % EB;
                const CUtensorMap* m = SPLIT ? (e == 0 ? &tmK : e == 1 ? &tmKl : e == 2 ? &tmV : &tmVl) : (e ? &tmV : &tmK);
                for (int c = 0; c < DC; c++)
                    tma_load_4d(sKV + uint32_t(s) * kTile + uint32_t(c) * 16384u, m, kv_full(s), c * 64, (i / EB) * kBKV, h, b);
            }
        }
    } else if (warp == 1) {
        // ---------------- UMMA issuer ----------------
        if (lane == 0 && n_max > 0) {
            constexpr uint32_t idesc_qk = make_idesc(kBQ, kBKV, IS_BF16 ? 1 : 0, 0, 0);
            constexpr uint32_t idesc_pv = make_idesc(kBQ, D, IS_BF16 ? 1 : 0, 0, 1);
            bool ok = true;
            auto wait_slot = [&](int i) -> uint32_t {  // returns the slot base, 0 on timeout
                const int s = i % NS;
                if (!mbar_wait(kv_full(s), uint32_t(i / NS) & 1u)) { attn_timeout(p.status, 32); ok = false; return 0u; }
                tc_fence_after();
                return sKV + uint32_t(s) * kTile;
            };
            // Q K^T of tile t: hi*hi, plus the two cross terms for fp32 operands (small terms first)
            // Descriptors are built once per operand tile; the k-steps only add a constant to the address
            // field (16-byte units), which keeps the issuing thread ahead of the tensor pipe.
            auto issue_qk = [&](int t, uint32_t kb_hi, uint32_t kb_lo) {
                const uint32_t d_tmem = tmem_base + uint32_t(t) * 128u;
                const uint64_t q_hi = make_smem_desc(sQ + uint32_t(t * QP) * kTile, 16u, 1024u);
                const uint64_t q_lo = q_hi + uint64_t(kTile >> 4);
                uint32_t acc = 0;
                auto product = [&](uint64_t qd, uint32_t kb) {
                    const uint64_t kd = make_smem_desc(kb, 16u, 1024u);
#pragma unroll
                    for (int kk = 0; kk < D / 16; kk++) {
                        const uint64_t off = uint64_t((uint32_t(kk / 4) * 16384u + uint32_t(kk % 4) * 32u) >> 4);
                        umma_f16_ss(d_tmem, qd + off, kd + off, idesc_qk, acc);
                        acc = 1;
                    }
                };
                if (SPLIT) {
                    product(q_lo, kb_hi);
                    product(q_hi, kb_lo);
                }
                product(q_hi, kb_hi);
                umma_commit(s_full(t));
            };
            for (int t = 0; t < 2 && ok; t++) {
                if (nb[t] == 0) continue;
                if (!mbar_wait(q_full(t), 0)) { attn_timeout(p.status, 33); ok = false; }
            }
            if (ok) {
                const uint32_t k_hi = wait_slot(0);
                const uint32_t k_lo = (SPLIT && ok) ? wait_slot(1) : 0u;
                if (ok) {
                    for (int t = 0; t < 2; t++) if (nb[t] > 0) issue_qk(t, k_hi, k_lo);
                    umma_commit(kv_empty(0 % NS));
                    if (SPLIT) umma_commit(kv_empty(1 % NS));
                }
            }
            for (int j = 0; j < n_max && ok; j++) {
                const int iv = EB * j + (SPLIT ? 2 : 1);      // first V entry of block j
                const int ik = EB * (j + 1);                  // first K entry of block j+1
                const uint32_t v_hi = wait_slot(iv);
                if (!ok) break;
                const uint32_t v_lo = SPLIT ? wait_slot(iv + 1) : 0u;
                if (!ok) break;
                uint32_t k_hi = 0, k_lo = 0;
                if (j + 1 < n_max) {
                    k_hi = wait_slot(ik);
                    if (!ok) break;
                    if (SPLIT) k_lo = wait_slot(ik + 1);
                    if (!ok) break;
                }
                for (int t = 0; t < 2 && ok; t++) {
                    if (j >= nb[t]) continue;
                    if (!mbar_wait(p_full(t), uint32_t(j) & 1u)) { attn_timeout(p.status, 34); ok = false; break; }
                    tc_fence_after();
                    const uint32_t o_tmem = tmem_base + 256u + uint32_t(t) * 128u;
                    const uint32_t p_hi = tmem_base + uint32_t(t) * 128u;  // P_t over the first 64 columns of S_t
                    const uint32_t p_lo = p_hi + 64u;                       // (fp32 path) low part over the last 64
                    uint32_t acc = j > 0 ? 1u : 0u;
                    auto product = [&](uint32_t pa, uint32_t vb) {
                        const uint64_t vd = make_smem_desc(vb, 16384u, 1024u);
#pragma unroll
                        for (int kk = 0; kk < kBKV / 16; kk++) {
                            umma_f16_ts(o_tmem, pa + uint32_t(kk) * 8u, vd + uint64_t(kk * (2048 / 16)), idesc_pv, acc);
                            acc = 1;
                        }
                    };
                    if (SPLIT) {
                        product(p_lo, v_hi);
                        product(p_hi, v_lo);
                    }
                    product(p_hi, v_hi);
                    umma_commit(o_full(t));
                    if (j + 1 < nb[t]) issue_qk(t, k_hi, k_lo);
                }
                if (!ok) break;
                umma_commit(kv_empty(iv % NS));
                if (SPLIT) umma_commit(kv_empty((iv + 1) % NS));
                if (j + 1 < n_max) {
                    umma_commit(kv_empty(ik % NS));
                    if (SPLIT) umma_commit(kv_empty((ik + 1) % NS));
                }
            }
        }
    } else {
        // ---------------- softmax groups ----------------
        const int t = (warp - 2) >> 2;
        const int quad = warp & 3;
        const int r = quad * 32 + lane;
        const int row = q0[t] + r;
        const uint32_t lane_addr = tmem_base + (uint32_t(quad * 32) << 16);
        const uint32_t s_addr = lane_addr + uint32_t(t) * 128u;
        const uint32_t o_addr = lane_addr + 256u + uint32_t(t) * 128u;
        const int n_t = nb[t];
        float m = -INFINITY;  // maximum the stored exponentials are relative to
        float l = 0.f;
        bool ok = true;
        const int row_limit = p.causal ? row + p.causal_off : p.Skv - 1;

        for (int j = 0; j < n_t && ok; j++) {
            const int k0 = j * kBKV;
            if (!mbar_wait(s_full(t), uint32_t(j) & 1u)) {
                if (lane == 0) attn_timeout(p.status, 35);
                ok = false;
                break;
            }
            tc_fence_after();
            const bool need_mask = (k0 + kBKV > p.Skv) || (p.causal && k0 + kBKV - 1 > q0[t] + p.causal_off);
            const int visible = (row_limit < p.Skv - 1 ? row_limit : p.Skv - 1) - k0;
            // The block body exists twice, with and without masking: the mask test is uniform over the warp, and as a
            // run-time condition inside the loops it costs two compare/select instructions per score on every block.
            auto block_body = [&](auto mask_c) {
            constexpr bool MASK = decltype(mask_c)::value;
            // Pass 1 (block maximum) with two chunk loads in flight: the next 32 columns are requested
            // before the current ones are reduced, so the TMEM read latency overlaps the arithmetic.
            // four independent running maxima / sums: a single chain of 128 dependent operations would
            // leave the two warps per scheduler waiting on arithmetic latency
            float bm4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            uint32_t sa[32], sb[32];
            auto max_chunk = [&](const uint32_t (&sv)[32], int c) {
                if (MASK) {
#pragma unroll
                    for (int i = 0; i < 32; i++)
                        if (c * 32 + i <= visible) bm4[i & 3] = fmaxf(bm4[i & 3], __uint_as_float(sv[i]));
                } else {
#pragma unroll
                    for (int i = 0; i < 16; i++) bm4[i & 3] = max3(bm4[i & 3], __uint_as_float(sv[2 * i]), __uint_as_float(sv[2 * i + 1]));
                }
            };
            tmem_ld_x32(s_addr, sa);
            tmem_ld_wait();
            tmem_ld_x32(s_addr + 32u, sb);
            max_chunk(sa, 0);
            tmem_ld_wait();
            tmem_ld_x32(s_addr + 64u, sa);
            max_chunk(sb, 1);
            tmem_ld_wait();
            tmem_ld_x32(s_addr + 96u, sb);
            max_chunk(sa, 2);
            tmem_ld_wait();
            tmem_ld_x32(s_addr, sa);  // first chunk of pass 2
            max_chunk(sb, 3);
            const float bm = fmaxf(fmaxf(bm4[0], bm4[1]), fmaxf(bm4[2], bm4[3]));
            const float m_cand = fmaxf(m, bm * p.scale_log2);
            // raise the reference maximum only when it moved by more than 8 (a factor 256 of headroom)
            const bool raise = m_cand > m + 8.0f;  // also true on the first block (m = -inf) when any key is visible
            if (__any_sync(0xffffffffu, raise)) {
                const float m_new = raise ? m_cand : m;
                const float f = raise ? ex2(m - m_new) : 1.0f;  // 0 when m = -inf
                if (j > 0) {
                    // S_t of this block is complete, hence the previous P V has finished: O_t is quiescent
#pragma unroll
                    for (int c = 0; c < D / 32; c++) {
                        uint32_t o[32];
                        tmem_ld_x32(o_addr + uint32_t(c) * 32u, o);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
                        tmem_st_x32(o_addr + uint32_t(c) * 32u, o);
                    }
                    tmem_st_wait();
                }
                l *= f;
                m = m_new;
            }
            const float m_ref = (m == -INFINITY) ? 0.f : m;
            float bl4[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t pk_lo[SPLIT ? 64 : 1];  // low parts wait in registers: their columns still hold unread scores
            auto exp_chunk = [&](const uint32_t (&sv)[32], int c) {
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    // two scores per instruction for the scaling and for the row sum (packed fp32 pairs, sm_100): the softmax
                    // warps are bound by instruction issue, not by the exponential unit
                    float a0, a1;
                    fma2(a0, a1, __uint_as_float(sv[2 * i]), __uint_as_float(sv[2 * i + 1]), p.scale_log2, -m_ref);
                    float x0 = ex2(a0);
                    float x1 = ex2(a1);
                    if (MASK) {
                        if (c * 32 + 2 * i > visible) x0 = 0.f;
                        if (c * 32 + 2 * i + 1 > visible) x1 = 0.f;
                    }
                    add2(bl4[(i & 1) * 2], bl4[(i & 1) * 2 + 1], x0, x1);
                    pk[i] = pack2<IS_BF16>(x0, x1);
                    if (SPLIT) {
                        const float h0 = __uint_as_float(pk[i] << 16), h1 = __uint_as_float(pk[i] & 0xffff0000u);
                        pk_lo[c * 16 + i] = pack2<true>(x0 - h0, x1 - h1);
                    }
                }
                // keys 32c..32c+31 -> columns 16c..16c+15 of S_t (already consumed: they held keys < 32(c/2+1))
                tmem_st_x16(s_addr + uint32_t(c) * 16u, pk);
            };
            // Pass 2, same two-deep pipeline (chunk 0 was requested at the end of pass 1; the rescale branch
            // above waited for it if it ran, which is harmless).
            tmem_ld_wait();
            tmem_ld_x32(s_addr + 32u, sb);
            exp_chunk(sa, 0);
            tmem_ld_wait();
            tmem_ld_x32(s_addr + 64u, sa);
            exp_chunk(sb, 1);
            tmem_ld_wait();
            tmem_ld_x32(s_addr + 96u, sb);
            exp_chunk(sa, 2);
            tmem_ld_wait();
            exp_chunk(sb, 3);
            if (SPLIT) {
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    uint32_t part[16];
#pragma unroll
                    for (int i = 0; i < 16; i++) part[i] = pk_lo[c * 16 + i];
                    tmem_st_x16(s_addr + 64u + uint32_t(c) * 16u, part);
                }
            }
            l += (bl4[0] + bl4[1]) + (bl4[2] + bl4[3]);
            };
            if (need_mask) block_body(std::true_type{});
            else block_body(std::false_type{});
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full(t));
        }

        if (n_t > 0 && ok) {
            if (!mbar_wait(o_full(t), uint32_t(n_t - 1) & 1u)) {
                if (lane == 0) attn_timeout(p.status, 36);
                ok = false;
            }
            tc_fence_after();
        }
        using T = typename std::conditional<SPLIT, float, typename std::conditional<IS_BF16, __nv_bfloat16, __half>::type>::type;
        const float inv = l > 0.f ? 1.f / l : 0.f;
        T* optr = static_cast<T*>(p.O) + b * p.os_b + h * p.os_h + (long long)row * p.os_s;
        if (q0[t] < p.Sq) {
#pragma unroll
            for (int c = 0; c < D / 32; c++) {
                uint32_t o[32];
                if (n_t > 0 && ok) {
                    tmem_ld_x32(o_addr + uint32_t(c) * 32u, o);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i++) o[i] = 0u;
                }
                if (row < p.Sq && SPLIT) {
#pragma unroll
                    for (int v4 = 0; v4 < 8; v4++) {
                        float4 w;
                        w.x = __uint_as_float(o[v4 * 4 + 0]) * inv;
                        w.y = __uint_as_float(o[v4 * 4 + 1]) * inv;
                        w.z = __uint_as_float(o[v4 * 4 + 2]) * inv;
                        w.w = __uint_as_float(o[v4 * 4 + 3]) * inv;
                        *reinterpret_cast<float4*>(reinterpret_cast<float*>(optr) + c * 32 + v4 * 4) = w;
                    }
                } else if (row < p.Sq) {
#pragma unroll
                    for (int v4 = 0; v4 < 4; v4++) {
                        uint4 w;
                        w.x = pack2<IS_BF16>(__uint_as_float(o[v4 * 8 + 0]) * inv, __uint_as_float(o[v4 * 8 + 1]) * inv);
                        w.y = pack2<IS_BF16>(__uint_as_float(o[v4 * 8 + 2]) * inv, __uint_as_float(o[v4 * 8 + 3]) * inv);
                        w.z = pack2<IS_BF16>(__uint_as_float(o[v4 * 8 + 4]) * inv, __uint_as_float(o[v4 * 8 + 5]) * inv);
                        w.w = pack2<IS_BF16>(__uint_as_float(o[v4 * 8 + 6]) * inv, __uint_as_float(o[v4 * 8 + 7]) * inv);
                        *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(optr) + c * 32 + v4 * 8) = w;
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

template <int D, bool IS_BF16, bool SPLIT>
__global__ void __launch_bounds__(320, 1)
    attention_tc2p_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                         const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmQl,
                         const __grid_constant__ CUtensorMap tmKl, const __grid_constant__ CUtensorMap tmVl,
                         const AttnKernelParams p) {
    constexpr int DC = D / 64;
    constexpr uint32_t kTile = uint32_t(DC) * 16384u;
    constexpr int QP = SPLIT ? 2 : 1;  // planes per query tile
    constexpr int EB = SPLIT ? 4 : 2;  // ring entries per key block: K_hi, [K_lo], V_hi, [V_lo]
    constexpr int NS = attn2_slots(D, SPLIT);
    constexpr uint32_t kTmemCols = 512;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    const uint32_t sQ = base;                      // two query tiles (x hi/lo planes): tile t plane pl at (t*QP + pl)*kTile
    const uint32_t sKV = sQ + 2 * QP * kTile;      // NS ring slots
    const uint32_t bars = sKV + uint32_t(NS) * kTile;
    auto kv_full = [&](int i) { return bars + 8u * uint32_t(i); };
    auto kv_empty = [&](int i) { return bars + 64u + 8u * uint32_t(i); };
    auto q_full = [&](int t) { return bars + 128u + 8u * uint32_t(t); };
    auto s_full = [&](int t) { return bars + 144u + 8u * uint32_t(t); };
    auto p_full = [&](int t) { return bars + 160u + 8u * uint32_t(t); };
    auto o_full = [&](int t) { return bars + 176u + 8u * uint32_t(t); };
    auto q_empty = [&](int t) { return bars + 192u + 8u * uint32_t(t); };  // issuer -> producer: Q_t may be overwritten
    auto o_empty = [&](int t) { return bars + 208u + 8u * uint32_t(t); };  // softmax group -> issuer: O_t has been stored
    volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem_raw + (bars + 224u - raw_addr));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_pairs = (p.n_qtiles + 1) / 2;
    // work item = (batch, head, pair of query tiles). Without a mask every item costs the same and a CTA walks items
    // blockIdx.x, blockIdx.x + gridDim.x, ... Under a causal mask an item's cost grows with its pair index, so the items are
    // ordered heaviest first (all (batch, head) of the last pair, then of the pair before, ...) and dealt out in alternating
    // direction (CTA c takes position c of the even rounds and position G - 1 - c of the odd ones), which gives every CTA
    // about the same number of key blocks without any run-time scheduling.
    int q0[2], nb[2], n_max = 0, h = 0, b = 0;
    const int n_bh = p.n_items / n_pairs;
    auto item_of = [&](int k) {  // the CTA's k-th item, -1 when it has none left
        const int G = int(gridDim.x);
        const int pos = (p.causal && (k & 1)) ? G - 1 - int(blockIdx.x) : int(blockIdx.x);
        const long long L = (long long)k * G + pos;
        return L < p.n_items ? int(L) : -1;
    };
    auto set_item = [&](int item) {
        const int pair = p.causal ? n_pairs - 1 - item / n_bh : item % n_pairs;
        const int bh = p.causal ? item % n_bh : item / n_pairs;
        h = bh % p.H;
        b = bh / p.H;
        for (int t = 0; t < 2; t++) {
            q0[t] = (pair * 2 + t) * kBQ;
            int kv_end = p.Skv;
            if (p.causal) {
                const int last = q0[t] + kBQ - 1 + p.causal_off;  // last key visible to the last row of the tile
                kv_end = last + 1 < p.Skv ? last + 1 : p.Skv;
                if (kv_end < 0) kv_end = 0;
            }
            nb[t] = q0[t] < p.Sq ? (kv_end + kBKV - 1) / kBKV : 0;
        }
        n_max = nb[0] > nb[1] ? nb[0] : nb[1];
    };

    if (warp == 0 && lane == 0) {
        for (int i = 0; i < NS; i++) {
            mbar_init(kv_full(i), 1);
            mbar_init(kv_empty(i), 1);
        }
        for (int t = 0; t < 2; t++) {
            mbar_init(q_full(t), 1);
            mbar_init(s_full(t), 1);
            mbar_init(p_full(t), 4);
            mbar_init(o_full(t), 1);
            mbar_init(q_empty(t), 1);
            mbar_init(o_empty(t), 4);
        }
        fence_barrier_init();
        prefetch_tensormap(&tmQ);
        prefetch_tensormap(&tmK);
        prefetch_tensormap(&tmV);
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

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
          uint32_t ring = 0;          // ring entries issued so far (the ring runs on across items)
          uint32_t q_use[2] = {0, 0};  // items in which tile t was active so far
          bool alive = true;
          for (int k = 0; alive; k++) {
            const int item = item_of(k);
            if (item < 0) break;
            set_item(item);
            for (int t = 0; t < 2; t++) {
                if (nb[t] == 0) continue;
                // the previous item's last Q K^T of this tile has read the old Q_t
                if (!mbar_wait(q_empty(t), (q_use[t] & 1u) ^ 1u)) { attn_timeout(p.status, 38); alive = false; break; }
                q_use[t]++;
                mbar_arrive_expect_tx(q_full(t), QP * kTile);
                for (int pl = 0; pl < QP; pl++)
                    for (int c = 0; c < DC; c++)
                        tma_load_4d(sQ + uint32_t(t * QP + pl) * kTile + uint32_t(c) * 16384u, pl ? &tmQl : &tmQ, q_full(t), c * 64, q0[t], h, b);
            }
            for (int i = 0; i < EB * n_max && alive; i++, ring++) {  // entry e = i % EB of block j = i / EB
                const int s = int(ring % uint32_t(NS));
                const uint32_t ph = (ring / uint32_t(NS)) & 1u;
                if (!mbar_wait(kv_empty(s), ph ^ 1u)) { attn_timeout(p.status, 31); alive = false; break; }
                mbar_arrive_expect_tx(kv_full(s), kTile);
                const int e = i % EB;
                const CUtensorMap* m = SPLIT ? (e == 0 ? &tmK : e == 1 ? &tmKl : e == 2 ? &tmV : &tmVl) : (e ? &tmV : &tmK);
                for (int c = 0; c < DC; c++)
                    tma_load_4d(sKV + uint32_t(s) * kTile + uint32_t(c) * 16384u, m, kv_full(s), c * 64, (i / EB) * kBKV, h, b);
            }
          }
        }
    } else if (warp == 1) {
        // ---------------- UMMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc_qk = make_idesc(kBQ, kBKV, IS_BF16 ? 1 : 0, 0, 0);
            constexpr uint32_t idesc_pv = make_idesc(kBQ, D, IS_BF16 ? 1 : 0, 0, 1);
            bool ok = true;
            uint32_t q_use[2] = {0, 0}, p_cnt[2] = {0, 0};  // items with tile t active / P_t blocks consumed so far
            // The ring's entries are consumed strictly in the order they were produced (K of block 0, then V of block j and K
            // of block j + 1 for every j), across items: the next entry's slot and phase are kept as a counter, not derived
            // from the entry number by divisions (scalar work of this one thread sits on the tensor pipe's critical path).
            uint32_t rs = 0, rph = 0;
            auto take_slot = [&](uint32_t& idx) -> uint32_t {  // waits for the next entry: its slot index, and its base (0 on timeout)
                idx = rs;
                if (!mbar_wait(kv_full(int(rs)), rph)) { attn_timeout(p.status, 32); ok = false; return 0u; }
                tc_fence_after();
                const uint32_t slot_base = sKV + rs * kTile;
                if (++rs == uint32_t(NS)) {
                    rs = 0;
                    rph ^= 1u;
                }
                return slot_base;
            };
            // Q K^T of tile t: hi*hi, plus the two cross terms for fp32 operands (small terms first)
            // Descriptors are built once per operand tile; the k-steps only add a constant to the address
            // field (16-byte units), which keeps the issuing thread ahead of the tensor pipe.
            auto issue_qk = [&](int t, uint32_t kb_hi, uint32_t kb_lo) {
                const uint32_t d_tmem = tmem_base + uint32_t(t) * 128u;
                const uint64_t q_hi = make_smem_desc(sQ + uint32_t(t * QP) * kTile, 16u, 1024u);
                const uint64_t q_lo = q_hi + uint64_t(kTile >> 4);
                uint32_t acc = 0;
                auto product = [&](uint64_t qd, uint32_t kb) {
                    const uint64_t kd = make_smem_desc(kb, 16u, 1024u);
#pragma unroll
                    for (int kk = 0; kk < D / 16; kk++) {
                        const uint64_t off = uint64_t((uint32_t(kk / 4) * 16384u + uint32_t(kk % 4) * 32u) >> 4);
                        umma_f16_ss(d_tmem, qd + off, kd + off, idesc_qk, acc);
                        acc = 1;
                    }
                };
                if (SPLIT) {
                    product(q_lo, kb_hi);
                    product(q_hi, kb_lo);
                }
                product(q_hi, kb_hi);
                umma_commit(s_full(t));
            };
          for (int k = 0; ok; k++) {
            const int item = item_of(k);
            if (item < 0) break;
            set_item(item);
            for (int t = 0; t < 2 && ok; t++) {
                if (nb[t] == 0) continue;
                if (!mbar_wait(q_full(t), q_use[t] & 1u)) { attn_timeout(p.status, 33); ok = false; }
            }
            if (ok) {
                uint32_t i_k0 = 0, i_k1 = 0;
                const uint32_t k_hi = take_slot(i_k0);
                const uint32_t k_lo = (SPLIT && ok) ? take_slot(i_k1) : 0u;
                if (ok) {
                    for (int t = 0; t < 2; t++) {
                        if (nb[t] == 0) continue;
                        issue_qk(t, k_hi, k_lo);
                        if (nb[t] == 1) umma_commit(q_empty(t));  // that was this item's last read of Q_t
                    }
                    umma_commit(kv_empty(int(i_k0)));
                    if (SPLIT) umma_commit(kv_empty(int(i_k1)));
                }
            }
            for (int j = 0; j < n_max && ok; j++) {
                uint32_t i_v0 = 0, i_v1 = 0, i_k0 = 0, i_k1 = 0;  // slots of V of block j and K of block j + 1
                const uint32_t v_hi = take_slot(i_v0);
                if (!ok) break;
                const uint32_t v_lo = SPLIT ? take_slot(i_v1) : 0u;
                if (!ok) break;
                uint32_t k_hi = 0, k_lo = 0;
                if (j + 1 < n_max) {
                    k_hi = take_slot(i_k0);
                    if (!ok) break;
                    if (SPLIT) k_lo = take_slot(i_k1);
                    if (!ok) break;
                }
                for (int t = 0; t < 2 && ok; t++) {
                    if (j >= nb[t]) continue;
                    // the previous item's O_t must have left tensor memory before this item's first P V overwrites it
                    if (j == 0 && !mbar_wait(o_empty(t), (q_use[t] & 1u) ^ 1u)) { attn_timeout(p.status, 39); ok = false; break; }
                    if (!mbar_wait(p_full(t), p_cnt[t] & 1u)) { attn_timeout(p.status, 34); ok = false; break; }
                    p_cnt[t]++;
                    tc_fence_after();
                    const uint32_t o_tmem = tmem_base + 256u + uint32_t(t) * 128u;
                    const uint32_t p_hi = tmem_base + uint32_t(t) * 128u;  // P_t over the first 64 columns of S_t
                    const uint32_t p_lo = p_hi + 64u;                       // (fp32 path) low part over the last 64
                    uint32_t acc = j > 0 ? 1u : 0u;
                    auto product = [&](uint32_t pa, uint32_t vb) {
                        const uint64_t vd = make_smem_desc(vb, 16384u, 1024u);
#pragma unroll
                        for (int kk = 0; kk < kBKV / 16; kk++) {
                            umma_f16_ts(o_tmem, pa + uint32_t(kk) * 8u, vd + uint64_t(kk * (2048 / 16)), idesc_pv, acc);
                            acc = 1;
                        }
                    };
                    if (SPLIT) {
                        product(p_lo, v_hi);
                        product(p_hi, v_lo);
                    }
                    product(p_hi, v_hi);
                    umma_commit(o_full(t));
                    if (j + 1 < nb[t]) {
                        issue_qk(t, k_hi, k_lo);
                        if (j + 2 == nb[t]) umma_commit(q_empty(t));
                    }
                }
                if (!ok) break;
                umma_commit(kv_empty(int(i_v0)));
                if (SPLIT) umma_commit(kv_empty(int(i_v1)));
                if (j + 1 < n_max) {
                    umma_commit(kv_empty(int(i_k0)));
                    if (SPLIT) umma_commit(kv_empty(int(i_k1)));
                }
            }
            for (int t = 0; t < 2; t++) if (nb[t] > 0) q_use[t]++;
          }
        }
    } else {
        // ---------------- softmax groups ----------------
        const int t = (warp - 2) >> 2;
        const int quad = warp & 3;
        const int r = quad * 32 + lane;
        const uint32_t lane_addr = tmem_base + (uint32_t(quad * 32) << 16);
        const uint32_t s_addr = lane_addr + uint32_t(t) * 128u;
        const uint32_t o_addr = lane_addr + 256u + uint32_t(t) * 128u;
        bool ok = true;
        uint32_t s_cnt = 0, o_cnt = 0;  // score blocks consumed / P V products awaited so far (all items)
      for (int k = 0; ok; k++) {
        const int item = item_of(k);
        if (item < 0) break;
        set_item(item);
        const int row = q0[t] + r;
        const int n_t = nb[t];
        if (n_t == 0) continue;  // odd tile count: the second tile of the last pair does not exist
        float m = -INFINITY;  // maximum the stored exponentials are relative to
        float l = 0.f;
        const int row_limit = p.causal ? row + p.causal_off : p.Skv - 1;  // last visible key of this row

        for (int j = 0; j < n_t && ok; j++) {
            const int k0 = j * kBKV;
            if (!mbar_wait(s_full(t), s_cnt & 1u)) {
                if (lane == 0) attn_timeout(p.status, 35);
                ok = false;
                break;
            }
            tc_fence_after();
            s_cnt++;
            const bool need_mask = (k0 + kBKV > p.Skv) || (p.causal && k0 + kBKV - 1 > q0[t] + p.causal_off);
            const int visible = (row_limit < p.Skv - 1 ? row_limit : p.Skv - 1) - k0;
            // The block body exists twice, with and without masking: the mask test is uniform over the warp, and as a
            // run-time condition inside the loops it costs two compare/select instructions per score on every block.
            auto block_body = [&](auto mask_c) {
            constexpr bool MASK = decltype(mask_c)::value;
            // Pass 1 (block maximum) with two chunk loads in flight: the next 32 columns are requested
            // before the current ones are reduced, so the TMEM read latency overlaps the arithmetic.
            // four independent running maxima / sums: a single chain of 128 dependent operations would
            // leave the two warps per scheduler waiting on arithmetic latency
            float bm4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            uint32_t sa[32], sb[32];
            auto max_chunk = [&](const uint32_t (&sv)[32], int c) {
                if (MASK) {
#pragma unroll
                    for (int i = 0; i < 32; i++)
                        if (c * 32 + i <= visible) bm4[i & 3] = fmaxf(bm4[i & 3], __uint_as_float(sv[i]));
                } else {
#pragma unroll
                    for (int i = 0; i < 16; i++) bm4[i & 3] = max3(bm4[i & 3], __uint_as_float(sv[2 * i]), __uint_as_float(sv[2 * i + 1]));
                }
            };
            tmem_ld_x32(s_addr, sa);
            tmem_ld_wait();
            tmem_ld_x32(s_addr + 32u, sb);
            max_chunk(sa, 0);
            tmem_ld_wait();
            tmem_ld_x32(s_addr + 64u, sa);
            max_chunk(sb, 1);
            tmem_ld_wait();
            tmem_ld_x32(s_addr + 96u, sb);
            max_chunk(sa, 2);
            tmem_ld_wait();
            tmem_ld_x32(s_addr, sa);  // first chunk of pass 2
            max_chunk(sb, 3);
            const float bm = fmaxf(fmaxf(bm4[0], bm4[1]), fmaxf(bm4[2], bm4[3]));
            const float m_cand = fmaxf(m, bm * p.scale_log2);
            // raise the reference maximum only when it moved by more than 8 (a factor 256 of headroom)
            const bool raise = m_cand > m + 8.0f;  // also true on the first block (m = -inf) when any key is visible
            if (__any_sync(0xffffffffu, raise)) {
                const float m_new = raise ? m_cand : m;
                const float f = raise ? ex2(m - m_new) : 1.0f;  // 0 when m = -inf
                if (j > 0) {
                    // S_t of this block is complete, hence the previous P V has finished: O_t is quiescent
#pragma unroll
                    for (int c = 0; c < D / 32; c++) {
                        uint32_t o[32];
                        tmem_ld_x32(o_addr + uint32_t(c) * 32u, o);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
                        tmem_st_x32(o_addr + uint32_t(c) * 32u, o);
                    }
                    tmem_st_wait();
                }
                l *= f;
                m = m_new;
            }
            const float m_ref = (m == -INFINITY) ? 0.f : m;
            float bl4[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t pk_lo[SPLIT ? 64 : 1];  // low parts wait in registers: their columns still hold unread scores
            auto exp_chunk = [&](const uint32_t (&sv)[32], int c) {
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    // two scores per instruction for the scaling and for the row sum (packed fp32 pairs, sm_100): the softmax
                    // warps are bound by instruction issue, not by the exponential unit
                    float a0, a1;
                    fma2(a0, a1, __uint_as_float(sv[2 * i]), __uint_as_float(sv[2 * i + 1]), p.scale_log2, -m_ref);
                    float x0 = ex2(a0);
                    float x1 = ex2(a1);
                    if (MASK) {
                        if (c * 32 + 2 * i > visible) x0 = 0.f;
                        if (c * 32 + 2 * i + 1 > visible) x1 = 0.f;
                    }
                    add2(bl4[(i & 1) * 2], bl4[(i & 1) * 2 + 1], x0, x1);
                    pk[i] = pack2<IS_BF16>(x0, x1);
                    if (SPLIT) {
                        const float h0 = __uint_as_float(pk[i] << 16), h1 = __uint_as_float(pk[i] & 0xffff0000u);
                        pk_lo[c * 16 + i] = pack2<true>(x0 - h0, x1 - h1);
                    }
                }
                // keys 32c..32c+31 -> columns 16c..16c+15 of S_t (already consumed: they held keys < 32(c/2+1))
                tmem_st_x16(s_addr + uint32_t(c) * 16u, pk);
            };
            // Pass 2, same two-deep pipeline (chunk 0 was requested at the end of pass 1; the rescale branch
            // above waited for it if it ran, which is harmless).
            tmem_ld_wait();
            tmem_ld_x32(s_addr + 32u, sb);
            exp_chunk(sa, 0);
            tmem_ld_wait();
            tmem_ld_x32(s_addr + 64u, sa);
            exp_chunk(sb, 1);
            tmem_ld_wait();
            tmem_ld_x32(s_addr + 96u, sb);
            exp_chunk(sa, 2);
            tmem_ld_wait();
            exp_chunk(sb, 3);
            if (SPLIT) {
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    uint32_t part[16];
#pragma unroll
                    for (int i = 0; i < 16; i++) part[i] = pk_lo[c * 16 + i];
                    tmem_st_x16(s_addr + 64u + uint32_t(c) * 16u, part);
                }
            }
            l += (bl4[0] + bl4[1]) + (bl4[2] + bl4[3]);
            };
            if (need_mask) block_body(std::true_type{});
            else block_body(std::false_type{});
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full(t));
        }

        if (ok) {
            if (!mbar_wait(o_full(t), (o_cnt + uint32_t(n_t - 1)) & 1u)) {
                if (lane == 0) attn_timeout(p.status, 36);
                ok = false;
            }
            tc_fence_after();
        }
        o_cnt += uint32_t(n_t);
        using T = typename std::conditional<SPLIT, float, typename std::conditional<IS_BF16, __nv_bfloat16, __half>::type>::type;
        const float inv = l > 0.f ? 1.f / l : 0.f;
        T* optr = static_cast<T*>(p.O) + b * p.os_b + h * p.os_h + (long long)row * p.os_s;
        if (q0[t] < p.Sq) {
#pragma unroll
            for (int c = 0; c < D / 32; c++) {
                uint32_t o[32];
                if (n_t > 0 && ok) {
                    tmem_ld_x32(o_addr + uint32_t(c) * 32u, o);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i++) o[i] = 0u;
                }
                if (row < p.Sq && SPLIT && p.O_hi) {
                    // the out-projection's operand planes: 32 values -> 64 bytes of each plane
                    const long long off = b * p.os_b + h * p.os_h + (long long)row * p.os_s + c * 32;
                    uint4* ph = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.O_hi) + off);
                    uint4* pl = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.O_lo) + off);
#pragma unroll
                    for (int v8 = 0; v8 < 4; v8++) {
                        uint32_t wh[4], wl[4];
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            const float x0 = __uint_as_float(o[v8 * 8 + 2 * e]) * inv, x1 = __uint_as_float(o[v8 * 8 + 2 * e + 1]) * inv;
                            wh[e] = pack2<true>(x0, x1);
                            const float h0 = __uint_as_float(wh[e] << 16), h1 = __uint_as_float(wh[e] & 0xffff0000u);
                            wl[e] = pack2<true>(x0 - h0, x1 - h1);
                        }
                        ph[v8] = make_uint4(wh[0], wh[1], wh[2], wh[3]);
                        pl[v8] = make_uint4(wl[0], wl[1], wl[2], wl[3]);
                    }
                } else if (row < p.Sq && SPLIT) {
#pragma unroll
                    for (int v4 = 0; v4 < 8; v4++) {
                        float4 w;
                        w.x = __uint_as_float(o[v4 * 4 + 0]) * inv;
                        w.y = __uint_as_float(o[v4 * 4 + 1]) * inv;
                        w.z = __uint_as_float(o[v4 * 4 + 2]) * inv;
                        w.w = __uint_as_float(o[v4 * 4 + 3]) * inv;
                        *reinterpret_cast<float4*>(reinterpret_cast<float*>(optr) + c * 32 + v4 * 4) = w;
                    }
                } else if (row < p.Sq) {
#pragma unroll
                    for (int v4 = 0; v4 < 4; v4++) {
                        uint4 w;
                        w.x = pack2<IS_BF16>(__uint_as_float(o[v4 * 8 + 0]) * inv, __uint_as_float(o[v4 * 8 + 1]) * inv);
                        w.y = pack2<IS_BF16>(__uint_as_float(o[v4 * 8 + 2]) * inv, __uint_as_float(o[v4 * 8 + 3]) * inv);
                        w.z = pack2<IS_BF16>(__uint_as_float(o[v4 * 8 + 4]) * inv, __uint_as_float(o[v4 * 8 + 5]) * inv);
                        w.w = pack2<IS_BF16>(__uint_as_float(o[v4 * 8 + 6]) * inv, __uint_as_float(o[v4 * 8 + 7]) * inv);
                        *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(optr) + c * 32 + v4 * 8) = w;
                    }
                }
            }
        }
        // O_t is in registers / memory: the next item's first P V may overwrite it
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(o_empty(t));
      }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

bool g_attr2_done[16][6] = {};

template <int D, bool IS_BF16, bool SPLIT>
int launch2(Ctx* ctx, const AttnProblem& p, const CUtensorMap* maps, const AttnKernelParams& kp, int slot) {
    constexpr int kTileBytes = (D / 64) * 16384;
    constexpr int NS = attn2_slots(D, SPLIT);
    constexpr size_t smem = size_t(kTileBytes) * (2 * (SPLIT ? 2 : 1) + NS) + 1024 + 256;
    auto kern = attention_tc2_kernel<D, IS_BF16, SPLIT>;
    if (!g_attr2_done[ctx->device & 15][slot]) {
        DOCC_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        g_attr2_done[ctx->device & 15][slot] = true;
    }
    const int64_t grid = p.B * p.H * ((kp.n_qtiles + 1) / 2);
    DOCC_CUDA_TRY(launch_pdl(kern, dim3(unsigned(grid)), dim3(320), smem, ctx->stream, maps[0], maps[1], maps[2], maps[3], maps[4], maps[5], kp));
    return after_launch(ctx, "attention_tc2_kernel");
}

// Persistent variant: one CTA per SM walks the work items, so tensor-memory allocation, barrier set-up,
// the first Q / K loads and the final store of O overlap the neighbouring items instead of costing every item its own
// prologue and epilogue (with S = 512 an item is only four key blocks long).
bool g_attr2p_done[16][6] = {};

template <int D, bool IS_BF16, bool SPLIT>
int launch2p(Ctx* ctx, const AttnProblem& p, const CUtensorMap* maps, AttnKernelParams kp, int slot) {
    constexpr int kTileBytes = (D / 64) * 16384;
    constexpr int NS = attn2_slots(D, SPLIT);
    constexpr size_t smem = size_t(kTileBytes) * (2 * (SPLIT ? 2 : 1) + NS) + 1024 + 256;
    auto kern = attention_tc2p_kernel<D, IS_BF16, SPLIT>;
    if (!g_attr2p_done[ctx->device & 15][slot]) {
        DOCC_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        g_attr2p_done[ctx->device & 15][slot] = true;
    }
    const int64_t items = p.B * p.H * ((kp.n_qtiles + 1) / 2);
    kp.n_items = int(items);
    const int64_t grid = items < ctx->sm_count ? items : ctx->sm_count;
    DOCC_CUDA_TRY(launch_pdl(kern, dim3(unsigned(grid)), dim3(320), smem, ctx->stream, maps[0], maps[1], maps[2], maps[3], maps[4], maps[5], kp));
    return after_launch(ctx, "attention_tc2p_kernel");
}

// fp32 [B,H,S,D] (strided, D contiguous) -> contiguous bf16 hi / lo planes.
__global__ void __launch_bounds__(256) split_heads_kernel(const float* __restrict__ X, long long sb, long long sh, long long ss,
                                                          int H, int S, int D, long long total4, __nv_bfloat16* __restrict__ hi,
                                                          __nv_bfloat16* __restrict__ lo) {
    griddep_wait();
    griddep_launch_dependents();
    const int d4 = D / 4;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total4; i += (long long)gridDim.x * blockDim.x) {
        const int dq = int(i % d4);
        long long r = i / d4;
        const int s = int(r % S); r /= S;
        const int h = int(r % H);
        const long long b = r / H;
        const float4 x = *reinterpret_cast<const float4*>(X + b * sb + h * sh + s * ss + dq * 4);
        const float xs[4] = {x.x, x.y, x.z, x.w};
        Pack<__nv_bfloat16, 4> ph, pl;
#pragma unroll
        for (int e = 0; e < 4; e++) {
            ph.v[e] = __float2bfloat16_rn(xs[e]);
            pl.v[e] = __float2bfloat16_rn(xs[e] - __bfloat162float(ph.v[e]));
        }
        *reinterpret_cast<Pack<__nv_bfloat16, 4>*>(hi + i * 4) = ph;
        *reinterpret_cast<Pack<__nv_bfloat16, 4>*>(lo + i * 4) = pl;
    }
}

bool g_attr_done[16][4] = {};

template <int D, bool IS_BF16>
int launch(Ctx* ctx, const AttnProblem& p, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
           const AttnKernelParams& kp, int slot) {
    constexpr size_t smem = size_t(D / 64) * 16384 * 5 + 32768 + 1024 + 256;
    auto kern = attention_tc_kernel<D, IS_BF16>;
    if (!g_attr_done[ctx->device & 15][slot]) {
        DOCC_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
        g_attr_done[ctx->device & 15][slot] = true;
    }
    const int64_t grid = p.B * p.H * kp.n_qtiles;
    DOCC_CUDA_TRY(launch_pdl(kern, dim3(unsigned(grid)), dim3(kAttnThreads), smem, ctx->stream, tq, tk, tv, kp));
    return after_launch(ctx, "attention_tc_kernel");
}

}  // namespace

int attention_tc(Ctx* ctx, const AttnProblem& p, const void* Q, const void* K, const void* V, void* O) {
    if (p.D != 64 && p.D != 128) return set_error(DOCC_B200_ERR_UNSUPPORTED, "attention_tc: head_dim %lld", (long long)p.D);
    if (p.Skv <= 0 || p.Sq <= 0) return set_error(DOCC_B200_ERR_UNSUPPORTED, "attention_tc: empty sequence");
    // the block maximum is taken before scaling, which needs a positive scale
    if (!(p.scale > 0.f)) return set_error(DOCC_B200_ERR_UNSUPPORTED, "attention_tc: non-positive scale");
    auto ok_strides = [](const void* ptr, const int64_t* s) {
        return reinterpret_cast<uintptr_t>(ptr) % 16 == 0 && s[0] % 8 == 0 && s[1] % 8 == 0 && s[2] % 8 == 0 && s[2] > 0;
    };
    if (!ok_strides(Q, p.qs) || !ok_strides(K, p.ks) || !ok_strides(V, p.vs) || !ok_strides(O, p.os))
        return set_error(DOCC_B200_ERR_UNSUPPORTED, "attention_tc: strides are not multiples of 16 bytes");
    if (p.B * p.H * ceil_div(p.Sq, kBQ) > 0x7fffffff || p.Sq > INT32_MAX / 2 || p.Skv > INT32_MAX / 2)
        return set_error(DOCC_B200_ERR_UNSUPPORTED, "attention_tc: extent too large");

    auto encode = [&](CUtensorMap* m, const void* ptr, const int64_t* s, int64_t S) -> int {
        // dims innermost first: D, S, H, B. A size-1 dim still needs a legal (16-byte multiple) stride.
        const uint64_t dims[4] = {uint64_t(p.D), uint64_t(S), uint64_t(p.H), uint64_t(p.B)};
        auto st = [&](int64_t v) { return uint64_t(v > 0 ? v : p.D) * 2; };
        const uint64_t strides[3] = {st(s[2]), st(s[1]), st(s[0])};
        const uint32_t box[4] = {64, 128, 1, 1};
        return encode_tmap_16bit(m, ptr, 4, dims, strides, box);
    };
    CUtensorMap tq, tk, tv;
    DOCC_TRY(encode(&tq, Q, p.qs, p.Sq));
    DOCC_TRY(encode(&tk, K, p.ks, p.Skv));
    DOCC_TRY(encode(&tv, V, p.vs, p.Skv));

    AttnKernelParams kp;
    kp.Sq = int(p.Sq); kp.Skv = int(p.Skv); kp.H = int(p.H);
    kp.n_qtiles = int(ceil_div(p.Sq, kBQ));
    kp.causal = p.causal;
    kp.causal_off = int(p.Skv - p.Sq);
    kp.scale_log2 = p.scale * 1.4426950408889634f;
    kp.O = O; kp.os_b = p.os[0]; kp.os_h = p.os[1]; kp.os_s = p.os[2];
    kp.O_hi = nullptr; kp.O_lo = nullptr;
    kp.status = ctx->status_dev;
    const bool bf = p.prec == DOCC_B200_PREC_B;
    static const bool single_tile = [] { const char* e = getenv("DOCC_B200_ATTENTION_SINGLE_TILE"); return e && e[0] == '1'; }();
    static const bool persistent = [] { const char* e = getenv("DOCC_B200_ATTENTION_PERSISTENT"); return !e || e[0] != '0'; }();
    // under a causal mask the persistent walk needs every query row to see at least one key (Skv >= Sq)
    static const bool persistent_causal = [] { const char* e = getenv("DOCC_B200_ATTENTION_PERSISTENT_CAUSAL"); return !e || e[0] != '0'; }();
    const bool walk = persistent && (!p.causal || (persistent_causal && p.Skv >= p.Sq));
    if (!single_tile && p.Sq > kBQ && walk) {
        const CUtensorMap maps[6] = {tq, tk, tv, tq, tk, tv};
        if (p.D == 128) return bf ? launch2p<128, true, false>(ctx, p, maps, kp, 0) : launch2p<128, false, false>(ctx, p, maps, kp, 1);
        return bf ? launch2p<64, true, false>(ctx, p, maps, kp, 2) : launch2p<64, false, false>(ctx, p, maps, kp, 3);
    }
    if (!single_tile && p.Sq > kBQ) {
        const CUtensorMap maps[6] = {tq, tk, tv, tq, tk, tv};
        if (p.D == 128) return bf ? launch2<128, true, false>(ctx, p, maps, kp, 0) : launch2<128, false, false>(ctx, p, maps, kp, 1);
        return bf ? launch2<64, true, false>(ctx, p, maps, kp, 2) : launch2<64, false, false>(ctx, p, maps, kp, 3);
    }
    if (p.D == 128) return bf ? launch<128, true>(ctx, p, tq, tk, tv, kp, 0) : launch<128, false>(ctx, p, tq, tk, tv, kp, 1);
    return bf ? launch<64, true>(ctx, p, tq, tk, tv, kp, 2) : launch<64, false>(ctx, p, tq, tk, tv, kp, 3);
}

// fp32 attention on the tensor cores: operands split into bf16 hi/lo planes, three products per contraction.
int attention_tc_f32(Ctx* ctx, const AttnProblem& p, const void* Q, const void* K, const void* V, void* O) {
    if (p.D != 64) return set_error(DOCC_B200_ERR_UNSUPPORTED, "attention_tc_f32: head_dim %lld (64 only)", (long long)p.D);
    if (p.Skv <= 0 || p.Sq <= 0 || !(p.scale > 0.f)) return set_error(DOCC_B200_ERR_UNSUPPORTED, "attention_tc_f32: empty sequence or scale");
    auto ok_in = [](const void* ptr, const int64_t* s) {
        return reinterpret_cast<uintptr_t>(ptr) % 16 == 0 && s[0] % 4 == 0 && s[1] % 4 == 0 && s[2] % 4 == 0;
    };
    if (!ok_in(Q, p.qs) || !ok_in(K, p.ks) || !ok_in(V, p.vs) || !ok_in(O, p.os))
        return set_error(DOCC_B200_ERR_UNSUPPORTED, "attention_tc_f32: strides are not multiples of 16 bytes");
    if (p.B * p.H * ceil_div(p.Sq, kBQ) > 0x7fffffff || p.Sq > INT32_MAX / 2 || p.Skv > INT32_MAX / 2)
        return set_error(DOCC_B200_ERR_UNSUPPORTED, "attention_tc_f32: extent too large");
    const size_t nq = size_t(p.B * p.H * p.Sq * p.D), nk = size_t(p.B * p.H * p.Skv * p.D);
    void* ws;
    DOCC_TRY(get_workspace(ctx, 3, (2 * nq + 4 * nk) * sizeof(__nv_bfloat16), &ws));
    __nv_bfloat16* planes[6];  // q_hi, k_hi, v_hi, q_lo, k_lo, v_lo
    __nv_bfloat16* base = static_cast<__nv_bfloat16*>(ws);
    planes[0] = base; planes[3] = base + nq;
    planes[1] = base + 2 * nq; planes[4] = planes[1] + nk;
    planes[2] = planes[4] + nk; planes[5] = planes[2] + nk;
    const void* src[3] = {Q, K, V};
    const int64_t* str[3] = {p.qs, p.ks, p.vs};
    const int64_t seq[3] = {p.Sq, p.Skv, p.Skv};
    for (int i = 0; i < 3; i++) {
        const long long total4 = (long long)(p.B * p.H * seq[i] * p.D / 4);
        long long blocks = (total4 + 255) / 256;
        if (blocks > ctx->sm_count * 16) blocks = ctx->sm_count * 16;
        DOCC_CUDA_TRY(launch_pdl(split_heads_kernel, dim3(unsigned(blocks)), dim3(256), 0, ctx->stream, static_cast<const float*>(src[i]),
                                 (long long)str[i][0], (long long)str[i][1], (long long)str[i][2], int(p.H), int(seq[i]), int(p.D), total4,
                                 planes[i], planes[3 + i]));
        DOCC_TRY(after_launch(ctx, "split_heads_kernel"));
    }
    CUtensorMap maps[6];
    for (int i = 0; i < 6; i++) {
        const int64_t S = seq[i % 3];
        const uint64_t dims[4] = {uint64_t(p.D), uint64_t(S), uint64_t(p.H), uint64_t(p.B)};
        const uint64_t strides[3] = {uint64_t(p.D) * 2, uint64_t(S * p.D) * 2, uint64_t(p.H * S * p.D) * 2};
        const uint32_t box[4] = {64, 128, 1, 1};
        DOCC_TRY(encode_tmap_16bit(&maps[i], planes[i], 4, dims, strides, box));
    }
    AttnKernelParams kp;
    kp.Sq = int(p.Sq); kp.Skv = int(p.Skv); kp.H = int(p.H);
    kp.n_qtiles = int(ceil_div(p.Sq, kBQ));
    kp.causal = p.causal;
    kp.causal_off = int(p.Skv - p.Sq);
    kp.scale_log2 = p.scale * 1.4426950408889634f;
    kp.O = O; kp.os_b = p.os[0]; kp.os_h = p.os[1]; kp.os_s = p.os[2];
    kp.O_hi = nullptr; kp.O_lo = nullptr;
    kp.status = ctx->status_dev;
    static const bool persistent = [] { const char* e = getenv("DOCC_B200_ATTENTION_PERSISTENT"); return !e || e[0] != '0'; }();
    static const bool persistent_causal = [] { const char* e = getenv("DOCC_B200_ATTENTION_PERSISTENT_CAUSAL"); return !e || e[0] != '0'; }();
    if (persistent && (!p.causal || (persistent_causal && p.Skv >= p.Sq)) && p.Sq > kBQ) {
        // the caller's operand planes for what consumes O (16-byte stores: strides and bases as for the fp32 output)
        const bool planes = p.o_hi && p.o_lo && p.planes_done && reinterpret_cast<uintptr_t>(p.o_hi) % 16 == 0 &&
                            reinterpret_cast<uintptr_t>(p.o_lo) % 16 == 0 && p.os[0] % 8 == 0 && p.os[1] % 8 == 0 && p.os[2] % 8 == 0;
        if (planes) {
            kp.O_hi = p.o_hi;
            kp.O_lo = p.o_lo;
            *p.planes_done = true;
        }
        return launch2p<64, true, true>(ctx, p, maps, kp, 4);
    }
    return launch2<64, true, true>(ctx, p, maps, kp, 4);
}

}  // namespace docc_b200
