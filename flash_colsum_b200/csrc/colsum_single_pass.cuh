// Single-pass attention column mean for short key axes (S_k <= 2048, head
// dimension 64, non-causal), one thread-block cluster per stream of (batch, head)
// pairs.
//
// The two-pass kernels evaluate every score and every exp twice.  When the whole
// key axis fits a cluster of up to eight CTAs (256 keys each), one pass is enough:
//
//   S      = Q_tile K_slice^T            tcgen05 MMA, 128 queries x 256 keys, fp32 in tensor memory
//   P~     = exp2(c*S - m_g)             per thread (= query row) and 64-key group g, fp16 -> shared memory
//   (m, l) exchange                      per row: 4 groups in the CTA, then all CTAs of the cluster
//                                        through distributed shared memory (st.async + mbarrier
//                                        byte counts: nobody waits for a store to land)
//   w_g    = exp2(m_g - M) / L           the factor that turns P~ into softmax probabilities
//   D2    += P~^T W                      second MMA: contraction over the 128 query rows; W holds
//                                        w_g as two fp16 parts (hi + lo) in columns of a 16-wide
//                                        operand, so D2[key][2a], D2[key][2a+1] are the column
//                                        sums of the keys of 64-key group a of a key tile
//
// D2 lives in tensor memory across all query tiles and heads of a batch entry and
// is added to the output once per (cluster, batch entry).  P~ is double-buffered:
// the column-sum MMA of tile i runs while the consumers work on tiles i+1 and i+2,
// which is the time the statistics of tile i have to go around the cluster.
//
// Measured against the two-pass kernels (fp16, B = 32, H = 16): 1.2-1.3x at 400-1024
// keys, 1.07-1.14x at 1152-1536, 0.84x / 0.95x at 1792 / 2048 (only 15 clusters of seven
// or eight CTAs are resident at a time: 105 / 120 of the 148 SMs); key lengths that fill
// less than ~75 % of their cluster's slices lose to the padding.  The host side picks
// accordingly.
#pragma once

#include "colsum_math.cuh"
#include "schedule.h"
#include "sm100_ptx.cuh"

namespace fcs {

struct SinglePassParams {
    int B, H, Sq, Sk;
    int NQ;                 // 128-row query tiles
    int CL;                 // CTAs per cluster = 256-key slices (1 .. 8)
    int units;              // B * H
    int clusters;           // gridDim.x / CL
    int flush_units;        // most (batch, head) pairs accumulated in tensor memory before a flush
    float c;                // |scale| * log2(e)
    float out_scale;        // 1 / (h_norm * R * 2^10): the weights are stored times 2^10
    float* out;
    long long out_ld;
    int* status;
    uint32_t idesc_scores;  // 128 x 256 x 16, K-major operands
    uint32_t idesc_colsum;  // 128 x 16 x 16, A = P~ (M-major), B = W (K-major), fp16
};

namespace sp {

constexpr int CONSUMER_GROUPS = 4;
constexpr int CONSUMER_WARPS = 16;
constexpr int CONSUMER_THREADS = 512;
constexpr int HALF_THREADS = 256;          // consumers of one half (two groups)
constexpr int PRODUCER_WARP = 16;
constexpr int MMA_WARP = 17;
constexpr int XCHG_WARP = 18;
constexpr int XCHG_WARPS = 2;
constexpr int XCHG_ROWS_PER_WARP = 128 / XCHG_WARPS;
constexpr int XCHG_ROWS_PER_LANE = XCHG_ROWS_PER_WARP / 32;
constexpr int THREADS = 32 * (XCHG_WARP + XCHG_WARPS);
constexpr int MAX_CL = 8;
constexpr int TMEM_COLS = 512;
constexpr int D2_COL = 256;            // tensor-memory column of the column-sum accumulators
constexpr int W_N = 16;                // columns of the weight operand
constexpr float W_SCALE_LOG2 = 10.f;   // weights are stored times 2^10 to stay in the fp16 normal range

// shared memory (head dimension 64)
constexpr int K_BYTES = 256 * 128;                 // key slice: 256 rows of 128 bytes, 128-byte swizzle
constexpr int Q_BYTES = 128 * 128;                 // query tile
constexpr int P_TILE_BYTES = 128 * 128 * 2;        // P~ of one key tile: 128 keys x 128 query rows fp16
constexpr int P_BYTES = 2 * P_TILE_BYTES;          // both key tiles of the slice
constexpr int P_ATOM_COL_BYTES = 16 * 1024;        // 64 keys x 128 query rows
constexpr int W_TILE_BYTES = 8 * 512;              // 8 slabs of [16 columns][16 query rows]
constexpr int K_OFF = 0;
constexpr int Q_OFF = K_OFF + K_BYTES;             // two buffers
constexpr int P_OFF = Q_OFF + 2 * Q_BYTES;         // two buffers
constexpr int W_OFF = P_OFF + 2 * P_BYTES;         // one buffer: [2 key tiles][W_TILE_BYTES]
constexpr int XCHG_OFF = W_OFF + 2 * W_TILE_BYTES; // float2 [2][MAX_CL][128]: every CTA's (max, sum) per row
constexpr int LST_OFF = XCHG_OFF + 2 * MAX_CL * 128 * 8;   // float2 [2][groups][128]
constexpr int BAR_OFF = LST_OFF + 2 * CONSUMER_GROUPS * 128 * 8;
constexpr int NUM_BARS = 28;
constexpr int MISC_OFF = BAR_OFF + NUM_BARS * 8;
constexpr int TOTAL = MISC_OFF + 16;               // tensor-memory address, abort flag
constexpr int DYN_BYTES = TOTAL + 1024;
static_assert(DYN_BYTES <= 227 * 1024, "shared memory budget");

// ---------------------------------------------------------------- cluster helpers
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// The shared::cluster address of `addr` (a shared::cta address) in CTA `rank`.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
// Asynchronous store of two floats into another CTA's shared memory; its 8 bytes are
// counted on that CTA's barrier `mbar` when they have landed, so the sender neither
// waits nor fences.
__device__ __forceinline__ void st_async_f32x2(uint32_t addr, float a, float b, uint32_t mbar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v2.f32 [%0], {%1, %2}, [%3];"
                 ::"r"(addr), "f"(a), "f"(b), "r"(mbar)
                 : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(kSuspendHintNs)
        : "memory");
    return ok != 0;
}
// Bounded wait on a barrier that other CTAs of the cluster arrive on.
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                  int* status, int code) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const long long t0 = clock64();
    unsigned spins = 0;
    while (true) {
        if (mbar_try_wait_cluster(bar, parity)) return true;
        if ((++spins & 15u) == 0u) {
            if (*abort_flag) return false;
            if (clock64() - t0 > kWaitLimitCycles) {
                *abort_flag = 1;
                if (status) atomicCAS(status, 0, code);
                return false;
            }
        }
    }
}

// 32 lanes x 16 consecutive fp32 columns.
__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait16(uint32_t (&r)[16]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                   "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]),
                   "+r"(r[15])
                 :
                 : "memory");
}

// Shared-memory descriptor of an M-major operand tile (the M index is contiguous in
// memory) with the 128-byte swizzle: atoms of 64 M-elements (128 bytes) x 8 K-rows
// (1024 bytes); the next 64 M-elements are `P_ATOM_COL_BYTES` further (leading
// offset), the next 8 K-rows 1024 bytes further (stride offset).
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr) {
    const uint32_t lo = ((smem_addr >> 4) & 0x3FFFu) | ((uint32_t)(P_ATOM_COL_BYTES >> 4) << 16);
    const uint32_t hi = 64u | (1u << 14) | (2u << 29);
    return (static_cast<uint64_t>(hi) << 32) | lo;
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d)
                 : "memory");
}
__device__ __forceinline__ void st_shared_u16(uint32_t addr, unsigned short v) {
    asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"(v) : "memory");
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

__device__ __forceinline__ float max_of_32(const uint32_t (&r)[32]) {
    float m0 = max3(__uint_as_float(r[0]), __uint_as_float(r[1]), __uint_as_float(r[2]));
    float m1 = max3(__uint_as_float(r[3]), __uint_as_float(r[4]), __uint_as_float(r[5]));
    float m2 = max3(__uint_as_float(r[6]), __uint_as_float(r[7]), __uint_as_float(r[8]));
    float m3 = max3(__uint_as_float(r[9]), __uint_as_float(r[10]), __uint_as_float(r[11]));
#pragma unroll
    for (int j = 12; j < 28; j += 8) {
        m0 = max3(m0, __uint_as_float(r[j]), __uint_as_float(r[j + 1]));
        m1 = max3(m1, __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
        m2 = max3(m2, __uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
        m3 = max3(m3, __uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
    }
    m0 = max3(m0, __uint_as_float(r[28]), __uint_as_float(r[29]));
    m1 = max3(m1, __uint_as_float(r[30]), __uint_as_float(r[31]));
    return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
}

// exp2(c*s - m) of 8 scores -> four packed fp16 pairs; adds the fp32 values to `sum`.
// `pair0` is the index (mod 16) of the first pair in the exp-unit / polynomial pattern.
__device__ __forceinline__ void exp8_packed(int pair0, const uint32_t* s, f32x2 c2, f32x2 nm2, f32x2& sum0,
                                            f32x2& sum1, uint32_t* h) {
#pragma unroll
    for (int pr = 0; pr < 4; ++pr) {
        const f32x2 t = fma2(pack2(__uint_as_float(s[2 * pr]), __uint_as_float(s[2 * pr + 1])), c2, nm2);
        f32x2 e;
        float e0, e1;
        if (pair_uses_polynomial((pair0 + pr) & 15)) {
            e = ex2_poly2(t);
            unpack2(e, e0, e1);
        } else {
            unpack2(t, e0, e1);
            e0 = ex2_approx(e0);
            e1 = ex2_approx(e1);
            e = pack2(e0, e1);
        }
        if (pr & 1) sum1 = add2(sum1, e); else sum0 = add2(sum0, e);
        h[pr] = pack_half2(e0, e1);
    }
}

}  // namespace sp

// ---------------------------------------------------------------------------
// tm_q: boxes of 128 query rows, tm_k: boxes of 256 key rows (both 64 elements
// wide, 128-byte swizzle).  Grid = clusters * CL CTAs, launched with cluster
// dimension CL; CTA `rank` of a cluster owns keys [256*rank, 256*rank + 256).
//
// Roles in a CTA (20 warps):
//   16 consumer warps  four groups of 128 threads (thread = query row of the tile, group =
//                      64 key columns).  Groups 0,1 and groups 2,3 form two "halves" (the two
//                      128-key tiles of the slice), each with its own P~ buffers, column-sum
//                      accumulator and barriers for the second MMA; the scores of both halves
//                      come from one 128 x 256 MMA (separate score accumulators per half or
//                      per group were measured: no faster, more instructions to issue).
//   1 TMA warp         key slice per (batch, head), query tile per step.
//   1 MMA warp         scores(i), column sums(i-2) of both halves, scores(i+1), ...
//   2 exchange warps   64 rows each: combine the four groups' (max, sum) of a row, post the
//                      result to every CTA of the cluster, and when all CTAs' values are in,
//                      write the weights W of the four groups.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(sp::THREADS, 1)
colsum_single_pass_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                          const SinglePassParams p) {
    using namespace sp;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t k_smem = smem_base + K_OFF;
    const uint32_t q_smem = smem_base + Q_OFF;
    const uint32_t p_smem = smem_base + P_OFF;
    const uint32_t w_smem = smem_base + W_OFF;
    const uint32_t xchg_smem = smem_base + XCHG_OFF;
    const uint32_t bars = smem_base + BAR_OFF;
    // barriers; `hf` is the half (key tile of the slice), `s` a P~ / statistics slot
    const uint32_t k_full = bars, k_empty = bars + 8;
    auto q_full = [&](int s) { return bars + 8u * (2 + s); };
    auto q_empty = [&](int s) { return bars + 8u * (4 + s); };
    const uint32_t s_full = bars + 8u * 6, s_empty = bars + 8u * 8;   // the score accumulator (slots 7, 9 unused)
    auto stats_bar = [&](int s) { return bars + 8u * (10 + s); };
    auto xchg_bar = [&](int s) { return bars + 8u * (12 + s); };
    auto w_ready = [&](int s) { return bars + 8u * (14 + s); };
    auto p_ready = [&](int s, int hf) { return bars + 8u * (16 + 2 * s + hf); };
    auto pw_free = [&](int s, int hf) { return bars + 8u * (20 + 2 * s + hf); };
    auto d2_full = [&](int hf) { return bars + 8u * (24 + hf); };
    auto d2_empty = [&](int hf) { return bars + 8u * (26 + hf); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + MISC_OFF);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + MISC_OFF + 4);
    float2* lstats = reinterpret_cast<float2*>(smem + LST_OFF);
    const float2* xchg = reinterpret_cast<const float2*>(smem + XCHG_OFF);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int CL = p.CL;
    const int cluster_id = blockIdx.x / CL;
    const int NQ = p.NQ;
    // this cluster's share of the (batch, head, query tile) list
    TileRange range;
    range.init(p.units, NQ, cluster_id, p.clusters);
    const int u0 = range.u0, u1 = range.u1;
    auto t_lo = [&](int u) { return range.t_lo(u); };
    auto t_hi = [&](int u) { return range.t_hi(u); };

    if (threadIdx.x == 0) {
        mbar_init(k_full, 1); mbar_init(k_empty, 1);
        mbar_init(s_full, 1); mbar_init(s_empty, CONSUMER_THREADS);
        for (int i = 0; i < 2; ++i) {
            mbar_init(q_full(i), 1); mbar_init(q_empty(i), 1);
            mbar_init(stats_bar(i), CONSUMER_THREADS);
            mbar_init(xchg_bar(i), XCHG_WARPS);   // this CTA's exchange warps; the data counts as bytes
            mbar_init(w_ready(i), XCHG_WARPS * 32);
            for (int hf = 0; hf < 2; ++hf) {
                mbar_init(p_ready(i, hf), HALF_THREADS);
                mbar_init(pw_free(i, hf), 1);
            }
            mbar_init(d2_full(i), 1); mbar_init(d2_empty(i), HALF_THREADS);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    {   // the weight operand: only columns 0..3 are ever written, the rest stays zero
        uint4* w = reinterpret_cast<uint4*>(smem + W_OFF);
        for (int i = threadIdx.x; i < 2 * W_TILE_BYTES / 16; i += THREADS) w[i] = make_uint4(0u, 0u, 0u, 0u);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == PRODUCER_WARP && lane == 0) {
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_k);
    }
    if (warp == MMA_WARP) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // every CTA's barriers exist before a peer signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    auto wait_all = [&](uint32_t bar, uint32_t parity, int code) -> bool {
        const bool ok = mbar_wait(bar, parity, abort_flag, p.status, code);
        return __all_sync(0xffffffffu, ok);
    };
    // The column sums leave tensor memory at the end of a batch entry, of this cluster's range,
    // and every `flush_units` pairs: the tensor core truncates when it adds into its fp32
    // accumulator (about half a unit in the last place lost per accumulation), and the bound
    // keeps that bias below ~1e-4 of a column sum however many heads there are.
    auto last_of_batch = [&](int u) { return range.flush_after(u, p.H, p.flush_units); };

    if (warp == PRODUCER_WARP) {
        // ------------------------------------------------ TMA producer
        int i = 0, uc = 0;
        bool ok = true;
        for (int u = u0; ok && u < u1; ++u, ++uc) {
            const int b = u / p.H, h = u - b * p.H;
            if (!wait_all(k_empty, (uc & 1) ^ 1, FCS_STATUS_WAIT_PRODUCER)) break;
            if (elect_one_sync()) {
                mbar_arrive_expect_tx(k_full, K_BYTES);
                tma_load_4d(k_smem, &tm_k, k_full, 0, 256 * (int)rank, h, b);
            }
            __syncwarp();
            for (int t = t_lo(u); t < t_hi(u); ++t, ++i) {
                const int qs = i & 1;
                if (!wait_all(q_empty(qs), ((i >> 1) & 1) ^ 1, FCS_STATUS_WAIT_PRODUCER)) { ok = false; break; }
                if (elect_one_sync()) {
                    mbar_arrive_expect_tx(q_full(qs), Q_BYTES);
                    tma_load_4d(q_smem + qs * Q_BYTES, &tm_q, q_full(qs), 0, t * 128, h, b);
                }
                __syncwarp();
            }
        }
    } else if (warp >= XCHG_WARP) {
        // ------------------------------------------------ statistics exchange and weights
        const int xw = warp - XCHG_WARP;
        const int total = range.tiles();
        // (the query tile of the share's i-th tile, kept by counting: decoding it is a 64-bit
        // modulo, a hundred instructions in the warp every tile's exchange waits for)
        int t = total > 0 ? range.tile_of(0) : 0;
        for (int i = 0; i < total; ++i, t = (t + 1 == p.NQ) ? 0 : t + 1) {
            const int slot = i & 1;
            // (1) the four groups' (max, sum) of this CTA -> one pair per row, posted to every CTA
            if (!wait_all(stats_bar(slot), (i >> 1) & 1, FCS_STATUS_WAIT_CONSUMER)) break;
            float mg[XCHG_ROWS_PER_LANE][CONSUMER_GROUPS];
#pragma unroll
            for (int rr = 0; rr < XCHG_ROWS_PER_LANE; ++rr) {
                const int row = xw * XCHG_ROWS_PER_WARP + rr * 32 + lane;
                const float2* ls = lstats + slot * CONSUMER_GROUPS * 128 + row;
                float2 o[CONSUMER_GROUPS];
#pragma unroll
                for (int g = 0; g < CONSUMER_GROUPS; ++g) { o[g] = ls[g * 128]; mg[rr][g] = o[g].x; }
                const float mm = fmaxf(fmaxf(o[0].x, o[1].x), fmaxf(o[2].x, o[3].x));
                const float ms = (mm == -INFINITY) ? 0.f : mm;
                float ll = 0.f;
#pragma unroll
                for (int g = 0; g < CONSUMER_GROUPS; ++g) ll = fmaf(o[g].y, ex2_approx(o[g].x - ms), ll);
                const uint32_t dst = xchg_smem + (uint32_t)(((slot * MAX_CL + (int)rank) * 128 + row) * 8);
                for (int r = 0; r < CL; ++r)
                    st_async_f32x2(map_to_cta(dst, (uint32_t)r), mm, ll, map_to_cta(xchg_bar(slot), (uint32_t)r));
            }
            // what this CTA's own barrier will receive for this warp's rows: 8 bytes per row and CTA
            if (lane == 0) mbar_arrive_expect_tx(xchg_bar(slot), (uint32_t)(CL * XCHG_ROWS_PER_WARP * 8));

            // (2) every CTA's pair of the row -> the weights of this CTA's four groups
            bool good = mbar_wait_cluster(xchg_bar(slot), (i >> 1) & 1, abort_flag, p.status,
                                          FCS_STATUS_WAIT_CONSUMER);
            if (good && i > 0) {   // the MMAs that read W(i-1) must be done before W is rewritten
                good = mbar_wait(pw_free((i - 1) & 1, 0), ((i - 1) >> 1) & 1, abort_flag, p.status,
                                 FCS_STATUS_WAIT_CONSUMER) &&
                       mbar_wait(pw_free((i - 1) & 1, 1), ((i - 1) >> 1) & 1, abort_flag, p.status,
                                 FCS_STATUS_WAIT_CONSUMER);
            }
            if (!__all_sync(0xffffffffu, good)) break;
#pragma unroll
            for (int rr = 0; rr < XCHG_ROWS_PER_LANE; ++rr) {
                const int row = xw * XCHG_ROWS_PER_WARP + rr * 32 + lane;
                const float2* xs = xchg + slot * MAX_CL * 128 + row;
                float2 o[MAX_CL];
#pragma unroll
                for (int r = 0; r < MAX_CL; ++r) o[r] = (r < CL) ? xs[r * 128] : make_float2(-INFINITY, 0.f);
                const float M = fmaxf(fmaxf(fmaxf(o[0].x, o[1].x), fmaxf(o[2].x, o[3].x)),
                                      fmaxf(fmaxf(o[4].x, o[5].x), fmaxf(o[6].x, o[7].x)));
                float L = 0.f;
#pragma unroll
                for (int r = 0; r < MAX_CL; ++r) L = fmaf(o[r].y, ex2_approx(o[r].x - M), L);
                const float base = W_SCALE_LOG2 - M - __log2f(L);
                const bool live = t * 128 + row < p.Sq;   // rows past the end of the query axis weigh nothing
                // columns 2a (hi), 2a + 1 (lo) of half hf's operand belong to group 2*hf + a
                const uint32_t w_row = w_smem + (row >> 4) * 512 + (row & 15) * 2;
#pragma unroll
                for (int g = 0; g < CONSUMER_GROUPS; ++g) {
                    const float w = live ? ex2_approx(mg[rr][g] + base) : 0.f;
                    const __half w_hi = __float2half_rn(w);
                    const __half w_lo = __float2half_rn(w - __half2float(w_hi));
                    const uint32_t a = w_row + (g >> 1) * W_TILE_BYTES + (2 * (g & 1)) * 32;
                    st_shared_u16(a, __half_as_ushort(w_hi));
                    st_shared_u16(a + 32, __half_as_ushort(w_lo));
                }
            }
            mbar_arrive(w_ready(slot));   // (the MMA warps fence before the tensor core reads W)
        }
    } else if (warp == MMA_WARP) {
        // ------------------------------------------------ MMA issuer
        // Issue order: scores(i), column sums(i-2) of both halves, scores(i+1), ... -- the order
        // in which their inputs become ready: scores(i+1) when the consumers have read scores(i)
        // out of tensor memory, column sums(i-1) only after the statistics of tile i-1 have gone
        // around the cluster.
        int i = 0, uc = 0, fc = 0;
        int first = 0;                // first tile of the current batch entry on this CTA
        bool ok = true, fresh = true; // fresh: the next column-sum MMAs start a new accumulation
        // column sums of tile j: D2_hf (+)= P~_hf(j)^T W_hf(j)
        auto colsum_mma = [&](int j, bool last) -> bool {
            const int slot = j & 1;
            if (!wait_all(w_ready(slot), (j >> 1) & 1, FCS_STATUS_WAIT_MMA)) return false;
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                if (!wait_all(p_ready(slot, hf), (j >> 1) & 1, FCS_STATUS_WAIT_MMA)) return false;
                if (fresh && fc > 0) {   // the previous sums have been read out
                    if (!wait_all(d2_empty(hf), (fc - 1) & 1, FCS_STATUS_WAIT_MMA)) return false;
                }
                // P~ and W were written with ordinary stores by threads this warp has just
                // synchronised with; the fence orders them before the tensor core's reads
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                tc_fence_after();
                const uint64_t da = umma_desc_mn_sw128(p_smem + slot * P_BYTES + hf * P_TILE_BYTES);
                const uint64_t db = umma_desc_k_sw32(w_smem + hf * W_TILE_BYTES);
                if (elect_one_sync()) {
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks)   // 16 query rows per instruction
                        umma_f16(tmem_base + D2_COL + W_N * hf, da + (uint64_t)((ks * 2048) >> 4),
                                 db + (uint64_t)((ks * 512) >> 4), p.idesc_colsum, (fresh && ks == 0) ? 0u : 1u);
                    umma_commit(pw_free(slot, hf));
                    if (last) umma_commit(d2_full(hf));
                }
                __syncwarp();
            }
            fresh = false;
            return true;
        };
        for (int u = u0; ok && u < u1; ++u, ++uc) {
            if (!wait_all(k_full, uc & 1, FCS_STATUS_WAIT_MMA)) break;
            const int t_end = t_hi(u);
            for (int t = t_lo(u); t < t_end; ++t, ++i) {
                const int qs = i & 1;
                if (!wait_all(q_full(qs), (i >> 1) & 1, FCS_STATUS_WAIT_MMA)) { ok = false; break; }
                const uint64_t dq = umma_desc_k_sw128(q_smem + qs * Q_BYTES);
                {
                    if (!wait_all(s_empty, (i & 1) ^ 1, FCS_STATUS_WAIT_MMA)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t dk = umma_desc_k_sw128(k_smem);
                    if (elect_one_sync()) {
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks)
                            umma_f16(tmem_base, dq + (uint64_t)((ks * 32) >> 4),
                                     dk + (uint64_t)((ks * 32) >> 4), p.idesc_scores, ks > 0 ? 1u : 0u);
                        umma_commit(s_full);
                        umma_commit(q_empty(qs));
                        if (t + 1 == t_end) umma_commit(k_empty);
                    }
                    __syncwarp();
                }
                if (!ok) break;
                if (i - first >= 2) {
                    if (!colsum_mma(i - 2, false)) { ok = false; break; }
                }
            }
            if (!ok) break;
            if (last_of_batch(u)) {
                // drain: the last two tiles (or the only one)
                if (i - first >= 2 && !colsum_mma(i - 2, false)) break;
                if (!colsum_mma(i - 1, true)) break;
                first = i;
                fresh = true;
                ++fc;
            }
        }
    } else {
        // ------------------------------------------------ consumers
        const int wg = warp >> 2;                  // group: columns 64*wg .. 64*wg+63 of the scores
        const int hf = wg >> 1;                    // half = key tile of the slice
        const int half64 = wg & 1;                 // 64-key half of that key tile
        const int w4 = warp & 3;                   // 32-row block of the tile
        const int row = (w4 << 5) | lane;          // tensor-memory lane = query row of the tile
        const uint32_t lane_base = tmem_base + ((uint32_t)(w4 << 5) << 16);
        const float c = p.c;
        const int keys_valid = p.Sk - (256 * (int)rank + 64 * wg);   // >= 64: the whole group is real keys
        // this thread's 128-byte line of P~ (one line per query row and 64-key group)
        const uint32_t p_line = (uint32_t)(hf * P_TILE_BYTES + half64 * P_ATOM_COL_BYTES + (row >> 3) * 1024 +
                                           (row & 7) * 128);
        const uint32_t sw = (uint32_t)(row & 7);
        int i = 0, fc = 0;
        bool ok = true;
        for (int u = u0; ok && u < u1; ++u) {
            for (int t = t_lo(u); t < t_hi(u); ++t, ++i) {
                const int slot = i & 1;
                // ---- scores of this thread's row and group
                ok = mbar_wait(s_full, i & 1, abort_flag, p.status, FCS_STATUS_WAIT_CONSUMER);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                uint32_t sa[32], sb[32];   // columns 0..31 and 32..63 of the group
                tmem_ld_x32(lane_base + 64 * wg, sa);
                tmem_ld_x32(lane_base + 64 * wg + 32, sb);
                tmem_ld_wait(sa);
                tmem_ld_wait(sb);
                tc_fence_before();
                mbar_arrive(s_empty);

                // ---- P~ = exp2(c*s - m_g) as packed fp16
                uint32_t h[32];
                float m_g, l_g;
                if (keys_valid >= 64) {
                    m_g = fmaxf(max_of_32(sa), max_of_32(sb)) * c;
                    const f32x2 c2 = pack2(c, c), nm2 = pack2(-m_g, -m_g);
                    f32x2 sum0 = pack2(0.f, 0.f), sum1 = sum0;
#pragma unroll
                    for (int j8 = 0; j8 < 4; ++j8) exp8_packed(j8 * 4, &sa[8 * j8], c2, nm2, sum0, sum1, &h[4 * j8]);
#pragma unroll
                    for (int j8 = 0; j8 < 4; ++j8)
                        exp8_packed(j8 * 4, &sb[8 * j8], c2, nm2, sum0, sum1, &h[16 + 4 * j8]);
                    float x0, x1;
                    unpack2(add2(sum0, sum1), x0, x1);
                    l_g = x0 + x1;
                } else {
                    // ragged end of the key axis: keys past S_k (zero rows of the TMA box) are excluded
                    float cm = -INFINITY;
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        if (j < keys_valid) cm = fmaxf(cm, __uint_as_float(sa[j]));
                        if (j + 32 < keys_valid) cm = fmaxf(cm, __uint_as_float(sb[j]));
                    }
                    m_g = (cm == -INFINITY) ? -INFINITY : cm * c;
                    const float m_safe = (m_g == -INFINITY) ? 0.f : m_g;
                    float acc = 0.f;
#pragma unroll
                    for (int pr = 0; pr < 32; ++pr) {
                        const int j = 2 * pr;
                        const float s0 = __uint_as_float(pr < 16 ? sa[j & 31] : sb[j & 31]);
                        const float s1 = __uint_as_float(pr < 16 ? sa[(j + 1) & 31] : sb[(j + 1) & 31]);
                        float ta = fmaf(s0, c, -m_safe), tb = fmaf(s1, c, -m_safe);
                        ta = (j < keys_valid) ? ta : -INFINITY;       // c may be 0: select after the multiply
                        tb = (j + 1 < keys_valid) ? tb : -INFINITY;
                        const float ea = ex2_approx(ta), eb = ex2_approx(tb);
                        acc += ea + eb;
                        h[pr] = pack_half2(ea, eb);
                    }
                    l_g = acc;
                }
                // ---- tile i-2 is through: its column-sum MMA has read P~(i-2), and (before that)
                // the exchange warps have read its statistics -- both slots are free
                ok = mbar_wait(pw_free(slot, hf), ((i >> 1) & 1) ^ 1, abort_flag, p.status, FCS_STATUS_WAIT_CONSUMER);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                // ---- this group's (max, sum), for the exchange warps
                lstats[(slot * CONSUMER_GROUPS + wg) * 128 + row] = make_float2(m_g, l_g);
                mbar_arrive(stats_bar(slot));
                {
                    const uint32_t line = p_smem + slot * P_BYTES + p_line;
#pragma unroll
                    for (int j8 = 0; j8 < 8; ++j8)
                        st_shared_v4(line + ((((uint32_t)j8) ^ sw) << 4), h[4 * j8], h[4 * j8 + 1], h[4 * j8 + 2],
                                     h[4 * j8 + 3]);
                }
                // (the MMA warp makes these stores visible to the tensor core: it fences after its wait)
                mbar_arrive(p_ready(slot, hf));
            }
            if (!ok) break;
            if (last_of_batch(u)) {
                // ---- column sums of this batch entry -> output
                ok = mbar_wait(d2_full(hf), fc & 1, abort_flag, p.status, FCS_STATUS_WAIT_CONSUMER);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                if (half64 == 0) {
                    uint32_t d[16];
                    tmem_ld_x16(lane_base + D2_COL + W_N * hf, d);
                    tmem_ld_wait16(d);
                    const int b = u / p.H;
                    // lanes 0..63 hold keys of the first 64-key group (columns 0, 1), the rest columns 2, 3
                    const float v = (row >> 6) ? __uint_as_float(d[2]) + __uint_as_float(d[3])
                                               : __uint_as_float(d[0]) + __uint_as_float(d[1]);
                    const int key = 256 * (int)rank + 128 * hf + row;
                    if (key < p.Sk) atomicAdd_system(p.out + (long long)b * p.out_ld + key, v * p.out_scale);
                }
                tc_fence_before();
                mbar_arrive(d2_empty(hf));
                ++fc;
            }
        }
    }

    // ---------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // nobody leaves while a peer may still write into its shared memory
    if (warp == MMA_WARP) {
        if (*abort_flag) __nanosleep(1000000);   // let copies and MMAs in flight land
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

}  // namespace fcs
