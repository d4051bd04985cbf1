// Single-pass attention column mean for short key axes (S_k <= 2048, head
// dimension 64, non-causal), one thread-block cluster per (batch, head) stream.
//
// The two-pass kernels evaluate every score and every exp twice.  When the whole
// key axis fits a cluster of up to eight CTAs (256 keys each), one pass is enough:
//
//   S      = Q_tile K_slice^T            tcgen05 MMA, 128 queries x 256 keys, fp32 in tensor memory
//   P~     = exp2(c*S - m_g)             per thread (= query row) and 64-key group g, fp16 -> shared memory
//   (m, l) exchange                      per row: 4 groups in the CTA, then all CTAs of the cluster
//                                        through distributed shared memory
//   w_g    = exp2(m_g - M) / L           the factor that turns P~ into softmax probabilities
//   D2    += P~^T W                      second MMA: contraction over the 128 query rows; W holds
//                                        w_g as two fp16 parts (hi + lo) in columns of a 16-wide
//                                        operand, so D2[key][2a], D2[key][2a+1] are the column
//                                        sums of the keys of 64-key group a of a key tile
//
// D2 lives in tensor memory across all query tiles and heads of a batch entry and
// is added to the output once per (cluster, batch entry).
//
// Pipeline per CTA (i = running tile number):
//   MMA warp   : scores(i) as soon as the consumers have read scores(i-1) out of
//                tensor memory; column sums(i-1) once its P~ and W are in shared memory.
//   consumers  : read scores(i), write P~(i) and their (max, sum); finish tile i-1
//                (read the cluster's statistics, write W(i-1)); one group, a
//                different one every tile, combines the CTA's four partials and posts
//                them to every CTA of the cluster.
// Because tile i-1 is finished a whole tile after its statistics were posted, the
// exchange latency is off the critical path.
#pragma once

#include "colsum_math.cuh"
#include "sm100_ptx.cuh"

#ifndef FCS_SP_X
#define FCS_SP_X 0
#endif
#ifdef FCS_SP_TIMING
#define TICK(k) { const long long now_ = clock64(); tacc[k] += now_ - tlast; tlast = now_; }
#else
#define TICK(k)
#endif
namespace fcs {

struct SinglePassParams {
    int B, H, Sq, Sk;
    int NQ;                 // 128-row query tiles
    int CL;                 // CTAs per cluster = 256-key slices (1, 2, 4 or 8)
    int units;              // B * H
    int clusters;           // gridDim.x / CL
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
constexpr int PRODUCER_WARP = 16;
constexpr int MMA_WARP = 17;
constexpr int THREADS = 576;
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
constexpr int XCHG_OFF = W_OFF + 2 * W_TILE_BYTES; // float2 [2][MAX_CL][128]
constexpr int LST_OFF = XCHG_OFF + 2 * MAX_CL * 128 * 8;   // float2 [2][groups][128]
constexpr int BAR_OFF = LST_OFF + 2 * CONSUMER_GROUPS * 128 * 8;
constexpr int NUM_BARS = 16;
constexpr int MISC_OFF = BAR_OFF + NUM_BARS * 8;
constexpr int TOTAL = MISC_OFF + 16 + 32;   // tensor-memory address, abort flag, post counters
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
    const uint32_t k_full = bars, k_empty = bars + 8;
    auto q_full = [&](int i) { return bars + 8u * (2 + i); };
    auto q_empty = [&](int i) { return bars + 8u * (4 + i); };
    const uint32_t s_full = bars + 8 * 6, s_empty = bars + 8 * 7;
    auto xchg_bar = [&](int i) { return bars + 8u * (8 + i); };
    auto pw_ready = [&](int i) { return bars + 8u * (10 + i); };
    auto pw_free = [&](int i) { return bars + 8u * (12 + i); };
    const uint32_t d2_full = bars + 8 * 14, d2_empty = bars + 8 * 15;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + MISC_OFF);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + MISC_OFF + 4);
    int* post_count = reinterpret_cast<int*>(smem + MISC_OFF + 16);   // [2 slots][4 row blocks]
    float2* lstats = reinterpret_cast<float2*>(smem + LST_OFF);
    const float2* xchg = reinterpret_cast<const float2*>(smem + XCHG_OFF);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int CL = p.CL;
    const int cluster_id = blockIdx.x / CL;
    const int u0 = (int)((long long)p.units * cluster_id / p.clusters);
    const int u1 = (int)((long long)p.units * (cluster_id + 1) / p.clusters);

    if (threadIdx.x == 0) {
        mbar_init(k_full, 1); mbar_init(k_empty, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(q_full(i), 1); mbar_init(q_empty(i), 1);
            mbar_init(xchg_bar(i), 4);   // this CTA's four posting warps; the data counts as bytes
            mbar_init(pw_ready(i), CONSUMER_THREADS);
            mbar_init(pw_free(i), 1);
        }
        mbar_init(s_full, 1); mbar_init(s_empty, CONSUMER_THREADS);
        mbar_init(d2_full, 1); mbar_init(d2_empty, CONSUMER_THREADS);
        for (int i = 0; i < 8; ++i) post_count[i] = 0;
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
    auto last_of_batch = [&](int u) { return (u + 1 == u1) || ((u + 1) / p.H != u / p.H); };

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
            for (int t = 0; t < p.NQ; ++t, ++i) {
                const int qs = i & 1;
                if (!wait_all(q_empty(qs), ((i >> 1) & 1) ^ 1, FCS_STATUS_WAIT_PRODUCER)) { ok = false; break; }
                if (elect_one_sync()) {
                    mbar_arrive_expect_tx(q_full(qs), Q_BYTES);
                    tma_load_4d(q_smem + qs * Q_BYTES, &tm_q, q_full(qs), 0, t * 128, h, b);
                }
                __syncwarp();
            }
        }
    } else if (warp == MMA_WARP) {
        // ------------------------------------------------ MMA issuer
        // Issue order: scores(i), column sums(i-2), scores(i+1), ... -- the order in which
        // their inputs become ready (scores(i+1) when the consumers have read scores(i),
        // column sums(i-1) only when the consumers are through with tile i).
        int i = 0, uc = 0, fc = 0;
        int first = 0;                // first tile of the current batch entry on this CTA
        bool ok = true, d2_fresh = true;
#ifdef FCS_SP_TIMING
        long long tacc[8] = {0, 0, 0, 0, 0, 0, 0, 0}, tlast = clock64();
#endif
        // column sums of tile j: D2[kt] (+)= P~(j, kt)^T W(j, kt)
        auto colsum_mma = [&](int j, bool last) -> bool {
            const int slot = j & 1;
            TICK(7)
            if (!wait_all(pw_ready(slot), (j >> 1) & 1, FCS_STATUS_WAIT_MMA)) return false;
            TICK(4)
            if (d2_fresh && fc > 0) {   // the previous batch entry's sums have been read out
                if (!wait_all(d2_empty, (fc - 1) & 1, FCS_STATUS_WAIT_MMA)) return false;
            }
            tc_fence_after();
            if (elect_one_sync()) {
#pragma unroll
                for (int kt = 0; kt < 2; ++kt) {
                    const uint64_t da = umma_desc_mn_sw128(p_smem + slot * P_BYTES + kt * P_TILE_BYTES);
                    const uint64_t db = umma_desc_k_sw32(w_smem + kt * W_TILE_BYTES);
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks)   // 16 query rows per instruction
                        if (!(FCS_SP_X & 1)) umma_f16(tmem_base + D2_COL + W_N * kt, da + (uint64_t)((ks * 2048) >> 4),
                                 db + (uint64_t)((ks * 512) >> 4), p.idesc_colsum,
                                 (d2_fresh && ks == 0) ? 0u : 1u);
                }
                umma_commit(pw_free(slot));
                if (last) umma_commit(d2_full);
            }
            __syncwarp();
            TICK(5)
#ifdef FCS_SP_TIME_MMA2
            wait_all(pw_free(slot), (j >> 1) & 1, FCS_STATUS_WAIT_MMA);
            TICK(6)
#endif
            d2_fresh = false;
            return true;
        };
        for (int u = u0; ok && u < u1; ++u, ++uc) {
            TICK(7)
            if (!wait_all(k_full, uc & 1, FCS_STATUS_WAIT_MMA)) break;
            TICK(0)
            const uint64_t dk = umma_desc_k_sw128(k_smem);
            for (int t = 0; t < p.NQ; ++t, ++i) {
                const int qs = i & 1;
                TICK(7)
                if (!wait_all(q_full(qs), (i >> 1) & 1, FCS_STATUS_WAIT_MMA)) { ok = false; break; }
                TICK(1)
                if (!wait_all(s_empty, (i & 1) ^ 1, FCS_STATUS_WAIT_MMA)) { ok = false; break; }
                TICK(2)
                tc_fence_after();
                const uint64_t dq = umma_desc_k_sw128(q_smem + qs * Q_BYTES);
                if (elect_one_sync()) {
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks)
                        umma_f16(tmem_base, dq + (uint64_t)((ks * 32) >> 4), dk + (uint64_t)((ks * 32) >> 4),
                                 p.idesc_scores, ks > 0 ? 1u : 0u);
                    umma_commit(s_full);
                    umma_commit(q_empty(qs));
                    if (t + 1 == p.NQ) umma_commit(k_empty);
                }
                __syncwarp();
                TICK(3)
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
                d2_fresh = true;
                ++fc;
            }
        }
#ifdef FCS_SP_TIMING
        if (blockIdx.x == 0 && lane == 0)
            printf("mma tiles %d: k_full %lld q_full %lld s_empty %lld issue1 %lld pw_ready %lld issue2 %lld mma2-exec %lld other %lld\n",
                   i, tacc[0], tacc[1], tacc[2], tacc[3], tacc[4], tacc[5], tacc[6], tacc[7]);
#endif
    } else {
        // ------------------------------------------------ consumers
        const int wg = warp >> 2;                  // group: columns 64*wg .. 64*wg+63 of the scores
        const int w4 = warp & 3;                   // 32-row block of the tile
        const int row = (w4 << 5) | lane;          // tensor-memory lane = query row of the tile
        const uint32_t lane_base = tmem_base + ((uint32_t)(w4 << 5) << 16);
        const float c = p.c;
        const int kt = wg >> 1;                    // key tile of the slice, and 64-key half of it
        const int half64 = wg & 1;
        const int keys_valid = p.Sk - (256 * (int)rank + 64 * wg);   // >= 64: the whole group is real keys
        // this thread's 128-byte line of P~ (one line per query row and 64-key group)
        const uint32_t p_line = (uint32_t)(kt * P_TILE_BYTES + half64 * P_ATOM_COL_BYTES + (row >> 3) * 1024 +
                                           (row & 7) * 128);
        const uint32_t sw = (uint32_t)(row & 7);
        // this thread's two weight elements: columns 2*half64 (hi), 2*half64 + 1 (lo)
        const uint32_t w_addr = w_smem + kt * W_TILE_BYTES + (row >> 4) * 512 + (2 * half64) * 32 + (row & 15) * 2;
        int i = 0, fc = 0;
        bool ok = true, have_prev = false;
#ifdef FCS_SP_TIMING
        long long tacc[8] = {0, 0, 0, 0, 0, 0, 0, 0}, tlast = clock64();
#endif
        float m_prev = 0.f;
        int t_prev = 0;

        // Finish tile j: all CTAs' (max, sum) of the row -> this group's weight.
        auto finish_tile = [&](int j) -> bool {
            const int slot = j & 1;
            bool good = (FCS_SP_X & 2) ? true : mbar_wait_cluster(xchg_bar(slot), (j >> 1) & 1, abort_flag, p.status,
                                          FCS_STATUS_WAIT_CONSUMER);
            // the MMA that read W(j-1) must be done before W is rewritten
            if (good && j > 0)
                good = mbar_wait(pw_free((j - 1) & 1), ((j - 1) >> 1) & 1, abort_flag, p.status,
                                 FCS_STATUS_WAIT_CONSUMER);
            good = __all_sync(0xffffffffu, good);
            if (!good) return false;
            TICK(5)
            const float2* xs = xchg + slot * MAX_CL * 128 + row;
            float2 o[MAX_CL];
#pragma unroll
            for (int r = 0; r < MAX_CL; ++r) o[r] = (r < CL) ? xs[r * 128] : make_float2(-INFINITY, 0.f);
            float M = fmaxf(fmaxf(fmaxf(o[0].x, o[1].x), fmaxf(o[2].x, o[3].x)),
                            fmaxf(fmaxf(o[4].x, o[5].x), fmaxf(o[6].x, o[7].x)));
            float L = 0.f;
#pragma unroll
            for (int r = 0; r < MAX_CL; ++r) L = fmaf(o[r].y, ex2_approx(o[r].x - M), L);
            float w = ex2_approx(m_prev - M - __log2f(L) + W_SCALE_LOG2);
            if (t_prev * 128 + row >= p.Sq) w = 0.f;   // rows past the end of the query axis
            const __half w_hi = __float2half_rn(w);
            const __half w_lo = __float2half_rn(w - __half2float(w_hi));
            st_shared_u16(w_addr, __half_as_ushort(w_hi));
            st_shared_u16(w_addr + 32, __half_as_ushort(w_lo));
            TICK(6)
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P~ and W -> the MMA's view
            mbar_arrive(pw_ready(slot));
            TICK(7)
            return true;
        };

        for (int u = u0; ok && u < u1; ++u) {
            for (int t = 0; t < p.NQ; ++t, ++i) {
                const int slot = i & 1;
                // ---- scores of this thread's row and group
                ok = mbar_wait(s_full, i & 1, abort_flag, p.status, FCS_STATUS_WAIT_CONSUMER);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                TICK(0)
                tc_fence_after();
                uint32_t sa[32], sb[32];   // columns 0..31 and 32..63 of the group
                tmem_ld_x32(lane_base + 64 * wg, sa);
                tmem_ld_x32(lane_base + 64 * wg + 32, sb);
                tmem_ld_wait(sa);
                tmem_ld_wait(sb);
                tc_fence_before();
                mbar_arrive(s_empty);
                TICK(1)

                // ---- P~ = exp2(c*s - m_g) as packed fp16, kept in registers until its buffer is free
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
                TICK(2)
                // ---- finish the previous tile, whose statistics were posted a tile ago
                if (have_prev) { ok = finish_tile(i - 1); if (!ok) break; }

                // ---- this group's (max, sum); the last of the four groups to get here for a
                // block of 32 rows combines them and posts the result to every CTA of the cluster
                lstats[(slot * CONSUMER_GROUPS + wg) * 128 + row] = make_float2(m_g, l_g);
                __threadfence_block();
                __syncwarp();
                int arrived = 0;
                if (lane == 0) arrived = atomicAdd(&post_count[slot * 4 + w4], 1);
                arrived = __shfl_sync(0xffffffffu, arrived, 0);
                if (!(FCS_SP_X & 8) && arrived == CONSUMER_GROUPS - 1) {
                    if (lane == 0) post_count[slot * 4 + w4] = 0;
                    __threadfence_block();
                    const float2* ls = lstats + slot * CONSUMER_GROUPS * 128 + row;
                    float mm = -INFINITY;
#pragma unroll
                    for (int g = 0; g < CONSUMER_GROUPS; ++g) mm = fmaxf(mm, ls[g * 128].x);
                    const float ms = (mm == -INFINITY) ? 0.f : mm;
                    float ll = 0.f;
#pragma unroll
                    for (int g = 0; g < CONSUMER_GROUPS; ++g) {
                        const float2 o = ls[g * 128];
                        ll += o.y * ex2_approx(o.x - ms);
                    }
                    const uint32_t dst = xchg_smem + (uint32_t)(((slot * MAX_CL + (int)rank) * 128 + row) * 8);
                    for (int r = 0; r < CL; ++r)
                        st_async_f32x2(map_to_cta(dst, (uint32_t)r), mm, ll, map_to_cta(xchg_bar(slot), (uint32_t)r));
                    // what this CTA's own barrier will receive for these 32 rows: 8 bytes per row and CTA
                    if (lane == 0) mbar_arrive_expect_tx(xchg_bar(slot), (uint32_t)CL * 32u * 8u);
                }
                // ---- P~(i) may overwrite P~(i-2) once the MMA that read it is done
                ok = mbar_wait(pw_free(slot), ((i >> 1) & 1) ^ 1, abort_flag, p.status, FCS_STATUS_WAIT_CONSUMER);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                TICK(3)
                {
                    const uint32_t line = p_smem + slot * P_BYTES + p_line;
#pragma unroll
                    for (int j8 = 0; j8 < 8; ++j8)
                        if (!(FCS_SP_X & 4)) st_shared_v4(line + ((((uint32_t)j8) ^ sw) << 4), h[4 * j8], h[4 * j8 + 1], h[4 * j8 + 2],
                                     h[4 * j8 + 3]);
                }
                TICK(4)
                m_prev = m_g;
                t_prev = t;
                have_prev = true;
            }
            if (!ok) break;
            if (last_of_batch(u)) {
                ok = finish_tile(i - 1);
                if (!ok) break;
                have_prev = false;
                // ---- column sums of this batch entry -> output
                ok = mbar_wait(d2_full, fc & 1, abort_flag, p.status, FCS_STATUS_WAIT_CONSUMER);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                if (wg == 0) {
                    uint32_t d[32];
                    tmem_ld_x32(lane_base + D2_COL, d);
                    tmem_ld_wait(d);
                    const int b = u / p.H;
                    const int a = row >> 6;   // 64-key half of the tile this lane's key belongs to
#pragma unroll
                    for (int kk = 0; kk < 2; ++kk) {
                        const float v0 = __uint_as_float(d[W_N * kk]) + __uint_as_float(d[W_N * kk + 1]);
                        const float v1 = __uint_as_float(d[W_N * kk + 2]) + __uint_as_float(d[W_N * kk + 3]);
                        const int key = 256 * (int)rank + 128 * kk + row;
                        if (key < p.Sk)
                            atomicAdd_system(p.out + (long long)b * p.out_ld + key, (a ? v1 : v0) * p.out_scale);
                    }
                }
                tc_fence_before();
                mbar_arrive(d2_empty);
                ++fc;
            }
        }
#ifdef FCS_SP_TIMING
        if (blockIdx.x == 0 && lane == 0 && (warp & 3) == 0)
            printf("grp %d tiles %d: s_full %lld ld %lld math %lld post+pw_free %lld store %lld xchg-wait %lld weights %lld fence+arrive %lld\n",
                   wg, i, tacc[0], tacc[1], tacc[2], tacc[3], tacc[4], tacc[5], tacc[6], tacc[7]);
#endif
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
