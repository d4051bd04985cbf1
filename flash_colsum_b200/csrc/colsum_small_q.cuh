// Column mean when only a handful of query rows enter it (a CLS prefix, or a few
// decode queries): per (batch, head) the work is R dot products per key, i.e. a
// matrix-vector product that reads every key once.  That is bound by HBM, not by
// the tensor cores, so it is not reshaped into a GEMM; what matters is that every
// SM streams keys without pause.
//
//   * Few units over long key axes (a decode query over 32 heads): persistent CTAs, one per
//     SM, grouped into thread-block clusters of 1..8.  A cluster walks a list of (batch, head)
//     units; CTA r of the cluster owns the r-th range of every unit's key axis.  The cluster
//     size is the one with which the busiest CTA has the least to read (32 heads over 32768
//     keys: clusters of four, 128 CTAs of 2 MiB each).
//   * Many short units (a CLS call over 512 units of 74 KB): four CTAs per SM, one unit each,
//     no cut -- the units in flight on an SM hide each other's latency chains.
//   * One warp per CTA issues bulk asynchronous copies (cp.async.bulk, completion counted on an
//     mbarrier -- no tensor map, no multicast) of 16 KiB runs of key rows into a ring of up to
//     ten shared-memory stages, and runs ahead of the consumers across unit boundaries.  (One
//     such warp moves 33-35 GB/s per SM whatever the ring depth -- measured with the scoring
//     switched off -- which is what bounds the long-key form.)
//   * The consumer warps compute the scores of a unit's range as the stages land: a warp takes
//     32 rows, D/8 lanes per row over D/8 passes, then transposes and adds the partial dot
//     products with D/8 - 1 shuffles, after which every lane holds one row's score.  Scores stay
//     in shared memory; a running (maximum, sum) per thread is merged once per unit and posted
//     into every CTA of the cluster with st.async, counted on the receiver's mbarrier -- no
//     cluster-wide barrier per unit.  A unit is finished (weights, one add per key into the
//     output) one unit late, behind the scores of the next, when every range's values are in.
//   * The output is cleared by a small kernel launched just before; this kernel is a
//     programmatic dependent of it and waits for it only before its first add, so the
//     clear costs no time on the device.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../../include/flash_colsum_b200.h"
#include "sm100_ptx.cuh"

namespace fcs {

constexpr int SMALLQ_MAX_ROWS = 4;
constexpr int SMALLQ_CONSUMER_WARPS = 8;     // most consumer warps of a CTA (+ one warp that issues the copies)
constexpr int SMALLQ_WIDE_WARPS = 4;         // consumer warps of a CTA when four CTAs share an SM
constexpr int SMALLQ_WIDE_STAGES = 3;        // ... and their ring
constexpr int SMALLQ_STAGE_BYTES = 16 * 1024;
constexpr int SMALLQ_MAX_STAGES = 10;
constexpr int SMALLQ_MIN_STAGES = 3;
constexpr int SMALLQ_MAX_CLUSTER = 8;
constexpr size_t SMALLQ_MAX_SMEM = 200 * 1024;

struct SmallQParams {
    const void* q;
    const void* k;
    float* out;
    long long out_ld;
    int H, R, Sk;
    int units;        // (batch, head) pairs
    int keys;         // keys that some row sees (causal: min(Sk, k_past + R)); the rest stay zero
    int CL;           // CTAs (key ranges) per unit = cluster size
    int clusters;     // clusters in the grid; cluster i takes units i, i + clusters, ...
    int range_rows;   // key rows per CTA (the last range may be shorter or empty)
    int stages;       // ring stages in use
    int bufs;         // score buffers (2 when a cluster walks more than one unit)
    int wide;         // 1: four CTAs of four consumer warps per SM (many short units), 0: one persistent CTA per SM
    long long qsb, qsh, qss, ksb, ksh, kss;   // strides in elements
    float c;          // scale * log2(e), sign included
    int causal, k_past;
    float inv_norm;   // 1 / (h_norm * R)
    int* status;
};

// Shared-memory layout: [ring: stages x 16 KiB][scores: bufs x R x range_rows fp32][fixed part]
constexpr int SMALLQ_XCH_FLOATS = 2 * SMALLQ_MAX_CLUSTER * SMALLQ_MAX_ROWS * 2;    // two units in flight
constexpr int SMALLQ_RED_FLOATS = 2 * SMALLQ_CONSUMER_WARPS * SMALLQ_MAX_ROWS * 2; // (max, sum) per warp, two units
constexpr int SMALLQ_FIXED_BYTES = (2 * SMALLQ_MAX_STAGES + 2) * 8                 // full / empty / exchange barriers
                                   + 16                                            // abort flag
                                   + SMALLQ_RED_FLOATS * 4
                                   + SMALLQ_XCH_FLOATS * 4;                        // (max, sum) of every CTA of the cluster

// `bufs`: score buffers -- two when a cluster walks more than one unit (a unit is finished
// while the next one's scores are computed), else one.
inline size_t smallq_smem_for(int R, int range_rows, int stages, int bufs) {
    return (size_t)stages * SMALLQ_STAGE_BYTES + (size_t)bufs * R * range_rows * 4 + SMALLQ_FIXED_BYTES + 128;
}

// Cluster size, grid and ring depth.
// Many short units (at least two per SM, each at most 160 KiB of keys): four CTAs per SM, four
// consumer warps and a ring of three stages each, no key split -- the units in flight on an SM
// hide each other's latency chains.
// Otherwise one persistent CTA per SM with eight consumer warps and a deep ring; a cluster size
// cl gives sms / cl clusters, the busiest CTA reads ceil(units / clusters) ranges of
// ceil(keys / cl) rows, and the size with the least such rows wins (ties: the smaller cluster).
// Returns false when no cluster size holds the scores of a key range next to the shortest ring.
inline bool smallq_plan(int units, int R, int keys, int D, int sms, int* CL, int* clusters, int* range_rows,
                        int* stages, int* bufs, int* wide, size_t* smem) {
    if (D != 64 && D != 128) return false;   // rows are dealt over D/8 lanes: a power of two
    if (R < 1 || R > SMALLQ_MAX_ROWS || units < 1 || keys < 1) return false;
    if (units >= 2 * sms && (long long)keys * 2 * D <= 160 * 1024) {
        const int ncl = units < 4 * sms ? units : 4 * sms;
        const int nb = units > ncl ? 2 : 1;
        const size_t need = smallq_smem_for(R, keys, SMALLQ_WIDE_STAGES, nb);
        if (need <= 55 * 1024) {   // four such CTAs (plus 1 KiB each that the system reserves) fit an SM
            if (CL) *CL = 1;
            if (clusters) *clusters = ncl;
            if (range_rows) *range_rows = keys;
            if (stages) *stages = SMALLQ_WIDE_STAGES;
            if (bufs) *bufs = nb;
            if (wide) *wide = 1;
            if (smem) *smem = need;
            return true;
        }
    }
    int best_cl = 0;
    long long best_rows = 0;
    for (int cl = 1; cl <= SMALLQ_MAX_CLUSTER; ++cl) {
        const int rr = (keys + cl - 1) / cl;
        if (cl > 1 && rr < 32) break;     // ranges this short are all overhead
        int ncl = sms / cl;
        if (ncl < 1) ncl = 1;
        if (ncl > units) ncl = units;
        if (smallq_smem_for(R, rr, SMALLQ_MIN_STAGES, units > ncl ? 2 : 1) > SMALLQ_MAX_SMEM) continue;
        const long long rows = (long long)((units + ncl - 1) / ncl) * rr;
        if (best_cl == 0 || rows < best_rows) { best_cl = cl; best_rows = rows; }
    }
    if (best_cl == 0) return false;
    const int cl = best_cl;
    const int rr = (keys + cl - 1) / cl;
    int ncl = sms / cl;
    if (ncl < 1) ncl = 1;
    if (ncl > units) ncl = units;
    const int nb = units > ncl ? 2 : 1;
    int st = SMALLQ_MAX_STAGES;
    while (st > SMALLQ_MIN_STAGES && smallq_smem_for(R, rr, st, nb) > SMALLQ_MAX_SMEM) --st;
    if (CL) *CL = cl;
    if (clusters) *clusters = ncl;
    if (range_rows) *range_rows = rr;
    if (stages) *stages = st;
    if (bufs) *bufs = nb;
    if (wide) *wide = 0;
    if (smem) *smem = smallq_smem_for(R, rr, st, nb);
    return true;
}

// Whether the few-row kernel takes a call with R rows, Sk keys and `units` (batch, head) pairs.
inline bool smallq_fits(int R, int Sk, int D, int units, int sms) {
    return smallq_plan(units, R, Sk, D, sms, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr);
}

template <bool BF16>
__device__ __forceinline__ float2 unpack16x2(uint32_t v) {
    if (BF16) {
        return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
    } else {
        const __half2 h = *reinterpret_cast<const __half2*>(&v);
        return __half22float2(h);
    }
}

// ---------------------------------------------------------------- cluster helpers
__device__ __forceinline__ uint32_t smallq_cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t smallq_cluster_id() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void smallq_cluster_arrive() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void smallq_cluster_wait() {
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Asynchronous store of (a, b) to the shared memory of CTA `rank` of this cluster, at the address
// `local_addr` has in this CTA; its 8 bytes are counted on that CTA's barrier at `local_bar`.
__device__ __forceinline__ void smallq_post(uint32_t local_addr, uint32_t local_bar, uint32_t rank, float a, float b) {
    uint32_t addr, bar;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(addr) : "r"(local_addr), "r"(rank));
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(bar) : "r"(local_bar), "r"(rank));
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v2.f32 [%0], {%1, %2}, [%3];"
                 ::"r"(addr), "f"(a), "f"(b), "r"(bar)
                 : "memory");
}
// Barrier among the consumer warps only (the copy warp runs ahead on its own).
template <int W>
__device__ __forceinline__ void smallq_consumer_sync() {
    asm volatile("bar.sync 1, %0;" ::"n"(32 * W) : "memory");
}

// (maximum, sum of exp2 relative to it) of two sets of scores -> of their union
__device__ __forceinline__ void smallq_merge(float& m, float& l, float mo, float lo) {
    const float mn = fmaxf(m, mo);
    const float ms = (mn == -INFINITY) ? 0.f : mn;
    l = l * ex2_approx(m - ms) + lo * ex2_approx(mo - ms);
    m = mn;
}

// Zero the B x S valid entries of `out`; lets the kernel behind it in the stream start at once.
__global__ void clear_rows_kernel(float* out, long long out_ld, int B, int S) {
    grid_launch_dependents();
    const long long n = (long long)B * S;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long b = idx / S;
        out[b * out_ld + (idx - b * S)] = 0.f;
    }
}

// RMAX: compile-time bound on the query rows (1, 2 or 4); W: consumer warps (8, or 4 with four CTAs per SM;
// sixteen were measured no faster on a decode query over 32768 keys: the scoring is bound by the count of
// its instructions, the 16-bit to fp32 conversions first, not by latency).
template <int D, bool BF16, int RMAX, int W>
__global__ void __launch_bounds__(32 * (W + 1), W == SMALLQ_WIDE_WARPS ? 4 : 1)
colsum_small_q_kernel(const SmallQParams p) {
    constexpr int SMALLQ_CONSUMER_THREADS = 32 * W;
    extern __shared__ __align__(128) uint8_t smallq_smem[];
    uint8_t* ring = smallq_smem;
    float* sc_base = reinterpret_cast<float*>(ring + (size_t)p.stages * SMALLQ_STAGE_BYTES);   // [bufs][R][range_rows]
    const size_t sc_buf = (size_t)p.R * p.range_rows;
    uint8_t* fixed = reinterpret_cast<uint8_t*>(sc_base + (size_t)p.bufs * sc_buf);
    fixed = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(fixed) + 15) & ~static_cast<uintptr_t>(15));
    const uint32_t bars = smem_u32(fixed);                    // full[MAX_STAGES], empty[MAX_STAGES], exchange[2]
    volatile int* abort_flag = reinterpret_cast<volatile int*>(fixed + (2 * SMALLQ_MAX_STAGES + 2) * 8);
    float* red = reinterpret_cast<float*>(fixed + (2 * SMALLQ_MAX_STAGES + 2) * 8 + 16);   // [2][warps][MAX_ROWS][2]
    float* xch = red + SMALLQ_RED_FLOATS;                                                  // [2][MAX_CLUSTER][MAX_ROWS][2]
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (SMALLQ_MAX_STAGES + s); };
    auto xch_bar = [&](int i) { return bars + 8u * (2 * SMALLQ_MAX_STAGES + i); };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cr = smallq_cluster_rank();
    const int cluster = (int)smallq_cluster_id();
    int k0 = (int)cr * p.range_rows, k1 = k0 + p.range_rows;
    if (k0 > p.keys) k0 = p.keys;
    if (k1 > p.keys) k1 = p.keys;
    const int rows = k1 - k0;
    constexpr int ROW_BYTES = 2 * D;
    constexpr int STAGE_ROWS = SMALLQ_STAGE_BYTES / ROW_BYTES;
    const int chunks = (rows + STAGE_ROWS - 1) / STAGE_ROWS;     // per unit

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), W); }
        mbar_init(xch_bar(0), 1);
        mbar_init(xch_bar(1), 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    // every CTA of the cluster has set up its barriers once this completes; it is waited for
    // before the first store into another CTA's shared memory
    smallq_cluster_arrive();

    if (warp == W) {
        // ------------------------------------------------ copy issuer: runs ahead across units
        // contiguous key rows: one copy per stage; strided rows: one copy per row, dealt over the lanes
        const bool dense = p.kss == D;
        bool ok = true;
        int n = 0;      // stages filled so far
        for (int unit = cluster; unit < p.units && ok; unit += p.clusters) {
            const int b = unit / p.H, h = unit % p.H;
            const uint16_t* kb = reinterpret_cast<const uint16_t*>(p.k) + b * p.ksb + h * p.ksh;
            for (int ch = 0; ch < chunks; ++ch, ++n) {
                const int s = n % p.stages;
                if (n >= p.stages) {
                    ok = mbar_wait(empty_bar(s), ((n / p.stages) & 1) ^ 1, abort_flag, p.status, FCS_STATUS_WAIT_PRODUCER);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                }
                const int r0 = k0 + ch * STAGE_ROWS;
                const int cnt = min(STAGE_ROWS, k1 - r0);
                const uint32_t dst = smem_u32(ring + (size_t)s * SMALLQ_STAGE_BYTES);
                if (lane == 0) mbar_arrive_expect_tx(full_bar(s), (uint32_t)cnt * ROW_BYTES);
                __syncwarp();
                if (dense) {
                    if (lane == 0) bulk_load(dst, kb + (long long)r0 * p.kss, (uint32_t)cnt * ROW_BYTES, full_bar(s));
                } else {
                    for (int i = lane; i < cnt; i += 32)
                        bulk_load(dst + i * ROW_BYTES, kb + (long long)(r0 + i) * p.kss, ROW_BYTES, full_bar(s));
                }
            }
        }
        smallq_cluster_wait();
    } else {
        // ------------------------------------------------ consumers
        // A warp takes 32 key rows at a time.  D/8 adjacent lanes share a row, 16 bytes each, over
        // D/8 passes; the partial dot products are then transposed and summed with D/8 - 1
        // shuffles, after which every lane holds the score of one row.
        constexpr int LPR = D / 8;            // lanes per key row = passes per 32 rows
        constexpr int RPW = 32 / LPR;         // key rows per pass
        constexpr int GROUPS = STAGE_ROWS / 32;
        const int piece = lane % LPR, sub = lane / LPR;
        auto load_q = [&](int unit, uint4 (&raw)[RMAX]) {
            const int b = unit / p.H, h = unit % p.H;
            const uint16_t* qb = reinterpret_cast<const uint16_t*>(p.q) + b * p.qsb + h * p.qsh;
#pragma unroll
            for (int r = 0; r < RMAX; ++r)
                raw[r] = (r < p.R) ? __ldg(reinterpret_cast<const uint4*>(qb + r * p.qss) + piece)
                                   : make_uint4(0u, 0u, 0u, 0u);
        };
        // A wait that runs out raises the abort flag (later waits then give up at once) but does not
        // end the loops: all consumer warps keep meeting at the named barrier, the results are void and
        // the status word says so.
        bool ok = true, peers_up = false, out_clear = false;

        // unit `u` (the uc-th of this cluster) is finished one unit late, behind the scores of the
        // next one: by then every range's (maximum, sum) has long arrived
        auto finish = [&](int unit, int uc) {
            const int xb = uc & 1;
            float M[SMALLQ_MAX_ROWS], w[SMALLQ_MAX_ROWS];
            if (p.CL == 1) {
                // the whole key axis is this CTA's: the warps' values are in shared memory since the
                // barrier that ended the unit, no exchange to wait for
                const float* rbp = red + (size_t)xb * SMALLQ_CONSUMER_WARPS * SMALLQ_MAX_ROWS * 2;
#pragma unroll
                for (int r = 0; r < SMALLQ_MAX_ROWS; ++r) {
                    M[r] = 0.f; w[r] = 0.f;
                    if (r < RMAX && r < p.R) {
                        float mm = -INFINITY, ll = 0.f;
                        for (int wi = 0; wi < W; ++wi)
                            smallq_merge(mm, ll, rbp[(wi * SMALLQ_MAX_ROWS + r) * 2], rbp[(wi * SMALLQ_MAX_ROWS + r) * 2 + 1]);
                        M[r] = mm;
                        w[r] = ok ? p.inv_norm / ll : 0.f;
                    }
                }
            } else {
            ok = ok && mbar_wait(xch_bar(xb), (uc >> 1) & 1, abort_flag, p.status, FCS_STATUS_WAIT_CONSUMER);
            ok = __all_sync(0xffffffffu, ok);
            const float* xv = xch + (size_t)xb * SMALLQ_MAX_CLUSTER * SMALLQ_MAX_ROWS * 2;
#pragma unroll
            for (int r = 0; r < SMALLQ_MAX_ROWS; ++r) {
                M[r] = 0.f; w[r] = 0.f;
                if (r < p.R) {
                    float mm = -INFINITY, ll = 0.f;
                    for (int i = 0; i < p.CL; ++i)
                        smallq_merge(mm, ll, xv[(i * SMALLQ_MAX_ROWS + r) * 2], xv[(i * SMALLQ_MAX_ROWS + r) * 2 + 1]);
                    M[r] = mm;
                    w[r] = ok ? p.inv_norm / ll : 0.f;
                }
            }
            }
            if (!out_clear) { grid_dependency_wait(); out_clear = true; }   // the output has been cleared
            const float* sc = sc_base + (size_t)(p.bufs == 2 ? xb : 0) * sc_buf;
            float* ob = p.out + (long long)(unit / p.H) * p.out_ld + k0;
            for (int kl = threadIdx.x; kl < rows; kl += SMALLQ_CONSUMER_THREADS) {
                float v = 0.f;
#pragma unroll
                for (int r = 0; r < SMALLQ_MAX_ROWS; ++r)
                    if (r < p.R) v += ex2_approx(sc[(size_t)r * p.range_rows + kl] - M[r]) * w[r];
                atomicAdd_system(ob + kl, v);   // `out` may live on another GPU
            }
        };

        uint4 qnext[RMAX];
        if (cluster < p.units) load_q(cluster, qnext);
        int n = 0, ucount = 0, prev_unit = -1;
        for (int unit = cluster; unit < p.units; unit += p.clusters, ++ucount) {
            float qreg[RMAX][8];
#pragma unroll
            for (int r = 0; r < RMAX; ++r) {
                const float2 f0 = unpack16x2<BF16>(qnext[r].x), f1 = unpack16x2<BF16>(qnext[r].y);
                const float2 f2 = unpack16x2<BF16>(qnext[r].z), f3 = unpack16x2<BF16>(qnext[r].w);
                qreg[r][0] = f0.x * p.c; qreg[r][1] = f0.y * p.c; qreg[r][2] = f1.x * p.c; qreg[r][3] = f1.y * p.c;
                qreg[r][4] = f2.x * p.c; qreg[r][5] = f2.y * p.c; qreg[r][6] = f3.x * p.c; qreg[r][7] = f3.y * p.c;
            }
            if (unit + p.clusters < p.units) load_q(unit + p.clusters, qnext);   // lands during this unit
            const int xb = ucount & 1;
            if (threadIdx.x == 0 && p.CL > 1) mbar_arrive_expect_tx(xch_bar(xb), (uint32_t)p.CL * SMALLQ_MAX_ROWS * 8);
            float* sc = sc_base + (size_t)(p.bufs == 2 ? xb : 0) * sc_buf;

            // scores (log2 domain) of this range, with a running (maximum, sum) per thread
            float tm[RMAX], tl[RMAX];
#pragma unroll
            for (int r = 0; r < RMAX; ++r) { tm[r] = -INFINITY; tl[r] = 0.f; }
            for (int ch = 0; ch < chunks; ++ch, ++n) {
                const int s = n % p.stages;
                ok = ok && mbar_wait(full_bar(s), (n / p.stages) & 1, abort_flag, p.status, FCS_STATUS_WAIT_CONSUMER);
                ok = __all_sync(0xffffffffu, ok);
                const uint4* st = reinterpret_cast<const uint4*>(ring + (size_t)s * SMALLQ_STAGE_BYTES);
                const int cnt = min(STAGE_ROWS, rows - ch * STAGE_ROWS);
                // the 32-row groups of the stages go round the warps
                for (int g = (warp - n * GROUPS) & (W - 1); g < GROUPS; g += W) {
                    if (g * 32 >= cnt) break;
                    float part[RMAX][LPR];
#pragma unroll
                    for (int j = 0; j < LPR; ++j) {
                        const int row = g * 32 + j * RPW + sub;
                        uint4 raw = make_uint4(0u, 0u, 0u, 0u);
                        if (row < cnt) raw = st[row * LPR + piece];
                        const float2 f0 = unpack16x2<BF16>(raw.x), f1 = unpack16x2<BF16>(raw.y);
                        const float2 f2 = unpack16x2<BF16>(raw.z), f3 = unpack16x2<BF16>(raw.w);
#pragma unroll
                        for (int r = 0; r < RMAX; ++r)
                            part[r][j] = ((f0.x * qreg[r][0] + f0.y * qreg[r][1]) + (f1.x * qreg[r][2] + f1.y * qreg[r][3])) +
                                         ((f2.x * qreg[r][4] + f2.y * qreg[r][5]) + (f3.x * qreg[r][6] + f3.y * qreg[r][7]));
                    }
                    // transpose and sum over the lanes of a row: afterwards part[r][0] is the score of
                    // the row of pass j = piece
#pragma unroll
                    for (int half = LPR / 2; half >= 1; half >>= 1) {
                        const bool up = (piece & half) != 0;
#pragma unroll
                        for (int r = 0; r < RMAX; ++r) {
#pragma unroll
                            for (int t = 0; t < half; ++t) {
                                const float send = up ? part[r][t] : part[r][t + half];
                                const float keep = up ? part[r][t + half] : part[r][t];
                                part[r][t] = keep + __shfl_xor_sync(0xffffffffu, send, half);
                            }
                        }
                    }
                    const int row = g * 32 + piece * RPW + sub;
                    if (row < cnt) {
                        const int kl = ch * STAGE_ROWS + row;       // row within the range
#pragma unroll
                        for (int r = 0; r < RMAX; ++r) {
                            if (r < p.R) {
                                const bool visible = !p.causal || (k0 + kl <= p.k_past + r);
                                const float sv = visible ? part[r][0] : -INFINITY;
                                sc[(size_t)r * p.range_rows + kl] = sv;
                                if (sv > tm[r]) { tl[r] = tl[r] * ex2_approx(tm[r] - sv) + 1.f; tm[r] = sv; }
                                else if (sv != -INFINITY) tl[r] += ex2_approx(sv - tm[r]);
                            }
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty_bar(s));    // the stage may be refilled
            }

            // the unit before this one: its exchange has completed while the scores above were computed
            if (prev_unit >= 0) finish(prev_unit, ucount - 1);

            // (maximum, sum) of the range: over the warp by shuffles, over the warps through shared
            // memory (one barrier; the staging buffer alternates between units)
            float* rb = red + (size_t)xb * SMALLQ_CONSUMER_WARPS * SMALLQ_MAX_ROWS * 2;
#pragma unroll
            for (int r = 0; r < RMAX; ++r) {
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    const float mo = __shfl_xor_sync(0xffffffffu, tm[r], o);
                    const float lo = __shfl_xor_sync(0xffffffffu, tl[r], o);
                    smallq_merge(tm[r], tl[r], mo, lo);
                }
                if (lane == 0) { rb[(warp * SMALLQ_MAX_ROWS + r) * 2] = tm[r]; rb[(warp * SMALLQ_MAX_ROWS + r) * 2 + 1] = tl[r]; }
            }
            smallq_consumer_sync<W>();   // also orders this unit's score stores, and the finish above before the next unit's
            if (!peers_up) { smallq_cluster_wait(); peers_up = true; }
            if (p.CL > 1 && threadIdx.x < p.CL * SMALLQ_MAX_ROWS) {
                const int dst = threadIdx.x / SMALLQ_MAX_ROWS, r = threadIdx.x % SMALLQ_MAX_ROWS;
                float mm = -INFINITY, ll = 0.f;
                if (r < RMAX && r < p.R)
                    for (int w = 0; w < W; ++w)
                        smallq_merge(mm, ll, rb[(w * SMALLQ_MAX_ROWS + r) * 2], rb[(w * SMALLQ_MAX_ROWS + r) * 2 + 1]);
                const uint32_t slot = smem_u32(xch + ((size_t)(xb * SMALLQ_MAX_CLUSTER + cr) * SMALLQ_MAX_ROWS + r) * 2);
                smallq_post(slot, xch_bar(xb), (uint32_t)dst, mm, ll);
            }
            prev_unit = unit;
        }
        if (prev_unit >= 0) finish(prev_unit, ucount - 1);
        if (!peers_up) smallq_cluster_wait();
    }
    // nobody leaves while a peer may still store into its shared memory (a CTA that gave up a wait
    // has not waited for those stores on its exchange barriers: it lingers until they have landed)
    smallq_cluster_arrive();
    smallq_cluster_wait();
    if (*abort_flag) __nanosleep(100000);
}

}  // namespace fcs
