// Column mean when only a handful of query rows enter it (a CLS prefix, or a few
// decode queries): per (batch, head) the work is R dot products per key, i.e. a
// matrix-vector product that reads every key once.  That is bound by HBM, not by
// the tensor cores, so it is not reshaped into a GEMM; what matters is that every
// SM keeps enough bytes in flight and that short calls have no dependent rounds.
//
//   * The key axis of a (batch, head) is cut into up to eight ranges, one CTA each,
//     the CTAs of a (batch, head) forming a thread-block cluster: a decode query over
//     32 heads then fills the device instead of 32 SMs, and a CLS call runs as many
//     small CTAs that the block scheduler balances.
//   * A CTA's key rows arrive through a ring of 16 KiB shared-memory stages filled by
//     bulk asynchronous copies (cp.async.bulk, completion counted on an mbarrier --
//     no tensor map, no multicast): all stages are requested when the CTA starts, so
//     a range of up to six stages is one round trip to memory.
//   * Scores of the range stay in shared memory between the sweeps (scores and maximum
//     while the rows arrive; exp2 and sum; weights and the add into the output).
//   * Each CTA posts its (maximum, sum) per query row into the shared memory of every
//     CTA of its cluster; after one cluster barrier each CTA has the row's global
//     normaliser and adds its keys' share into the output.
//   * The output is cleared by a small kernel launched just before; this kernel is a
//     programmatic dependent of it and waits for it only right before its adds, so
//     the clear costs no time on the device.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../../include/flash_colsum_b200.h"
#include "sm100_ptx.cuh"

namespace fcs {

constexpr int SMALLQ_MAX_ROWS = 4;
constexpr int SMALLQ_CONSUMER_WARPS = 8;
constexpr int SMALLQ_THREADS = 32 * (SMALLQ_CONSUMER_WARPS + 1);   // + one warp that issues the copies
constexpr int SMALLQ_STAGE_BYTES = 16 * 1024;
constexpr int SMALLQ_MAX_STAGES = 6;
constexpr int SMALLQ_MAX_CLUSTER = 8;
constexpr size_t SMALLQ_MAX_SMEM = 200 * 1024;

struct SmallQParams {
    const void* q;
    const void* k;
    float* out;
    long long out_ld;
    int H, R, Sk;
    int keys;         // keys that some row sees (causal: min(Sk, k_past + R)); the rest stay zero
    int CL;           // CTAs (key ranges) per (batch, head) = cluster size
    int range_rows;   // key rows per CTA (the last range may be shorter or empty)
    int stages;       // ring stages in use
    long long qsb, qsh, qss, ksb, ksh, kss;   // strides in elements
    float c;          // scale * log2(e), sign included
    int causal, k_past;
    float inv_norm;   // 1 / (h_norm * R)
    int* status;
};

// Shared-memory layout: [ring: stages x 16 KiB][scores: R x range_rows fp32][fixed part]
constexpr int SMALLQ_FIXED_BYTES = 2 * SMALLQ_MAX_STAGES * 8                       // full / empty barriers
                                   + 16                                            // abort flag
                                   + (SMALLQ_THREADS / 32) * SMALLQ_MAX_ROWS * 4  // reduction staging
                                   + SMALLQ_MAX_ROWS * 4                           // reduction result
                                   + SMALLQ_MAX_CLUSTER * SMALLQ_MAX_ROWS * 8;     // (max, sum) of every CTA of the cluster

inline size_t smallq_smem_for(int R, int range_rows, int stages) {
    return (size_t)stages * SMALLQ_STAGE_BYTES + (size_t)R * range_rows * 4 + SMALLQ_FIXED_BYTES + 128;
}

// Whether the few-row kernel takes a call with R rows and Sk keys at all: the scores of a key
// range (an eighth of the keys at least) must fit next to a ring of two stages.
inline bool smallq_fits(int R, int Sk, int D) {
    (void)D;
    if (R < 1 || R > SMALLQ_MAX_ROWS) return false;
    const int range_rows = (Sk + SMALLQ_MAX_CLUSTER - 1) / SMALLQ_MAX_CLUSTER;
    return smallq_smem_for(R, range_rows, 2) <= SMALLQ_MAX_SMEM;
}

// Cut of the key axis: as many ranges as give every CTA about 40 KiB of keys, more (down to
// 32 rows each) while the grid is below two CTAs per SM, never more than eight.
inline void smallq_plan(int units, int R, int keys, int D, int sms, int* CL, int* range_rows, int* stages,
                        size_t* smem) {
    const int row_bytes = 2 * D;
    const long long unit_bytes = (long long)keys * row_bytes;
    int cl = (int)((unit_bytes + 40 * 1024 - 1) / (40 * 1024));
    if (cl < 1) cl = 1;
    while (cl < SMALLQ_MAX_CLUSTER && (long long)units * cl < 2ll * sms && keys / (cl + 1) >= 32) ++cl;
    if (cl > SMALLQ_MAX_CLUSTER) cl = SMALLQ_MAX_CLUSTER;
    int rr = (keys + cl - 1) / cl;
    while (cl < SMALLQ_MAX_CLUSTER && smallq_smem_for(R, rr, 2) > SMALLQ_MAX_SMEM) { ++cl; rr = (keys + cl - 1) / cl; }
    const int rows_per_stage = SMALLQ_STAGE_BYTES / row_bytes;
    int st = (rr + rows_per_stage - 1) / rows_per_stage;
    if (st > SMALLQ_MAX_STAGES) st = SMALLQ_MAX_STAGES;
    if (st < 1) st = 1;
    while (st > 2 && smallq_smem_for(R, rr, st) > SMALLQ_MAX_SMEM) --st;
    *CL = cl; *range_rows = rr; *stages = st;
    *smem = smallq_smem_for(R, rr, st);
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
__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_arrive_relaxed() {
    asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_arrive_release() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait_acquire() {
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Store one fp32 into the shared memory of CTA `rank` of this cluster, at the address that
// `local_smem_addr` has in this CTA.
__device__ __forceinline__ void st_cluster_f32(uint32_t local_smem_addr, uint32_t rank, float v) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_smem_addr), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}

// max or sum over all warps of the CTA of R per-thread values; result in red_out[0..R)
template <bool IS_MAX>
__device__ __forceinline__ void smallq_reduce(float (&v)[SMALLQ_MAX_ROWS], float* red, float* red_out) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int r = 0; r < SMALLQ_MAX_ROWS; ++r) {
        float x = v[r];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float y = __shfl_xor_sync(0xffffffffu, x, o);
            x = IS_MAX ? fmaxf(x, y) : x + y;
        }
        if (lane == 0) red[warp * SMALLQ_MAX_ROWS + r] = x;
    }
    __syncthreads();
    if (threadIdx.x < SMALLQ_MAX_ROWS) {
        float x = IS_MAX ? -INFINITY : 0.f;
        for (int w = 0; w < SMALLQ_THREADS / 32; ++w) {
            const float y = red[w * SMALLQ_MAX_ROWS + threadIdx.x];
            x = IS_MAX ? fmaxf(x, y) : x + y;
        }
        red_out[threadIdx.x] = x;
    }
    __syncthreads();
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

// RMAX: compile-time bound on the query rows (1, 2 or 4).
template <int D, bool BF16, int RMAX>
__global__ void __launch_bounds__(SMALLQ_THREADS, RMAX == 4 ? 2 : 4)
colsum_small_q_kernel(const SmallQParams p) {
    extern __shared__ __align__(128) uint8_t smallq_smem[];
    uint8_t* ring = smallq_smem;
    float* sc = reinterpret_cast<float*>(ring + (size_t)p.stages * SMALLQ_STAGE_BYTES);   // [R][range_rows]
    uint8_t* fixed = reinterpret_cast<uint8_t*>(sc + (size_t)p.R * p.range_rows);
    fixed = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(fixed) + 15) & ~static_cast<uintptr_t>(15));
    const uint32_t bars = smem_u32(fixed);                                   // full[stages], empty[stages]
    volatile int* abort_flag = reinterpret_cast<volatile int*>(fixed + 2 * SMALLQ_MAX_STAGES * 8);
    float* red = reinterpret_cast<float*>(fixed + 2 * SMALLQ_MAX_STAGES * 8 + 16);
    float* red_out = red + (SMALLQ_THREADS / 32) * SMALLQ_MAX_ROWS;
    float* xch = red_out + SMALLQ_MAX_ROWS;                                  // [CL][MAX_ROWS][2]
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (SMALLQ_MAX_STAGES + s); };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cr = cluster_cta_rank();
    const int unit = blockIdx.x / p.CL;
    const int b = unit / p.H, h = unit % p.H;
    const uint16_t* qb = reinterpret_cast<const uint16_t*>(p.q) + b * p.qsb + h * p.qsh;
    const uint16_t* kb = reinterpret_cast<const uint16_t*>(p.k) + b * p.ksb + h * p.ksh;
    int k0 = (int)cr * p.range_rows, k1 = k0 + p.range_rows;
    if (k0 > p.keys) k0 = p.keys;
    if (k1 > p.keys) k1 = p.keys;
    const int rows = k1 - k0;
    constexpr int ROW_BYTES = 2 * D;
    constexpr int STAGE_ROWS = SMALLQ_STAGE_BYTES / ROW_BYTES;
    const int chunks = (rows + STAGE_ROWS - 1) / STAGE_ROWS;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), SMALLQ_CONSUMER_WARPS); }
        *abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    // every CTA of the cluster is running once this barrier completes; it is waited for only
    // before the first store into another CTA's shared memory
    cluster_arrive_relaxed();

    float vmax[SMALLQ_MAX_ROWS];
#pragma unroll
    for (int r = 0; r < SMALLQ_MAX_ROWS; ++r) vmax[r] = -INFINITY;

    if (warp == SMALLQ_CONSUMER_WARPS) {
        // ------------------------------------------------ copy issuer
        // contiguous key rows: one copy per stage; strided rows: one copy per row, dealt over the lanes
        const bool dense = p.kss == D;
        bool ok = true;
        for (int ch = 0; ch < chunks && ok; ++ch) {
            const int s = ch % p.stages;
            if (ch >= p.stages) {
                ok = mbar_wait(empty_bar(s), ((ch / p.stages) & 1) ^ 1, abort_flag, p.status, FCS_STATUS_WAIT_CONSUMER);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
            }
            const int r0 = k0 + ch * STAGE_ROWS;
            const int n = min(STAGE_ROWS, k1 - r0);
            const uint32_t dst = smem_u32(ring + (size_t)s * SMALLQ_STAGE_BYTES);
            if (lane == 0) mbar_arrive_expect_tx(full_bar(s), (uint32_t)n * ROW_BYTES);
            __syncwarp();
            if (dense) {
                if (lane == 0) bulk_load(dst, kb + (long long)r0 * p.kss, (uint32_t)n * ROW_BYTES, full_bar(s));
            } else {
                for (int i = lane; i < n; i += 32)
                    bulk_load(dst + i * ROW_BYTES, kb + (long long)(r0 + i) * p.kss, ROW_BYTES, full_bar(s));
            }
        }
    } else {
        // ------------------------------------------------ sweep 1: scores (log2 domain) and their maximum
        // D/8 adjacent lanes share a key row, 16 bytes each; partial dot products meet by shuffles
        constexpr int LPR = D / 8;            // lanes per key row
        constexpr int RPW = 32 / LPR;         // key rows per warp and step
        const int piece = lane % LPR, sub = lane / LPR;
        float qreg[RMAX][8];
#pragma unroll
        for (int r = 0; r < RMAX; ++r) {
            uint4 raw = make_uint4(0u, 0u, 0u, 0u);
            if (r < p.R) raw = __ldg(reinterpret_cast<const uint4*>(qb + r * p.qss) + piece);
            const float2 f0 = unpack16x2<BF16>(raw.x), f1 = unpack16x2<BF16>(raw.y);
            const float2 f2 = unpack16x2<BF16>(raw.z), f3 = unpack16x2<BF16>(raw.w);
            qreg[r][0] = f0.x * p.c; qreg[r][1] = f0.y * p.c; qreg[r][2] = f1.x * p.c; qreg[r][3] = f1.y * p.c;
            qreg[r][4] = f2.x * p.c; qreg[r][5] = f2.y * p.c; qreg[r][6] = f3.x * p.c; qreg[r][7] = f3.y * p.c;
        }
        bool ok = true;
        for (int ch = 0; ch < chunks && ok; ++ch) {
            const int s = ch % p.stages;
            ok = mbar_wait(full_bar(s), (ch / p.stages) & 1, abort_flag, p.status, FCS_STATUS_WAIT_CONSUMER);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const uint4* st = reinterpret_cast<const uint4*>(ring + (size_t)s * SMALLQ_STAGE_BYTES);
            const int n = min(STAGE_ROWS, rows - ch * STAGE_ROWS);
#pragma unroll 2
            for (int i0 = 0; i0 < n; i0 += SMALLQ_CONSUMER_WARPS * RPW) {
                const int i = i0 + warp * RPW + sub;
                uint4 raw = make_uint4(0u, 0u, 0u, 0u);
                if (i < n) raw = st[i * LPR + piece];
                const float2 f0 = unpack16x2<BF16>(raw.x), f1 = unpack16x2<BF16>(raw.y);
                const float2 f2 = unpack16x2<BF16>(raw.z), f3 = unpack16x2<BF16>(raw.w);
                const int kl = ch * STAGE_ROWS + i;       // row within the range
#pragma unroll
                for (int r = 0; r < RMAX; ++r) {
                    if (r < p.R) {      // uniform across the CTA
                        float d = f0.x * qreg[r][0] + f0.y * qreg[r][1] + f1.x * qreg[r][2] + f1.y * qreg[r][3] +
                                  f2.x * qreg[r][4] + f2.y * qreg[r][5] + f3.x * qreg[r][6] + f3.y * qreg[r][7];
#pragma unroll
                        for (int o = LPR / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
                        if (piece == 0 && i < n) {
                            const bool visible = !p.causal || (k0 + kl <= p.k_past + r);
                            const float sv = visible ? d : -INFINITY;
                            sc[(size_t)r * p.range_rows + kl] = sv;
                            vmax[r] = fmaxf(vmax[r], sv);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_bar(s));
        }
    }
    smallq_reduce<true>(vmax, red, red_out);
    float m[SMALLQ_MAX_ROWS];
#pragma unroll
    for (int r = 0; r < SMALLQ_MAX_ROWS; ++r) m[r] = red_out[r];
    __syncthreads();

    // sweep 2: exp2 relative to this range's maximum, and their sum
    float vsum[SMALLQ_MAX_ROWS] = {0.f, 0.f, 0.f, 0.f};
    for (int kl = threadIdx.x; kl < rows; kl += SMALLQ_THREADS) {
#pragma unroll
        for (int r = 0; r < SMALLQ_MAX_ROWS; ++r) {
            if (r < p.R) {
                const float ms = (m[r] == -INFINITY) ? 0.f : m[r];
                const float e = ex2_approx(sc[(size_t)r * p.range_rows + kl] - ms);
                sc[(size_t)r * p.range_rows + kl] = e;
                vsum[r] += e;
            }
        }
    }
    smallq_reduce<false>(vsum, red, red_out);

    // every CTA of the cluster gets every range's (maximum, sum)
    cluster_wait_acquire();   // (the barrier entered at the start: all CTAs are up)
    if (threadIdx.x < p.CL * SMALLQ_MAX_ROWS) {
        const int dst = threadIdx.x / SMALLQ_MAX_ROWS, r = threadIdx.x % SMALLQ_MAX_ROWS;
        const uint32_t slot = smem_u32(xch + ((size_t)cr * SMALLQ_MAX_ROWS + r) * 2);
        st_cluster_f32(slot, (uint32_t)dst, m[r]);
        st_cluster_f32(slot + 4, (uint32_t)dst, red_out[r]);
    }
    cluster_arrive_release();
    cluster_wait_acquire();
    float w[SMALLQ_MAX_ROWS];
#pragma unroll
    for (int r = 0; r < SMALLQ_MAX_ROWS; ++r) {
        float M = -INFINITY;
        for (int i = 0; i < p.CL; ++i) M = fmaxf(M, xch[(i * SMALLQ_MAX_ROWS + r) * 2]);
        float L = 0.f;
        for (int i = 0; i < p.CL; ++i) {
            const float mi = xch[(i * SMALLQ_MAX_ROWS + r) * 2];
            if (mi != -INFINITY) L += xch[(i * SMALLQ_MAX_ROWS + r) * 2 + 1] * ex2_approx(mi - M);
        }
        w[r] = (r < p.R && m[r] != -INFINITY) ? p.inv_norm * ex2_approx(m[r] - M) / L : 0.f;
    }

    // sweep 3: this range's share of the column means, once the output has been cleared
    grid_dependency_wait();
    float* ob = p.out + (long long)b * p.out_ld + k0;
    for (int kl = threadIdx.x; kl < rows; kl += SMALLQ_THREADS) {
        float v = 0.f;
#pragma unroll
        for (int r = 0; r < SMALLQ_MAX_ROWS; ++r)
            if (r < p.R) v += sc[(size_t)r * p.range_rows + kl] * w[r];
        atomicAdd_system(ob + kl, v);   // `out` may live on another GPU
    }
}

}  // namespace fcs
