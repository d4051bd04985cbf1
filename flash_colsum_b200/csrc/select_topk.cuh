// Token pruning on top of the column means: per batch row, the k key positions with
// the largest mean, in ascending position order (ties go to the lower position), on
// the stream that produced the means.  One CTA per row.
//
// Exact selection by radix: four passes over the row, most significant byte first,
// each counting the byte values of the elements that still match the prefix chosen so
// far; after the fourth pass the k-th largest value is known exactly, together with
// how many elements equal to it are still needed.  A last ordered pass writes the
// positions of everything above that value plus the first of the equal ones.  The row
// (at most a few hundred KiB) stays in L2 between passes.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace fcs {

constexpr int TOPK_THREADS = 1024;

// Order-preserving map from float to unsigned (larger float -> larger key).
__device__ __forceinline__ uint32_t topk_key(float v) {
    const uint32_t u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__global__ void __launch_bounds__(TOPK_THREADS)
select_topk_kernel(const float* __restrict__ colsum, long long ld, int S, int k, int* __restrict__ indices,
                   float* __restrict__ values) {
    __shared__ unsigned hist[256];
    __shared__ unsigned sh_prefix, sh_need;
    __shared__ unsigned warp_gt[TOPK_THREADS / 32], warp_eq[TOPK_THREADS / 32];
    __shared__ unsigned run_out, run_eq;
    const float* row = colsum + (long long)blockIdx.x * ld;
    int* out_idx = indices + (long long)blockIdx.x * k;
    float* out_val = values ? values + (long long)blockIdx.x * k : nullptr;
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;

    // ---- the k-th largest key, byte by byte
    unsigned prefix = 0, need = (unsigned)k;   // still to take among the elements matching `prefix`
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        const unsigned mask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        for (int i = tid; i < S; i += TOPK_THREADS) {
            const uint32_t key = topk_key(row[i]);
            if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
        }
        __syncthreads();
        if (tid == 0) {
            unsigned above = 0;
            int d = 255;
            for (; d > 0; --d) {
                if (above + hist[d] >= need) break;
                above += hist[d];
            }
            sh_prefix = prefix | ((unsigned)d << shift);
            sh_need = need - above;
        }
        __syncthreads();
        prefix = sh_prefix;
        need = sh_need;
        __syncthreads();
    }
    const uint32_t kth = prefix;   // exact key of the k-th largest element; `need` equal ones are wanted

    // ---- positions in ascending order: everything above kth, and the first `need` equal to it
    if (tid == 0) { run_out = 0; run_eq = 0; }
    __syncthreads();
    for (int base = 0; base < S; base += TOPK_THREADS) {
        const int i = base + tid;
        uint32_t key = 0;
        float v = 0.f;
        bool gt = false, eq = false;
        if (i < S) {
            v = row[i];
            key = topk_key(v);
            gt = key > kth;
            eq = key == kth;
        }
        const unsigned m_gt = __ballot_sync(0xffffffffu, gt), m_eq = __ballot_sync(0xffffffffu, eq);
        if (lane == 0) { warp_gt[wid] = __popc(m_gt); warp_eq[wid] = __popc(m_eq); }
        __syncthreads();
        unsigned gt_before = 0, eq_before = 0;   // in earlier warps of this chunk
        for (int w = 0; w < wid; ++w) { gt_before += warp_gt[w]; eq_before += warp_eq[w]; }
        const unsigned lower = (1u << lane) - 1u;
        gt_before += __popc(m_gt & lower);
        eq_before += __popc(m_eq & lower);
        const unsigned eq_seen = run_eq + eq_before;            // equal elements before this one in the row
        const unsigned eq_taken_before = eq_seen < need ? eq_seen : need;
        const bool take = gt || (eq && eq_seen < need);
        if (take) {
            // taken elements before this one: all greater ones, and the equal ones still within `need`
            const unsigned chunk_eq_taken = eq_taken_before - (run_eq < need ? run_eq : need);
            const unsigned pos = run_out + gt_before + chunk_eq_taken;
            out_idx[pos] = i;
            if (out_val) out_val[pos] = v;
        }
        __syncthreads();
        if (tid == TOPK_THREADS - 1) {
            const unsigned chunk_gt = gt_before + (gt ? 1u : 0u);
            const unsigned chunk_eq = eq_before + (eq ? 1u : 0u);
            const unsigned eq_old = run_eq < need ? run_eq : need;
            const unsigned eq_new_total = run_eq + chunk_eq;
            const unsigned eq_new = eq_new_total < need ? eq_new_total : need;
            run_out += chunk_gt + (eq_new - eq_old);
            run_eq = eq_new_total;
        }
        __syncthreads();
    }
}

// The threshold form of the pruning step: per batch row, the positions whose column mean is at
// least `threshold` (relative = 0) or at least `threshold` times the row's mean value
// (relative = 1; the means of a row sum to one, so that is threshold / S), ascending, written to
// indices[row][0 .. counts[row]); the rest of the row of `indices` is filled with -1.
__global__ void __launch_bounds__(TOPK_THREADS)
select_threshold_kernel(const float* __restrict__ colsum, long long ld, int S, float threshold, int relative,
                        int* __restrict__ indices, int* __restrict__ counts) {
    __shared__ unsigned warp_n[TOPK_THREADS / 32];
    __shared__ unsigned run_out;
    __shared__ float warp_sum[TOPK_THREADS / 32];
    const float* row = colsum + (long long)blockIdx.x * ld;
    int* out_idx = indices + (long long)blockIdx.x * S;
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    float thr = threshold;
    if (relative) {
        float part = 0.f;
        for (int i = tid; i < S; i += TOPK_THREADS) part += row[i];
        for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
        if (lane == 0) warp_sum[wid] = part;
        __syncthreads();
        float total = 0.f;
        for (int w = 0; w < TOPK_THREADS / 32; ++w) total += warp_sum[w];
        thr = threshold * total / (float)S;
    }
    if (tid == 0) run_out = 0;
    __syncthreads();
    for (int base = 0; base < S; base += TOPK_THREADS) {
        const int i = base + tid;
        const bool take = i < S && row[i] >= thr;
        const unsigned m = __ballot_sync(0xffffffffu, take);
        if (lane == 0) warp_n[wid] = __popc(m);
        __syncthreads();
        unsigned before = 0;
        for (int w = 0; w < wid; ++w) before += warp_n[w];
        before += __popc(m & ((1u << lane) - 1u));
        if (take) out_idx[run_out + before] = i;
        __syncthreads();
        if (tid == TOPK_THREADS - 1) run_out += before + (take ? 1u : 0u);
        __syncthreads();
    }
    const unsigned n = run_out;
    for (int i = (int)n + tid; i < S; i += TOPK_THREADS) out_idx[i] = -1;
    if (tid == 0) counts[blockIdx.x] = (int)n;
}

}  // namespace fcs
