// Column mean when only a handful of query rows enter it (a CLS prefix, or a few
// decode queries): per (batch, head) the work is R dot products per key, i.e. a
// matrix-vector product that reads every key once.  That is bound by HBM, not
// by the tensor cores, so it runs as plain loads: one CTA per (b, h), one thread
// per key row, scores kept in shared memory between the three sweeps (scores and
// maximum; exp2 and sum; normalise and add into the output).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "sm100_ptx.cuh"

namespace fcs {

constexpr int SMALLQ_MAX_ROWS = 4;
constexpr int SMALLQ_THREADS = 256;
constexpr size_t SMALLQ_MAX_SMEM = 200 * 1024;

struct SmallQParams {
    const void* q;
    const void* k;
    float* out;
    long long out_ld;
    int H, R, Sk;
    long long qsb, qsh, qss, ksb, ksh, kss;   // strides in elements
    float c;          // scale * log2(e), sign included
    int causal, k_past;
    float inv_norm;   // 1 / (h_norm * R)
};

inline size_t smallq_smem_bytes(int R, int Sk, int D) {
    return (size_t)R * D * 4 + (size_t)R * Sk * 4 + (SMALLQ_THREADS / 32) * SMALLQ_MAX_ROWS * 4 + 64;
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

// max or sum over the CTA of R per-thread values; result in red_out[0..R)
template <bool IS_MAX>
__device__ __forceinline__ void block_reduce(float (&v)[SMALLQ_MAX_ROWS], int R, float* red, float* red_out) {
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

// RMAX: compile-time bound on the query rows (1, 2 or 4); fewer rows need fewer
// registers, so that four CTAs fit on an SM and a 512-CTA grid runs as one wave.
template <int D, bool BF16, int RMAX>
__global__ void __launch_bounds__(SMALLQ_THREADS, 4)
colsum_small_q_kernel(const SmallQParams p) {
    extern __shared__ float smallq_smem[];
    float* qs = smallq_smem;                       // [R][D], scaled by c
    float* sc = qs + p.R * D;                      // [R][Sk]
    float* red = sc + (size_t)p.R * p.Sk;          // [warps][MAX_ROWS]
    float* red_out = red + (SMALLQ_THREADS / 32) * SMALLQ_MAX_ROWS;   // [MAX_ROWS] (+ spare)
    const int b = blockIdx.x / p.H, h = blockIdx.x % p.H;
    const uint16_t* qb = reinterpret_cast<const uint16_t*>(p.q) + b * p.qsb + h * p.qsh;
    const uint16_t* kb = reinterpret_cast<const uint16_t*>(p.k) + b * p.ksb + h * p.ksh;

    for (int i = threadIdx.x; i < p.R * D; i += SMALLQ_THREADS) {
        const int r = i / D, d = i % D;
        const uint32_t raw = qb[r * p.qss + d];
        const float v = BF16 ? __uint_as_float(raw << 16) : __half2float(__ushort_as_half((unsigned short)raw));
        qs[i] = v * p.c;
    }
    __syncthreads();

    // sweep 1: scores (log2 domain) and their maximum.  D/8 adjacent lanes share a
    // key row, 16 bytes each, so that a warp reads whole 128-byte lines; the
    // partial dot products are combined with shuffles.
    constexpr int LPR = D / 8;            // lanes per key row
    constexpr int RPW = 32 / LPR;         // key rows per warp and load
    constexpr int UNROLL = 4;             // independent loads in flight per lane
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int piece = lane % LPR, sub = lane / LPR;
    float qreg[RMAX][8];
#pragma unroll
    for (int r = 0; r < RMAX; ++r)
#pragma unroll
        for (int e = 0; e < 8; ++e) qreg[r][e] = (r < p.R) ? qs[r * D + piece * 8 + e] : 0.f;
    float vmax[SMALLQ_MAX_ROWS];
#pragma unroll
    for (int r = 0; r < SMALLQ_MAX_ROWS; ++r) vmax[r] = -INFINITY;
    constexpr int ROWS_PER_ITER = (SMALLQ_THREADS / 32) * RPW * UNROLL;
    for (int k0 = 0; k0 < p.Sk; k0 += ROWS_PER_ITER) {
        uint4 raw[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k = k0 + (u * (SMALLQ_THREADS / 32) + warp) * RPW + sub;
            raw[u] = (k < p.Sk) ? __ldg(reinterpret_cast<const uint4*>(kb + k * p.kss) + piece)
                                : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k = k0 + (u * (SMALLQ_THREADS / 32) + warp) * RPW + sub;
            const float2 f0 = unpack16x2<BF16>(raw[u].x), f1 = unpack16x2<BF16>(raw[u].y);
            const float2 f2 = unpack16x2<BF16>(raw[u].z), f3 = unpack16x2<BF16>(raw[u].w);
#pragma unroll
            for (int r = 0; r < RMAX; ++r) {
                if (r < p.R) {      // uniform across the CTA
                    float d = f0.x * qreg[r][0] + f0.y * qreg[r][1] + f1.x * qreg[r][2] + f1.y * qreg[r][3] +
                              f2.x * qreg[r][4] + f2.y * qreg[r][5] + f3.x * qreg[r][6] + f3.y * qreg[r][7];
#pragma unroll
                    for (int o = LPR / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
                    if (piece == 0 && k < p.Sk) {
                        const bool visible = !p.causal || (k <= p.k_past + r);
                        const float sv = visible ? d : -INFINITY;
                        sc[(size_t)r * p.Sk + k] = sv;
                        vmax[r] = fmaxf(vmax[r], sv);
                    }
                }
            }
        }
    }
    block_reduce<true>(vmax, p.R, red, red_out);
    float m[SMALLQ_MAX_ROWS];
#pragma unroll
    for (int r = 0; r < SMALLQ_MAX_ROWS; ++r) m[r] = red_out[r];
    __syncthreads();

    // sweep 2: exp2 and their sum
    float vsum[SMALLQ_MAX_ROWS] = {0.f, 0.f, 0.f, 0.f};
    for (int k = threadIdx.x; k < p.Sk; k += SMALLQ_THREADS) {
#pragma unroll
        for (int r = 0; r < SMALLQ_MAX_ROWS; ++r) {
            if (r < p.R) {
                const float e = ex2_approx(sc[(size_t)r * p.Sk + k] - m[r]);
                sc[(size_t)r * p.Sk + k] = e;
                vsum[r] += e;
            }
        }
    }
    block_reduce<false>(vsum, p.R, red, red_out);
    float w[SMALLQ_MAX_ROWS];
#pragma unroll
    for (int r = 0; r < SMALLQ_MAX_ROWS; ++r) w[r] = (r < p.R) ? p.inv_norm / red_out[r] : 0.f;

    // sweep 3: this head's share of the column means
    float* ob = p.out + (long long)b * p.out_ld;
    for (int k = threadIdx.x; k < p.Sk; k += SMALLQ_THREADS) {
        float v = 0.f;
#pragma unroll
        for (int r = 0; r < SMALLQ_MAX_ROWS; ++r)
            if (r < p.R) v += sc[(size_t)r * p.Sk + k] * w[r];
        atomicAdd_system(ob + k, v);   // `out` may live on another GPU
    }
}

}  // namespace fcs
