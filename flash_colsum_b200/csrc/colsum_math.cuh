// Per-thread arithmetic of the consumer warps: what is done with the scores of
// one accumulator row once they are in registers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>

#include "sm100_ptx.cuh"

namespace fcs {

// Of every 16 pairs of exps on fully visible tiles, this many are evaluated by
// the polynomial on the FMA pipe instead of the special-function unit (which
// issues 16 results per clock per SM and is the busiest unit of both passes).
#ifndef FCS_POLY_PAIRS
#define FCS_POLY_PAIRS 5
#endif
__host__ __device__ constexpr bool pair_uses_polynomial(int pair) {
    return ((pair * FCS_POLY_PAIRS) % 16) < FCS_POLY_PAIRS;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// Online (max, sum) update of one query row with 32 more scores.
// `last_valid`: columns 0..last_valid are visible (>= 31: all).
template <bool MASKED>
__device__ __forceinline__ void stats_block32(const uint32_t (&r)[32], int last_valid, float c, float& m,
                                              float& l) {
    float s[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        s[j] = __uint_as_float(r[j]);
        if (MASKED) s[j] = (j <= last_valid) ? s[j] : -INFINITY;
    }
    float m0 = max3(s[0], s[1], s[2]), m1 = max3(s[3], s[4], s[5]);
    float m2 = max3(s[6], s[7], s[8]), m3 = max3(s[9], s[10], s[11]);
#pragma unroll
    for (int j = 12; j < 28; j += 8) {
        m0 = max3(m0, s[j], s[j + 1]);
        m1 = max3(m1, s[j + 2], s[j + 3]);
        m2 = max3(m2, s[j + 4], s[j + 5]);
        m3 = max3(m3, s[j + 6], s[j + 7]);
    }
    m0 = max3(m0, s[28], s[29]);
    m1 = max3(m1, s[30], s[31]);
    const float cm = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
    float m_safe;
    if (MASKED) {   // a row may see nothing of this block (or nothing yet): keep -inf out of the arithmetic
        const float scaled = (cm == -INFINITY) ? -INFINITY : cm * c;
        const float m_new = fmaxf(m, scaled);
        m_safe = (m_new == -INFINITY) ? 0.f : m_new;
        l *= ex2_approx(m - m_safe);
        m = m_new;
    } else {        // all 32 scores are finite
        m_safe = fmaxf(m, cm * c);
        l *= ex2_approx(m - m_safe);
        m = m_safe;
    }
    if constexpr (!MASKED) {
        const f32x2 c2 = pack2(c, c), nm2 = pack2(-m_safe, -m_safe);
        f32x2 s0 = pack2(0.f, 0.f), s1 = s0;
#pragma unroll
        for (int pr = 0; pr < 16; ++pr) {
            const f32x2 t = fma2(pack2(s[2 * pr], s[2 * pr + 1]), c2, nm2);
            f32x2 e;
            if (pair_uses_polynomial(pr)) {
                e = ex2_poly2(t);
            } else {
                float t0, t1;
                unpack2(t, t0, t1);
                e = pack2(ex2_approx(t0), ex2_approx(t1));
            }
            if (pr & 1) s1 = add2(s1, e); else s0 = add2(s0, e);
        }
        float x0, x1;
        unpack2(add2(s0, s1), x0, x1);
        l += x0 + x1;
    } else {
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
            float t0 = fmaf(s[j], c, -m_safe), t1 = fmaf(s[j + 1], c, -m_safe);
            float t2 = fmaf(s[j + 2], c, -m_safe), t3 = fmaf(s[j + 3], c, -m_safe);
            // c may be 0 and s -inf: select after the multiply
            t0 = (j <= last_valid) ? t0 : -INFINITY;
            t1 = (j + 1 <= last_valid) ? t1 : -INFINITY;
            t2 = (j + 2 <= last_valid) ? t2 : -INFINITY;
            t3 = (j + 3 <= last_valid) ? t3 : -INFINITY;
            a0 += ex2_approx(t0); a1 += ex2_approx(t1);
            a2 += ex2_approx(t2); a3 += ex2_approx(t3);
        }
        l += (a0 + a1) + (a2 + a3);
    }
}

// Add exp2(c*s - lse[q]) of 32 query columns into a key's accumulators.  `nl`
// points at the 32 values -(lse) of these columns in shared memory.  Columns
// first_valid <= j < end_valid of this chunk are visible.
template <bool MASKED>
__device__ __forceinline__ void colsum_chunk(const uint32_t (&r)[32], const float4* nl, int first_valid,
                                             int end_valid, float c, float (&acc)[4]) {
    if constexpr (!MASKED) {
        const f32x2 c2 = pack2(c, c);
        f32x2 a01 = pack2(acc[0], acc[1]), a23 = pack2(acc[2], acc[3]);
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
            const float4 n = nl[j >> 2];
            const f32x2 ta = fma2(pack2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])), c2, pack2(n.x, n.y));
            const f32x2 tb = fma2(pack2(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3])), c2, pack2(n.z, n.w));
            f32x2 ea, eb;
            float u0, u1;
            if (pair_uses_polynomial((j >> 1) & 15)) { ea = ex2_poly2(ta); }
            else { unpack2(ta, u0, u1); ea = pack2(ex2_approx(u0), ex2_approx(u1)); }
            if (pair_uses_polynomial(((j >> 1) + 1) & 15)) { eb = ex2_poly2(tb); }
            else { unpack2(tb, u0, u1); eb = pack2(ex2_approx(u0), ex2_approx(u1)); }
            a01 = add2(a01, ea);
            a23 = add2(a23, eb);
        }
        unpack2(a01, acc[0], acc[1]);
        unpack2(a23, acc[2], acc[3]);
    } else {
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
        const float4 n = nl[j >> 2];
        float t0 = fmaf(__uint_as_float(r[j]), c, n.x);
        float t1 = fmaf(__uint_as_float(r[j + 1]), c, n.y);
        float t2 = fmaf(__uint_as_float(r[j + 2]), c, n.z);
        float t3 = fmaf(__uint_as_float(r[j + 3]), c, n.w);
        if (MASKED) {
            t0 = (j >= first_valid && j < end_valid) ? t0 : -INFINITY;
            t1 = (j + 1 >= first_valid && j + 1 < end_valid) ? t1 : -INFINITY;
            t2 = (j + 2 >= first_valid && j + 2 < end_valid) ? t2 : -INFINITY;
            t3 = (j + 3 >= first_valid && j + 3 < end_valid) ? t3 : -INFINITY;
        }
        acc[0] += ex2_approx(t0); acc[1] += ex2_approx(t1);
        acc[2] += ex2_approx(t2); acc[3] += ex2_approx(t3);
    }
    }
}

// ---------------------------------------------------------------------------
// Folding -(lse) into the MMA of the column pass.  The column pass needs
// exp2(c*s + nl[q]) with nl[q] constant down a column; loading it per element
// costs as much issue bandwidth as the exp itself.  Instead the contraction is
// extended by 16: the query block gets 16 more "features" holding v = nl/c as
// three 16-bit parts (hi + mid + lo, exact to ~2^-24 relative), the key tile
// gets a constant in the same three positions, so the accumulator already holds
// s + v and the consumers only multiply by c.
// fp16 parts are stored divided by 256 (the key-side constant is 256) so that
// |v| up to ~1.6e7 stays in range; bf16 needs no scaling.
// ---------------------------------------------------------------------------
constexpr float EXT_FP16_SCALE = 256.f;
constexpr float EXT_PAD_VALUE = -1.0e6f;   // stands in for -inf on rows that must add nothing

// The 32-byte row for one query: element 0..2 = hi, mid, lo, the rest zero.
// `inv_c` carries the sign of the scale: a negative scale negates the key-side
// operand of the MMA (and with it the key-side constant), so the parts are
// stored negated.
__device__ __forceinline__ void make_ext_row(float nl, float inv_c, bool bf16, uint4& first, uint4& second) {
    float v = (nl == -INFINITY) ? copysignf(EXT_PAD_VALUE, -inv_c) : nl * inv_c;
    unsigned short hi, mid, lo;
    if (bf16) {
        const __nv_bfloat16 a = __float2bfloat16_rn(v);
        const float r1 = v - __bfloat162float(a);
        const __nv_bfloat16 b = __float2bfloat16_rn(r1);
        const __nv_bfloat16 c3 = __float2bfloat16_rn(r1 - __bfloat162float(b));
        hi = __bfloat16_as_ushort(a); mid = __bfloat16_as_ushort(b); lo = __bfloat16_as_ushort(c3);
    } else {
        v *= (1.f / EXT_FP16_SCALE);
        const __half a = __float2half_rn(v);
        const float r1 = v - __half2float(a);
        const __half b = __float2half_rn(r1);
        const __half c3 = __float2half_rn(r1 - __half2float(b));
        hi = __half_as_ushort(a); mid = __half_as_ushort(b); lo = __half_as_ushort(c3);
    }
    first = make_uint4((uint32_t)hi | ((uint32_t)mid << 16), (uint32_t)lo, 0u, 0u);
    second = make_uint4(0u, 0u, 0u, 0u);
}

// Column-pass chunk when the accumulator already holds s + nl/c: add exp2(c * acc).
template <bool MASKED>
__device__ __forceinline__ void colsum_chunk_ext(const uint32_t (&r)[32], int first_valid, int end_valid, float c,
                                                 float (&acc)[4]) {
    const f32x2 c2 = pack2(c, c);
    if constexpr (!MASKED) {
        f32x2 a01 = pack2(acc[0], acc[1]), a23 = pack2(acc[2], acc[3]);
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
            const f32x2 ta = mul2(pack2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])), c2);
            const f32x2 tb = mul2(pack2(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3])), c2);
            f32x2 ea, eb;
            float u0, u1;
            if (pair_uses_polynomial((j >> 1) & 15)) { ea = ex2_poly2(ta); }
            else { unpack2(ta, u0, u1); ea = pack2(ex2_approx(u0), ex2_approx(u1)); }
            if (pair_uses_polynomial(((j >> 1) + 1) & 15)) { eb = ex2_poly2(tb); }
            else { unpack2(tb, u0, u1); eb = pack2(ex2_approx(u0), ex2_approx(u1)); }
            a01 = add2(a01, ea);
            a23 = add2(a23, eb);
        }
        unpack2(a01, acc[0], acc[1]);
        unpack2(a23, acc[2], acc[3]);
    } else {
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
            float t0 = __uint_as_float(r[j]) * c, t1 = __uint_as_float(r[j + 1]) * c;
            float t2 = __uint_as_float(r[j + 2]) * c, t3 = __uint_as_float(r[j + 3]) * c;
            t0 = (j >= first_valid && j < end_valid) ? t0 : -INFINITY;
            t1 = (j + 1 >= first_valid && j + 1 < end_valid) ? t1 : -INFINITY;
            t2 = (j + 2 >= first_valid && j + 2 < end_valid) ? t2 : -INFINITY;
            t3 = (j + 3 >= first_valid && j + 3 < end_valid) ? t3 : -INFINITY;
            acc[0] += ex2_approx(t0); acc[1] += ex2_approx(t1);
            acc[2] += ex2_approx(t2); acc[3] += ex2_approx(t3);
        }
    }
}

// The unmasked column-pass chunk for 16 columns (pairs PAIR0 .. PAIR0 + 7 of the 16-pair pattern).
template <int PAIR0>
__device__ __forceinline__ void colsum_chunk16_ext(const uint32_t (&r)[16], float c, float (&acc)[4]) {
    const f32x2 c2 = pack2(c, c);
    f32x2 a01 = pack2(acc[0], acc[1]), a23 = pack2(acc[2], acc[3]);
#pragma unroll
    for (int j = 0; j < 16; j += 4) {
        const f32x2 ta = mul2(pack2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])), c2);
        const f32x2 tb = mul2(pack2(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3])), c2);
        f32x2 ea, eb;
        float u0, u1;
        if (pair_uses_polynomial((PAIR0 + (j >> 1)) & 15)) { ea = ex2_poly2(ta); }
        else { unpack2(ta, u0, u1); ea = pack2(ex2_approx(u0), ex2_approx(u1)); }
        if (pair_uses_polynomial((PAIR0 + (j >> 1) + 1) & 15)) { eb = ex2_poly2(tb); }
        else { unpack2(tb, u0, u1); eb = pack2(ex2_approx(u0), ex2_approx(u1)); }
        a01 = add2(a01, ea);
        a23 = add2(a23, eb);
    }
    unpack2(a01, acc[0], acc[1]);
    unpack2(a23, acc[2], acc[3]);
}

}  // namespace fcs
