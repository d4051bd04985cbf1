// CPU walk of the two-pass tile schedule, for tests only.
//
// It includes the same header the CUDA kernels use for planning, step
// iteration and mask rules, and evaluates each 128x128 score tile with plain
// loops, following the roles of the GPU kernels: two consumer groups that take
// alternate steps, their merge at the end of an item, the key-range partials
// and their merge, and the column pass with per-CTA accumulators that are added
// into the output at `flush` steps.  A schedule that skips, repeats or mis-masks
// a tile shows up as a mismatch against the CPU checker.
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <vector>

#include "../flash_colsum_b200/csrc/schedule.h"

using namespace fcs;

static float dot(const float* a, const float* b, int D) {
    float s = 0.f;
    for (int d = 0; d < D; ++d) s += a[d] * b[d];
    return s;
}

extern "C" int emulate_colsum(const float* q, const float* k, float* out, int B, int H, int Sq_full, int Sk,
                              int D, float scale, int causal, int k_past, int cls_n, int h_norm, int sms,
                              int* nsplit_out, long long* steps_out) {
    int Sq = Sq_full;
    if (!causal && cls_n > 0 && cls_n < Sq_full) Sq = cls_n;
    if (causal && k_past < 0) k_past = Sk > Sq ? Sk - Sq : 0;
    if (h_norm <= 0) h_norm = H;
    Problem p;
    memset(&p, 0, sizeof(p));
    plan(p, B, H, Sq, Sk, causal, k_past, sms);
    if (nsplit_out) *nsplit_out = p.nsplit;
    if (steps_out) *steps_out = p.steps_total;
    const float c = fabsf(scale) * 1.4426950408889634f;
    const float sgn = scale < 0 ? -1.f : 1.f;
    const float log2_norm = log2f((float)h_norm * (float)Sq);
    const long long rows_all = (long long)B * H * p.NQ * TILE;
    std::vector<float> neg_lse(rows_all, NAN);
    std::vector<float> part_m((size_t)rows_all * p.nsplit, NAN), part_l((size_t)rows_all * p.nsplit, NAN);
    for (long long i = 0; i < (long long)B * Sk; ++i) out[i] = 0.f;

    auto qrow = [&](int b, int h, int r) -> const float* {
        static std::vector<float> zero;
        if ((int)zero.size() < D) zero.assign(D, 0.f);
        return r < Sq ? q + (((size_t)b * H + h) * Sq_full + r) * D : zero.data();
    };
    auto krow = [&](int b, int h, int r) -> const float* {
        static std::vector<float> zero;
        if ((int)zero.size() < D) zero.assign(D, 0.f);
        return r < Sk ? k + (((size_t)b * H + h) * Sk + r) * D : zero.data();
    };

    // ---------------- statistics pass
    const int grid1 = (int)(p.stats_items < sms ? p.stats_items : sms);
    for (int cta = 0; cta < grid1; ++cta) {
        WorkIter<MODE_STATS> it;
        it.init(p, cta, grid1);
        float m[2][TILE], l[2][TILE];
        for (int g = 0; g < 2; ++g) for (int r = 0; r < TILE; ++r) { m[g][r] = -INFINITY; l[g][r] = 0.f; }
        for (int i = 0; !it.done; it.next(p), ++i) {
            const int g = i & 1;
            const bool full = stats_tile_full(p, it.qt, it.kt);
            for (int r = 0; r < TILE; ++r) {
                const int lim = stats_last_visible(p, it.qt, it.kt, r);
                if (full && lim < TILE - 1) return -10;   // the two mask rules disagree
                const float* qr = qrow(it.b, it.h, it.a_row() + r);
                float s[TILE], cm = -INFINITY;
                for (int j = 0; j < TILE; ++j) {
                    s[j] = (full || j <= lim) ? sgn * dot(qr, krow(it.b, it.h, it.b_row() + j), D) : -INFINITY;
                    cm = fmaxf(cm, s[j]);
                }
                const float scaled = (cm == -INFINITY) ? -INFINITY : cm * c;
                const float m_new = fmaxf(m[g][r], scaled);
                const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
                float ll = l[g][r] * exp2f(m[g][r] - m_safe);
                for (int j = 0; j < TILE; ++j)
                    if (s[j] != -INFINITY) ll += exp2f(s[j] * c - m_safe);
                l[g][r] = ll;
                m[g][r] = m_new;
            }
            if (it.last) {
                for (int r = 0; r < TILE; ++r) {
                    const float mm = fmaxf(m[0][r], m[1][r]);
                    const float ms = (mm == -INFINITY) ? 0.f : mm;
                    const float ll = l[0][r] * exp2f(m[0][r] - ms) + l[1][r] * exp2f(m[1][r] - ms);
                    const long long ridx = (((long long)it.b * H + it.h) * p.NQ + it.qt) * TILE + r;
                    if (p.nsplit == 1) {
                        if (!isnan(neg_lse[ridx])) return -11;   // row written twice
                        neg_lse[ridx] = (it.qt * TILE + r) < Sq ? -(mm + log2f(ll) + log2_norm) : -INFINITY;
                    } else {
                        const size_t pi = (size_t)it.sp * rows_all + ridx;
                        if (!isnan(part_m[pi])) return -12;
                        part_m[pi] = mm; part_l[pi] = ll;
                    }
                    m[0][r] = m[1][r] = -INFINITY; l[0][r] = l[1][r] = 0.f;
                }
            }
        }
    }
    if (p.nsplit > 1) {
        for (long long idx = 0; idx < rows_all; ++idx) {
            const int q_abs = (int)(idx % ((long long)p.NQ * TILE));
            float v = -INFINITY;
            if (q_abs < Sq) {
                float mm = -INFINITY, ll = 0.f;
                for (int s = 0; s < p.nsplit; ++s) {
                    if (isnan(part_m[(size_t)s * rows_all + idx])) return -13;   // partial never written
                    mm = fmaxf(mm, part_m[(size_t)s * rows_all + idx]);
                }
                for (int s = 0; s < p.nsplit; ++s)
                    ll += part_l[(size_t)s * rows_all + idx] * exp2f(part_m[(size_t)s * rows_all + idx] - mm);
                v = -(mm + log2f(ll) + log2_norm);
            }
            neg_lse[idx] = v;
        }
    }
    for (long long idx = 0; idx < rows_all; ++idx)
        if (isnan(neg_lse[idx])) return -14;   // a query row got no statistics

    // ---------------- column pass
    const int grid2 = (int)(p.steps_total < sms ? p.steps_total : sms);
    long long walked = 0;
    for (int cta = 0; cta < grid2; ++cta) {
        WorkIter<MODE_COLSUM> it;
        it.init(p, cta, grid2);
        float acc[TILE];
        for (int r = 0; r < TILE; ++r) acc[r] = 0.f;
        int cur_b = -1, cur_kt = -1;
        bool pending = false;
        for (; !it.done; it.next(p)) {
            ++walked;
            if (pending && (it.b != cur_b || it.kt != cur_kt)) return -20;   // left a key tile without flushing
            cur_b = it.b; cur_kt = it.kt; pending = true;
            if (it.qt < 0 || it.qt >= p.NQ || it.kt < 0 || it.kt >= p.NKC || it.h < 0 || it.h >= H || it.b >= B)
                return -21;
            const bool full = colsum_tile_full(p, it.kt, it.qt);
            const float* nl = neg_lse.data() + (((long long)it.b * H + it.h) * p.NQ + it.qt) * TILE;
            for (int r = 0; r < TILE; ++r) {
                const int thr = colsum_first_visible(p, it.kt, it.qt, r);
                if (full && thr > 0) return -22;
                const float* kr = krow(it.b, it.h, it.a_row() + r);
                for (int j = 0; j < TILE; ++j) {
                    if (!(full || j >= thr)) continue;
                    const float s = sgn * dot(kr, qrow(it.b, it.h, it.b_row() + j), D);
                    acc[r] += exp2f(s * c + nl[j]);
                }
            }
            if (it.flush) {
                for (int r = 0; r < TILE; ++r) {
                    const int k_abs = it.kt * TILE + r;
                    if (k_abs < Sk) out[(size_t)it.b * Sk + k_abs] += acc[r];
                    acc[r] = 0.f;
                }
                pending = false;
            }
        }
        if (pending) return -23;   // range ended with unflushed accumulators
    }
    if (walked != p.steps_total) return -24;
    return 0;
}
