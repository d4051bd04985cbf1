// CPU walk of the two-pass tile schedule, for tests only.
//
// It includes the same header the CUDA kernels use for planning, item/step
// iteration and mask rules, and evaluates each 128x256 score tile with plain
// loops, following the roles of the GPU kernels: four consumer groups that each
// own 64 of the 256 columns, their merge at the end of an item, the key-range
// partials and their merge, and the column pass with per-CTA accumulators that
// are added into the output after `flush` items.  A schedule that skips, repeats or mis-masks
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
                              long long interleave_min_rows, int* nsplit_out, long long* steps_out) {
    int Sq = Sq_full;
    if (!causal && cls_n > 0 && cls_n < Sq_full) Sq = cls_n;
    if (causal && k_past < 0) k_past = Sk > Sq ? Sk - Sq : 0;
    if (h_norm <= 0) h_norm = H;
    Problem p;
    memset(&p, 0, sizeof(p));
    plan(p, B, H, Sq, Sk, causal, k_past, sms, interleave_min_rows);
    if (nsplit_out) *nsplit_out = p.nsplit;
    if (steps_out) *steps_out = p.steps_total;
    const float c = fabsf(scale) * 1.4426950408889634f;
    const float sgn = scale < 0 ? -1.f : 1.f;
    const float log2_norm = log2f((float)h_norm * (float)Sq);
    const long long part_rows = (long long)B * H * p.NQ * TILE;
    std::vector<float> neg_lse((size_t)B * H * p.lse_rows, NAN);
    std::vector<float> part_m((size_t)part_rows * p.nsplit, NAN), part_l((size_t)part_rows * p.nsplit, NAN);
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

    // ---------------- statistics pass: items of (query tile, key range), 256-key steps,
    // four consumer groups each owning 64 of the 256 columns
    const int grid1 = (int)(p.stats_items < sms ? p.stats_items : sms);
    const int G = 4, GC = BLOCK / G;
    for (int cta = 0; cta < grid1; ++cta) {
        StatsItems it;
        it.init(p, cta, grid1);
        for (; !it.done; it.next(p)) {
            if (it.s0 >= it.s1) return -15;   // an item without steps would never write its rows
            float m[4][TILE], l[4][TILE];
            for (int g = 0; g < G; ++g) for (int r = 0; r < TILE; ++r) { m[g][r] = -INFINITY; l[g][r] = 0.f; }
            int f_lo, f_hi;
            stats_full_range(p, it.qt, f_lo, f_hi);
            for (int st = it.s0; st < it.s1; ++st) {
                const bool full = stats_tile_full(p, it.qt, st);
                if (full != (st >= f_lo && st < f_hi)) return -17;   // the range form of the rule disagrees
                for (int g = 0; g < G; ++g) {
                    const int col0 = g * GC;
                    const bool skip = !full && (stats_last_visible(p, it.qt, st, TILE - 1) - col0 < 0);
                    for (int r = 0; r < TILE; ++r) {
                        const int lim = stats_last_visible(p, it.qt, st, r) - col0;
                        if (full && lim < GC - 1) return -10;   // the two mask rules disagree
                        if (skip) { if (lim >= 0) return -16; continue; }   // skipped a visible element
                        const float* qr = qrow(it.b, it.h, it.a_row() + r);
                        float s[GC], cm = -INFINITY;
                        for (int j = 0; j < GC; ++j) {
                            s[j] = (full || j <= lim) ? sgn * dot(qr, krow(it.b, it.h, it.b_row(st) + col0 + j), D)
                                                      : -INFINITY;
                            cm = fmaxf(cm, s[j]);
                        }
                        const float scaled = (cm == -INFINITY) ? -INFINITY : cm * c;
                        const float m_new = fmaxf(m[g][r], scaled);
                        const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
                        float ll = l[g][r] * exp2f(m[g][r] - m_safe);
                        for (int j = 0; j < GC; ++j)
                            if (s[j] != -INFINITY) ll += exp2f(s[j] * c - m_safe);
                        l[g][r] = ll;
                        m[g][r] = m_new;
                    }
                }
            }
            for (int r = 0; r < TILE; ++r) {
                float mm = -INFINITY;
                for (int g = 0; g < G; ++g) mm = fmaxf(mm, m[g][r]);
                const float ms = (mm == -INFINITY) ? 0.f : mm;
                float ll = 0.f;
                for (int g = 0; g < G; ++g) ll += l[g][r] * exp2f(m[g][r] - ms);
                const long long bh = (long long)it.b * H + it.h;
                const int q_abs = it.qt * TILE + r;
                if (p.nsplit == 1) {
                    const long long ridx = bh * p.lse_rows + q_abs;
                    if (!isnan(neg_lse[ridx])) return -11;   // row written twice
                    neg_lse[ridx] = q_abs < Sq ? -(mm + log2f(ll) + log2_norm) : -INFINITY;
                } else {
                    const size_t pi = ((size_t)it.sp * B * H + bh) * ((size_t)p.NQ * TILE) + q_abs;
                    if (!isnan(part_m[pi])) return -12;
                    part_m[pi] = mm; part_l[pi] = ll;
                }
            }
        }
    }
    if (p.nsplit > 1) {
        const long long rows = (long long)p.NQ * TILE;
        for (long long idx = 0; idx < part_rows; ++idx) {
            const long long bh = idx / rows;
            const int q_abs = (int)(idx - bh * rows);
            float v = -INFINITY;
            if (q_abs < Sq) {
                float mm = -INFINITY, ll = 0.f;
                for (int s = 0; s < p.nsplit; ++s) {
                    if (isnan(part_m[(size_t)s * part_rows + idx])) return -13;   // partial never written
                    mm = fmaxf(mm, part_m[(size_t)s * part_rows + idx]);
                }
                for (int s = 0; s < p.nsplit; ++s)
                    ll += part_l[(size_t)s * part_rows + idx] * exp2f(part_m[(size_t)s * part_rows + idx] - mm);
                v = -(mm + log2f(ll) + log2_norm);
            }
            neg_lse[bh * p.lse_rows + q_abs] = v;
        }
    }
    for (long long bh = 0; bh < (long long)B * H; ++bh)
        for (int q = 0; q < Sq; ++q)
            if (isnan(neg_lse[bh * p.lse_rows + q])) return -14;   // a query row got no statistics

    // ---------------- column pass: contiguous step ranges, 256-query steps
    long long col_items = p.steps_total;
    if (p.col_interleave == COL_HEAD_MAJOR) col_items = (long long)B * H * ceil_div(p.NKC, p.col_pack);
    const int grid2 = (int)(col_items < sms ? col_items : sms);
    long long walked = 0;
    if (p.col_interleave == COL_HEAD_MAJOR) {
        // one query block, contiguous runs of the (b, h, key tiles) list; every item flushes
        const int GQ = p.col_pack == 2 ? GC : BLOCK;       // query columns a consumer group covers
        const int NG = p.col_pack == 2 ? 2 : 1;
        if (p.NQB == 2) {
            // two resident query blocks: an item is one key tile against the blocks that see it
            for (int cta = 0; cta < grid2; ++cta) {
                ResidentItems it;
                it.init(p, cta, grid2);
                for (; !it.done; it.next(p)) {
                    if (!it.flush() || it.kt < 0 || it.kt >= p.NKC || it.h < 0 || it.h >= H || it.b < 0 || it.b >= B ||
                        it.s0 < 0 || it.s0 >= it.s1 || it.s1 != p.NQB)
                        return -29;
                    const float* nl_bh = neg_lse.data() + ((long long)it.b * H + it.h) * p.lse_rows;
                    for (int st = 0; st < p.NQB; ++st) {
                        const bool taken = st >= it.s0 && st < it.s1;
                        if (taken) ++walked;
                        const int end = colsum_end_visible(p, st);
                        for (int r = 0; r < TILE; ++r) {
                            const int thr = colsum_first_visible(p, it.kt, st, r);
                            const int k_abs = it.kt * TILE + r;
                            const float* kr = krow(it.b, it.h, k_abs);
                            for (int j = thr; j < end; ++j) {
                                if (!taken) return -30;   // a block with visible elements was left out
                                const float sc = sgn * dot(kr, qrow(it.b, it.h, st * BLOCK + j), D);
                                if (k_abs < Sk) out[(size_t)it.b * Sk + k_abs] += exp2f(sc * c + nl_bh[st * BLOCK + j]);
                            }
                        }
                    }
                }
            }
            if (walked != p.steps_total) return -24;
            return 0;
        }
        for (int cta = 0; cta < grid2; ++cta) {
            PackedItems it;
            it.init(p, cta, grid2);
            for (; !it.done; it.next(p)) {
                if (!it.flush() || it.nt < 1 || it.nt > p.col_pack || it.kt + it.nt > p.NKC || it.kt < 0 ||
                    it.h < 0 || it.h >= H || it.b < 0 || it.b >= B || (it.kt % p.col_pack))
                    return -28;
                const float* nl = neg_lse.data() + ((long long)it.b * H + it.h) * p.lse_rows;
                for (int tg = 0; tg < it.nt; ++tg) {
                    const int ktg = it.kt + tg;
                    ++walked;
                    for (int g2 = 0; g2 < NG; ++g2) {
                        const int q0 = g2 * GQ;
                        const int end = colsum_end_visible(p, 0) - q0;
                        const bool skip = !(end > 0 && colsum_first_visible(p, ktg, 0, 0) - q0 < GQ);
                        const bool full = end >= GQ && colsum_first_visible(p, ktg, 0, TILE - 1) - q0 <= 0;
                        for (int r = 0; r < TILE; ++r) {
                            const int thr = colsum_first_visible(p, ktg, 0, r) - q0;
                            const int k_abs = ktg * TILE + r;
                            const float* kr = krow(it.b, it.h, k_abs);
                            for (int j = 0; j < GQ; ++j) {
                                const bool vis = (j >= thr && j < end);
                                if (full && !vis) return -22;
                                if (!vis) continue;
                                if (skip) return -26;
                                const float sc = sgn * dot(kr, qrow(it.b, it.h, q0 + j), D);
                                if (k_abs < Sk) out[(size_t)it.b * Sk + k_abs] += exp2f(sc * c + nl[q0 + j]);
                            }
                        }
                    }
                }
            }
        }
        if (walked != p.steps_total) return -24;
        return 0;
    }
    for (int cta = 0; cta < grid2; ++cta) {
        ColsumItems it;
        it.init(p, cta, grid2);
        float acc[TILE];
        for (int r = 0; r < TILE; ++r) acc[r] = 0.f;
        int cur_b = -1, cur_kt = -1;
        bool pending = false;
        for (; !it.done; it.next(p)) {
            if (it.s0 >= it.s1) return -25;
            if (pending && (it.b != cur_b || it.kt != cur_kt)) return -20;   // left a key tile without flushing
            cur_b = it.b; cur_kt = it.kt; pending = true;
            if (it.s0 < 0 || it.s1 > p.NQB || it.kt < 0 || it.kt >= p.NKC || it.h < 0 || it.h >= H || it.b >= B)
                return -21;
            const float* nl_bh = neg_lse.data() + ((long long)it.b * H + it.h) * p.lse_rows;
            int f_lo, f_hi;
            colsum_full_range(p, it.kt, f_lo, f_hi);
            for (int st = it.s0; st < it.s1; ++st) {
                ++walked;
                const bool full = colsum_tile_full(p, it.kt, st);
                if (full != (st >= f_lo && st < f_hi)) return -27;   // the range form of the rule disagrees
                const float* nl = nl_bh + (long long)st * BLOCK;
                for (int g = 0; g < G; ++g) {
                    const int col0 = g * GC;
                    const int end = colsum_end_visible(p, st) - col0;
                    const bool skip = !full && !(end > 0 && colsum_first_visible(p, it.kt, st, 0) - col0 < GC);
                    for (int r = 0; r < TILE; ++r) {
                        const int thr = colsum_first_visible(p, it.kt, st, r) - col0;
                        if (full && (thr > 0 || end < GC)) return -22;
                        const float* kr = krow(it.b, it.h, it.a_row() + r);
                        for (int j = 0; j < GC; ++j) {
                            const bool vis = full || (j >= thr && j < end);
                            if (!vis) continue;
                            if (skip) return -26;   // skipped a visible element
                            const float s = sgn * dot(kr, qrow(it.b, it.h, it.b_row(st) + col0 + j), D);
                            acc[r] += exp2f(s * c + nl[col0 + j]);
                        }
                    }
                }
            }
            if (it.flush()) {
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

// Walk the single-pass kernel's work split: every (pair, query tile) must be visited exactly
// once, in list order, by the clusters in turn; the tile counter of a share must agree with
// `tile_of`; flush groups must not span batch entries nor exceed `flush_units` pairs.
extern "C" int check_tile_ranges(long long units, int NQ, int H, int clusters, int flush_units) {
    long long expect = 0;
    for (int c = 0; c < clusters; ++c) {
        TileRange r;
        r.init(units, NQ, c, clusters);
        if (r.g0 != expect) return -1;
        int i = 0, group_first = r.u0;
        for (int u = r.u0; u < r.u1; ++u) {
            if (r.t_lo(u) >= r.t_hi(u)) return -2;               // a touched pair without tiles
            for (int t = r.t_lo(u); t < r.t_hi(u); ++t, ++i) {
                if ((long long)u * NQ + t != expect) return -3;  // out of order, skipped or repeated
                if (r.tile_of(i) != t) return -4;
                ++expect;
            }
            if (r.flush_after(u, H, flush_units)) {
                if (group_first / H != u / H) return -5;          // a group spans two batch entries
                if (u - group_first + 1 > flush_units) return -6;
                group_first = u + 1;
            } else if (u + 1 == r.u1) {
                return -7;                                        // the share ends without a flush
            }
        }
        if (i != r.tiles() || expect != r.g1) return -8;
    }
    return expect == units * NQ ? 0 : -9;
}

// Scratch bytes the two streaming passes use for a call planned with this k_past on `sms`
// SMs: the plan and the layout of the kernels' own header, as the library's call computes them.
extern "C" long long scratch_need(int B, int H, int Sq, int Sk, int causal, int k_past, int sms, int* nsplit_out) {
    if (causal && k_past < 0) k_past = Sk > Sq ? Sk - Sq : 0;
    Problem p;
    memset(&p, 0, sizeof(p));
    plan(p, B, H, Sq, Sk, causal, k_past, sms);
    if (nsplit_out) *nsplit_out = p.nsplit;
    return (long long)workspace_layout(p, nullptr);
}

// The one-kernel form for short query axes: plan a call, then walk every CTA's run of key blocks the
// way the kernel does and check, element by element, that the mask rules of its two phases (row
// statistics with lane = query, column sums with lane = key) both see exactly the (query, key) pairs
// of the definition, each once.  Returns 0 when the plan declines the call, cl * 1000 + bpc when it
// takes it and the walk is clean, a negative code otherwise.
extern "C" int check_fused_short(int B, int H, int Sq, int Sk, int causal, int k_past, int sms,
                                 const int* max_clusters, int force) {
    if (causal && k_past < 0) k_past = Sk > Sq ? Sk - Sq : 0;
    if (!causal) k_past = 0;
    int cl = 0, nkb = 0, bpc = 0;
    if (!fused_short_plan(B, H, Sq, Sk, causal, k_past, sms, max_clusters, force != 0, &cl, &nkb, &bpc)) return 0;
    if (cl < 1 || cl > FUSED_SHORT_MAX_CLUSTER || bpc < 1) return -1;
    if ((long long)cl * bpc < nkb || (long long)(cl - 1) * bpc >= nkb) return -2;   // a CTA without a block
    Problem p;
    memset(&p, 0, sizeof(p));
    p.B = B; p.H = H; p.Sq = Sq; p.Sk = Sk; p.causal = causal; p.k_past = k_past;
    std::vector<int> seen_stats((size_t)Sq * Sk, 0), seen_cols((size_t)Sq * Sk, 0);
    int f_lo, f_hi;
    stats_full_range(p, 0, f_lo, f_hi);
    for (int r = 0; r < cl; ++r) {
        int kb0 = r * bpc, kb1 = kb0 + bpc;
        if (kb1 > nkb) kb1 = nkb;
        for (int kb = kb0; kb < kb1; ++kb) {
            // phase 1: rows are queries, columns the 256 keys of the block
            for (int row = 0; row < TILE; ++row) {
                const int lim = (kb >= f_lo && kb < f_hi) ? BLOCK - 1 : stats_last_visible(p, 0, kb, row);
                for (int col = 0; col <= lim && col < BLOCK; ++col) {
                    const long long key = (long long)kb * BLOCK + col;
                    if (row >= Sq) continue;              // padding rows: their statistics are dropped
                    if (key >= Sk) return -3;
                    ++seen_stats[(size_t)row * Sk + key];
                }
            }
            // phase 2: rows are the keys of a 128-key tile, columns the queries
            for (int t = 0; t < 2; ++t) {
                const int ktg = kb * 2 + t;
                const int end = colsum_end_visible(p, 0);
                for (int row = 0; row < TILE; ++row) {
                    const long long key = (long long)ktg * TILE + row;
                    const int first = colsum_first_visible(p, ktg, 0, row);
                    for (int qc = first; qc < end; ++qc) {
                        if (key >= Sk) continue;          // lanes past the key axis are not added
                        ++seen_cols[(size_t)qc * Sk + key];
                    }
                }
            }
        }
    }
    for (int qi = 0; qi < Sq; ++qi)
        for (int key = 0; key < Sk; ++key) {
            const int want = (!causal || key <= (long long)k_past + qi) ? 1 : 0;
            if (seen_stats[(size_t)qi * Sk + key] != want) return -4;
            if (seen_cols[(size_t)qi * Sk + key] != want) return -5;
        }
    return cl * 1000 + bpc;
}

// StatsItems::next with the grid's digits against a fresh decode of every item index: walks every
// CTA's items of a planned call.  Returns the number of items walked, or a negative code.
extern "C" long long check_stats_digits(int B, int H, int Sq, int Sk, int causal, int k_past, int sms) {
    if (causal && k_past < 0) k_past = Sk > Sq ? Sk - Sq : 0;
    Problem p;
    memset(&p, 0, sizeof(p));
    plan(p, B, H, Sq, Sk, causal, k_past, sms);
    const int grid = (int)(p.stats_items < sms ? p.stats_items : sms);
    stats_set_grid(p, grid);
    long long walked = 0;
    for (int cta = 0; cta < grid; ++cta) {
        StatsItems it;
        it.init(p, cta, grid);
        for (; !it.done; it.next(p)) {
            StatsItems ref;
            ref.done = false;
            ref.grid = grid;
            ref.item = it.item;
            ref.load(p);
            if (ref.done) return -1;
            if (ref.b != it.b || ref.h != it.h || ref.qt != it.qt || ref.sp != it.sp || ref.s0 != it.s0 || ref.s1 != it.s1)
                return -2;
            ++walked;
        }
        if (it.item < p.stats_items) return -3;
    }
    return walked == p.stats_items ? walked : -4;
}
