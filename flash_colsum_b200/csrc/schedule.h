// Work decomposition of the two attention-column-mean passes, shared by the CUDA
// kernels and by the host code that plans a call.  Everything here is plain
// integer logic, usable from host and device, so the step sequences and the
// mask rules can be checked on a CPU.
#pragma once

#include <stddef.h>
#include <stdint.h>

#if defined(__CUDACC__)
#define FCS_HD __host__ __device__
#else
#define FCS_HD
#endif

namespace fcs {

constexpr int TILE = 128;      // rows of an operand tile; one step is a 128x128 score tile
constexpr int MAX_SPLIT = 64;  // most key ranges a query tile is split into

enum : int { MODE_STATS = 0, MODE_COLSUM = 1 };

struct float2_ { float x, y; };

struct Problem {
    int B, H, Sq, Sk;   // Sq: query rows that enter the mean
    int NQ, NKT;        // query tiles, key tiles
    int NKC;            // key tiles that hold at least one visible key (column pass)
    int causal, k_past; // key j is visible to query i iff j <= k_past + i
    int nsplit;         // key ranges per (b, h, query tile) in the statistics pass
    int kreg;           // leading key tiles that every query tile contributes to
    long long stats_items;
    long long steps_per_batch;  // column pass: steps of one batch entry
    long long steps_total;
    float c;            // |scale| * log2(e)
    float log2_norm;    // log2(h_norm * R)
    float* neg_lse;     // [B*H][NQ*128]   -(lse2 + log2_norm), -inf on padding rows
    void* part;         // float2 [nsplit][B*H][NQ*128]   (max, sum) per key range
    float* out;
    long long out_ld;
    int* status;
    uint32_t idesc;
};

FCS_HD inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Key tiles a query tile needs in the statistics pass.
FCS_HD inline int stats_key_tiles(const Problem& p, int qt) {
    if (!p.causal) return p.NKT;
    int q_end = (qt + 1) * TILE;
    if (q_end > p.Sq) q_end = p.Sq;
    long long k_end = (long long)p.k_past + q_end;   // keys visible to the tile's last row
    if (k_end > p.Sk) k_end = p.Sk;
    return ceil_div((int)k_end, TILE);
}
// First query tile that contributes to a key tile in the column pass.
FCS_HD inline int colsum_first_q_tile(const Problem& p, int kt) {
    if (!p.causal) return 0;
    long long d = (long long)kt * TILE - p.k_past;
    return d <= 0 ? 0 : (int)(d / TILE);
}

// Statistics pass, score tile (qt, kt): the last visible key column (relative to
// the tile) for tile row `row`; and whether every element of the tile is visible.
FCS_HD inline int stats_last_visible(const Problem& p, int qt, int kt, int row) {
    long long lim = p.Sk - 1;
    if (p.causal) {
        const long long v = (long long)p.k_past + (long long)qt * TILE + row;
        if (v < lim) lim = v;
    }
    lim -= (long long)kt * TILE;
    return lim > TILE ? TILE : (lim < -1 ? -1 : (int)lim);
}
FCS_HD inline bool stats_tile_full(const Problem& p, int qt, int kt) {
    bool full = ((long long)kt * TILE + TILE <= p.Sk);
    if (p.causal)
        full = full && ((long long)kt * TILE + TILE - 1 <= (long long)p.k_past + (long long)qt * TILE);
    return full;
}
// Column pass, transposed score tile (kt, qt): the first visible query column
// (relative to the tile) for key row `row`; and whether the whole tile is visible.
FCS_HD inline int colsum_first_visible(const Problem& p, int kt, int qt, int row) {
    if (!p.causal) return 0;
    const long long t = (long long)kt * TILE + row - p.k_past - (long long)qt * TILE;
    return t > TILE ? TILE : (t < 0 ? 0 : (int)t);
}
FCS_HD inline bool colsum_tile_full(const Problem& p, int kt, int qt) {
    return !p.causal || ((long long)kt * TILE + TILE - 1 - p.k_past - (long long)qt * TILE <= 0);
}

// ---------------------------------------------------------------------------
// Work iterators.  Every role of a CTA (producer, MMA issuer, both consumer
// groups) walks the same deterministic sequence of steps.  An "item" is a run
// of steps that share the resident operand tile (`first`/`last` mark its ends);
// `flush` marks the step after which the column pass adds its accumulators
// into the output.
// ---------------------------------------------------------------------------
template <int MODE>
struct WorkIter;

// Statistics pass: item = (b, h, query tile, key range), taken round-robin.
template <>
struct WorkIter<MODE_STATS> {
    bool done, first, last, flush;
    int b, h, qt, kt, sp, kt_end, grid;
    long long item;

    FCS_HD void load(const Problem& p) {
        if (item >= p.stats_items) { done = true; return; }
        sp = (int)(item % p.nsplit);
        const long long t = item / p.nsplit;
        qt = (int)(t % p.NQ);
        const long long bh = t / p.NQ;
        h = (int)(bh % p.H);
        b = (int)(bh / p.H);
        const int nk = stats_key_tiles(p, qt);
        kt = (int)((long long)sp * nk / p.nsplit);
        kt_end = (int)((long long)(sp + 1) * nk / p.nsplit);
        first = true;
        last = (kt + 1 >= kt_end);
    }
    FCS_HD void init(const Problem& p, int cta, int grid_) {
        done = false; flush = false;
        grid = grid_;
        item = cta;
        load(p);
    }
    FCS_HD void next(const Problem& p) {
        if (kt + 1 < kt_end) {
            ++kt; first = false; last = (kt + 1 >= kt_end);
        } else {
            item += grid;
            load(p);
        }
    }
    FCS_HD int a_row() const { return qt * TILE; }   // resident operand = query tile
    FCS_HD int b_row() const { return kt * TILE; }   // streamed operand = key tile
};

// Column pass: steps ordered (b, key tile, h, query tile); a CTA takes one
// contiguous range of them.
template <>
struct WorkIter<MODE_COLSUM> {
    bool done, first, last, flush;
    int b, h, qt, kt, qlo;
    long long s, s_end;

    FCS_HD void flags(const Problem& p) {
        const bool end = (s + 1 >= s_end);
        last = (qt + 1 >= p.NQ) || end;
        flush = ((qt + 1 >= p.NQ) && (h + 1 >= p.H)) || end;
    }
    FCS_HD void init(const Problem& p, int cta, int grid) {
        s = p.steps_total * cta / grid;
        s_end = p.steps_total * (cta + 1) / grid;
        done = (s >= s_end);
        first = last = flush = false;
        b = h = qt = kt = qlo = 0;
        if (done) return;
        b = (int)(s / p.steps_per_batch);
        long long r = s % p.steps_per_batch;
        const long long per_kt = (long long)p.H * p.NQ;
        const long long regular = per_kt * p.kreg;
        if (r < regular) {
            kt = (int)(r / per_kt);
            r = r % per_kt;
            qlo = 0;
        } else {
            r -= regular;
            kt = p.kreg;
            qlo = colsum_first_q_tile(p, kt);
            for (int guard = 0; guard < p.NKC; ++guard) {
                const long long n = (long long)p.H * (p.NQ - qlo);
                if (r < n) break;
                r -= n;
                ++kt;
                qlo = colsum_first_q_tile(p, kt);
            }
        }
        const int nq = p.NQ - qlo;
        h = (int)(r / nq);
        qt = qlo + (int)(r % nq);
        first = true;
        flags(p);
    }
    FCS_HD void next(const Problem& p) {
        ++s;
        if (s >= s_end) { done = true; return; }
        if (qt + 1 < p.NQ) {
            ++qt; first = false;
        } else {
            first = true;
            if (h + 1 < p.H) {
                ++h;
            } else {
                h = 0;
                if (kt + 1 < p.NKC) { ++kt; } else { kt = 0; ++b; }
                qlo = colsum_first_q_tile(p, kt);
            }
            qt = qlo;
        }
        flags(p);
    }
    FCS_HD int a_row() const { return kt * TILE; }   // resident operand = key tile
    FCS_HD int b_row() const { return qt * TILE; }   // streamed operand = query tile
};

// ---------------------------------------------------------------------------
// Planning (host): fills the shape-derived fields of `p`.
// ---------------------------------------------------------------------------
inline void plan(Problem& p, int B, int H, int Sq, int Sk, int causal, int k_past, int sms) {
    p.B = B; p.H = H; p.Sq = Sq; p.Sk = Sk;
    p.NQ = ceil_div(Sq, TILE);
    p.NKT = ceil_div(Sk, TILE);
    p.causal = causal;
    p.k_past = causal ? k_past : 0;
    // statistics pass: split the key range when (b, h, query tile) items are too
    // few to fill the SMs; never into more ranges than the shortest item has tiles
    const long long base_items = (long long)B * H * p.NQ;
    int max_split = stats_key_tiles(p, 0);
    if (max_split > MAX_SPLIT) max_split = MAX_SPLIT;
    int best = 1;
    double best_eff = 0.0;
    for (int s = 1; s <= max_split; ++s) {
        const long long n = base_items * s;
        const long long waves = (n + sms - 1) / sms;
        const double eff = (double)n / (double)(waves * sms);
        if (eff > best_eff + 1e-9) { best_eff = eff; best = s; }
        if (eff >= 0.94) break;
    }
    p.nsplit = best;
    p.stats_items = base_items * p.nsplit;
    // column pass step space
    if (causal) {
        long long visible = (long long)p.k_past + Sq;   // keys past this are seen by no query
        if (visible > Sk) visible = Sk;
        p.NKC = ceil_div((int)visible, TILE);
        const long long kr = (long long)p.k_past / TILE + 1;
        p.kreg = kr > p.NKC ? p.NKC : (int)kr;
    } else {
        p.NKC = p.NKT;
        p.kreg = p.NKT;
    }
    long long steps = (long long)p.kreg * H * p.NQ;
    for (int kt = p.kreg; kt < p.NKC; ++kt) steps += (long long)H * (p.NQ - colsum_first_q_tile(p, kt));
    p.steps_per_batch = steps;
    p.steps_total = steps * B;
}

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Scratch layout: [neg_lse | part]; returns the total and the offset of `part`.
inline size_t workspace_layout(const Problem& p, size_t* part_off) {
    const size_t rows = (size_t)p.B * p.H * p.NQ * TILE;
    size_t off = align_up(rows * sizeof(float), 256);
    if (part_off) *part_off = off;
    if (p.nsplit > 1) off += align_up(rows * 2 * sizeof(float) * p.nsplit, 256);
    return off;
}

}  // namespace fcs
