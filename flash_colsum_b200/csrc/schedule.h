// Work decomposition of the two attention-column-mean passes, shared by the CUDA
// kernels and by the host code that plans a call.  Everything here is plain
// integer logic, usable from host and device, so the step sequences and the
// mask rules can be checked on a CPU.
//
// Geometry.  One MMA step multiplies a resident [128 x D] operand tile by a
// streamed [256 x D] operand block and fills a 128 x 256 fp32 accumulator:
//   statistics pass: resident = 128 queries, streamed = 256 keys;
//   column pass:     resident = 128 keys,    streamed = 256 queries.
#pragma once

#include <stddef.h>
#include <stdint.h>

#if defined(__CUDACC__)
#define FCS_HD __host__ __device__
#else
#define FCS_HD
#endif

namespace fcs {

constexpr int TILE = 128;      // rows of the resident operand tile (MMA M)
constexpr int BLOCK = 256;     // rows of the streamed operand block (MMA N)
constexpr int MAX_SPLIT = 64;  // most key ranges a query tile is split into

// MODE_COLSUM_EXT_SHORT: the column pass of a query axis that fits one streamed block --
// every item is a single step, so the key tiles are what streams: deep ring for them, one stage for the queries
// MODE_COLSUM_EXT_SHORT2: the same for a query axis of two blocks, both resident
// ..._COMBINE: the same two, with the consumer groups' sums of an item combined in shared memory
// before one add per key (for an output that may be another GPU's memory)
enum : int { MODE_STATS = 0, MODE_COLSUM = 1, MODE_COLSUM_EXT = 2, MODE_COLSUM_EXT_SHORT = 3, MODE_COLSUM_EXT_SHORT2 = 4,
             MODE_COLSUM_EXT_SHORT_COMBINE = 5, MODE_COLSUM_EXT_SHORT2_COMBINE = 6 };
// values of Problem::col_interleave (how the column pass deals out its work, see ColsumItems)
enum : int { COL_CONTIGUOUS = 0, COL_INTERLEAVED = 1, COL_HEAD_MAJOR = 2 };

struct Problem {
    int B, H, Sq, Sk;   // Sq: query rows that enter the mean
    int NQ, NKT;        // 128-row query tiles / key tiles (resident operands)
    int NQB, NKB;       // 256-row query blocks / key blocks (streamed operands)
    int NKC;            // key tiles that hold at least one visible key (column pass)
    int causal, k_past; // key j is visible to query i iff j <= k_past + i
    int clear_out;      // the statistics pass zeroes `out` before the column pass adds into it
    float* clear_extra; // the statistics pass also zeroes these clear_extra_n floats (NULL: nothing)
    long long clear_extra_n;
    int nsplit;         // key ranges per (b, h, query tile) in the statistics pass
    int kreg;           // leading key tiles that every query block contributes to
    int col_interleave; // column pass: COL_CONTIGUOUS steps, or (b, h, key tile) chunks dealt round-robin / in contiguous runs
    int col_parts;      // ... each cut into this many query-block ranges
    int col_pack;       // head-major order: key tiles per item (2 when the queries fill half an accumulator, else 1)
    int col_combine;    // head-major order: the kernels that combine the consumer groups' sums before one add per key are used
    long long stats_items;
    // the statistics pass's CTA count, as the steps an item index advances by in (key range, query tile,
    // head, batch entry) digits: lets a CTA go from one of its items to the next without a division
    int stats_grid, stats_d_sp, stats_d_qt, stats_d_h, stats_d_b;
    long long steps_per_batch;  // column pass: steps of one batch entry
    long long steps_total;
    long long lse_rows;         // rows of neg_lse per (b, h): NQB * 256
    float c;            // |scale| * log2(e)
    float log2_norm;    // log2(h_norm * R)
    float* neg_lse;     // [B*H][lse_rows]   -(lse2 + log2_norm)
    void* ext;          // [B*H][lse_rows][16] 16-bit: neg_lse / c split into three parts (see make_ext_row)
    float inv_c;        // 1 / c
    int ext_bf16;       // element type of `ext` (that of the inputs)
    void* part;         // float2 [nsplit][B*H][NQ*128]   (max, sum) per key range
    float* out;
    long long out_ld;
    int* status;
    uint32_t idesc;
    // Ordering against other GPUs, inside the column pass of a head-sharded call (all NULL / 0 otherwise):
    const int* sig_wait;      // this CTA's first thread waits (bounded) until *sig_wait >= sig_wait_value before anything is added
    int sig_wait_value;
    int* sig_post[15];        // CTA 0 stores sig_post_value to these flags (release, system scope) once the kernel before has completed
    int sig_post_n, sig_post_value;
    int* sig_counter;         // CTAs that have finished; the last one resets it and stores sig_done_value to *sig_done
    int* sig_done;
    int sig_done_value;
    int withhold_loads; // self-test only: the producer issues no copies, so that the bounded waits run out
};

FCS_HD inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Key blocks a query tile needs in the statistics pass.
FCS_HD inline int stats_key_blocks(const Problem& p, int qt) {
    if (!p.causal) return p.NKB;
    int q_end = (qt + 1) * TILE;
    if (q_end > p.Sq) q_end = p.Sq;
    long long k_end = (long long)p.k_past + q_end;   // keys visible to the tile's last row
    if (k_end > p.Sk) k_end = p.Sk;
    return ceil_div((int)k_end, BLOCK);
}
// First query block that contributes to a key tile in the column pass.
FCS_HD inline int colsum_first_q_block(const Problem& p, int kt) {
    if (!p.causal) return 0;
    const long long d = (long long)kt * TILE - p.k_past;   // first query that sees the tile's first key
    return d <= 0 ? 0 : (int)(d / BLOCK);
}

// Statistics pass, score tile (query tile qt, key block kb): the last visible key
// column (0..255, or -1) for tile row `row`, and whether every element is visible.
FCS_HD inline int stats_last_visible(const Problem& p, int qt, int kb, int row) {
    long long lim = p.Sk - 1;
    if (p.causal) {
        const long long v = (long long)p.k_past + (long long)qt * TILE + row;
        if (v < lim) lim = v;
    }
    lim -= (long long)kb * BLOCK;
    return lim > BLOCK ? BLOCK : (lim < -1 ? -1 : (int)lim);
}
FCS_HD inline bool stats_tile_full(const Problem& p, int qt, int kb) {
    bool full = ((long long)kb * BLOCK + BLOCK <= p.Sk);
    if (p.causal)
        full = full && ((long long)kb * BLOCK + BLOCK - 1 <= (long long)p.k_past + (long long)qt * TILE);
    return full;
}
// Column pass, transposed score tile (key tile kt, query block qb): query columns
// [first, end) are visible for key row `row`; and whether the whole tile is.
FCS_HD inline int colsum_first_visible(const Problem& p, int kt, int qb, int row) {
    if (!p.causal) return 0;
    const long long t = (long long)kt * TILE + row - p.k_past - (long long)qb * BLOCK;
    return t > BLOCK ? BLOCK : (t < 0 ? 0 : (int)t);
}
FCS_HD inline int colsum_end_visible(const Problem& p, int qb) {
    const long long n = (long long)p.Sq - (long long)qb * BLOCK;
    return n > BLOCK ? BLOCK : (n < 0 ? 0 : (int)n);
}
FCS_HD inline bool colsum_tile_full(const Problem& p, int kt, int qb) {
    if ((long long)qb * BLOCK + BLOCK > p.Sq) return false;
    return !p.causal || ((long long)kt * TILE + TILE - 1 - p.k_past - (long long)qb * BLOCK <= 0);
}

// Steps lo <= st < hi of an item are fully visible (the *_tile_full rule, solved
// for the step index), so that the per-step mask arithmetic can be skipped.
FCS_HD inline void stats_full_range(const Problem& p, int qt, int& lo, int& hi) {
    lo = 0;
    long long h = p.Sk / BLOCK;
    if (p.causal) {
        const long long c = ((long long)p.k_past + (long long)qt * TILE + 1) / BLOCK;
        if (c < h) h = c;
    }
    hi = (int)h;
}
FCS_HD inline void colsum_full_range(const Problem& p, int kt, int& lo, int& hi) {
    hi = p.Sq / BLOCK;
    lo = 0;
    if (p.causal) {
        const long long d = (long long)kt * TILE + TILE - 1 - p.k_past;
        if (d > 0) lo = (int)((d + BLOCK - 1) / BLOCK);
    }
}

// ---------------------------------------------------------------------------
// Item iterators.  Every role of a CTA (producer, MMA issuer, consumers) walks
// the same deterministic sequence of items; an item is a run of steps that
// share the resident operand tile, its steps are the streamed blocks
// [s0, s1).
// ---------------------------------------------------------------------------

// Statistics pass: item = (b, h, query tile, key range), taken round-robin.
struct StatsItems {
    bool done;
    int b, h, qt, sp, s0, s1, grid;   // steps = key blocks s0..s1-1
    long long item;

    // Decoding an item index is on the critical path of every role at every item boundary (the MMA
    // warp cannot issue the next item's first MMA before it): 32-bit arithmetic wherever the counts
    // allow it -- a 64-bit division is a subroutine of a hundred instructions, and eight of them
    // left the consumers waiting 1 500-2 600 cycles for the first tile of every item.
    FCS_HD void load(const Problem& p) {
        if (item >= p.stats_items) { done = true; return; }
        if (p.stats_items <= 0x7fffffffLL) {
            const unsigned it = (unsigned)item, ns = (unsigned)p.nsplit, nq = (unsigned)p.NQ, nh = (unsigned)p.H;
            const unsigned t = it / ns;
            sp = (int)(it - t * ns);
            const unsigned bh = t / nq;
            qt = (int)(t - bh * nq);
            const unsigned bb = bh / nh;
            h = (int)(bh - bb * nh);
            b = (int)bb;
        } else {
            sp = (int)(item % p.nsplit);
            const long long t = item / p.nsplit;
            qt = (int)(t % p.NQ);
            const long long bh = t / p.NQ;
            h = (int)(bh % p.H);
            b = (int)(bh / p.H);
        }
        ranges(p);
    }
    // key blocks of the item's key range
    FCS_HD void ranges(const Problem& p) {
        const int nk = stats_key_blocks(p, qt);
        if (p.nsplit == 1) {
            s0 = 0;
            s1 = nk;
        } else {
            // sp < 64 and nk < 2^23 (a key axis of 2^31 keys): the products fit 32 bits
            s0 = (int)((unsigned)sp * (unsigned)nk / (unsigned)p.nsplit);
            s1 = (int)((unsigned)(sp + 1) * (unsigned)nk / (unsigned)p.nsplit);
        }
    }
    FCS_HD void init(const Problem& p, int cta, int grid_) {
        done = false;
        grid = grid_;
        item = cta;
        load(p);
    }
    FCS_HD void next(const Problem& p) {
        item += grid;
        if (grid != p.stats_grid) { load(p); return; }    // (no digits for this grid: decode afresh)
        if (item >= p.stats_items) { done = true; return; }
        // add the grid's digits, with carries
        sp += p.stats_d_sp;
        int carry = sp >= p.nsplit ? 1 : 0;
        sp -= carry ? p.nsplit : 0;
        qt += p.stats_d_qt + carry;
        carry = qt >= p.NQ ? 1 : 0;
        qt -= carry ? p.NQ : 0;
        h += p.stats_d_h + carry;
        carry = h >= p.H ? 1 : 0;
        h -= carry ? p.H : 0;
        b += p.stats_d_b + carry;
        ranges(p);
    }
    FCS_HD int a_row() const { return qt * TILE; }        // resident = query tile
    FCS_HD int b_row(int s) const { return s * BLOCK; }   // streamed = key block
    FCS_HD bool flush() const { return false; }
};

// The digits of `grid` (the statistics pass's CTA count) for StatsItems::next; call before launching it.
inline void stats_set_grid(Problem& p, int grid) {
    p.stats_grid = grid;
    long long g = grid;
    p.stats_d_sp = (int)(g % p.nsplit);
    g /= p.nsplit;
    p.stats_d_qt = (int)(g % p.NQ);
    g /= p.NQ;
    p.stats_d_h = (int)(g % p.H);
    p.stats_d_b = (int)(g / p.H);
}

// Column pass, two ways of dealing out the steps.
// Contiguous (short inputs): steps ordered (b, key tile, h, query block); a CTA takes
// one contiguous range of them, cut into items at (b, key tile, h) boundaries --
// perfect balance, and the per-key accumulators stay in registers across the heads
// of a key tile.  `flush` marks the item after which they are added into the output
// (the CTA leaves the (b, key tile) group or ends).
// Interleaved (inputs far larger than the L2): chunks ordered (b, h, key tile, part of
// the query blocks) are dealt round-robin, so that at any moment the CTAs work on
// neighbouring key tiles of the same one or two heads and stream the same query blocks
// -- with contiguous ranges every CTA is in a different place and the working set is
// all heads at once (measured at B=1 H=16 S=32768: 4.3 GB read from DRAM for 134 MB of
// inputs).  Every chunk flushes.
// (A query axis of one block with many key tiles is dealt out a third way, head-major,
// by PackedItems below.)
struct ColsumItems {
    bool done, flush_;
    int b, h, kt, s0, s1, qlo;        // steps = query blocks s0..s1-1
    long long s, s_end;
    long long chunk;                  // interleaved mode: current chunk and the stride to the next
    int stride;

    FCS_HD void load_chunk(const Problem& p) {
        const long long total = (long long)p.B * p.H * p.NKC * p.col_parts;
        const bool small = total <= 0x7fffffffLL;     // 32-bit arithmetic (see StatsItems::load)
        for (; chunk < total; chunk += stride) {
            int part;
            if (small) {
                const unsigned c = (unsigned)chunk, cp = (unsigned)p.col_parts, nk = (unsigned)p.NKC, nh = (unsigned)p.H;
                const unsigned i0 = c / cp;
                part = (int)(c - i0 * cp);
                const unsigned i1 = i0 / nk;
                kt = (int)(i0 - i1 * nk);
                const unsigned i2 = i1 / nh;
                h = (int)(i1 - i2 * nh);
                b = (int)i2;
            } else {
                part = (int)(chunk % p.col_parts);
                long long item = chunk / p.col_parts;
                kt = (int)(item % p.NKC);
                item /= p.NKC;
                h = (int)(item % p.H);
                b = (int)(item / p.H);
            }
            qlo = colsum_first_q_block(p, kt);
            const unsigned n = (unsigned)(p.NQB - qlo), cp = (unsigned)p.col_parts;
            if (n <= 0xffffffffu / cp) {      // the products fit 32 bits
                s0 = qlo + (int)(n * (unsigned)part / cp);
                s1 = qlo + (int)(n * (unsigned)(part + 1) / cp);
            } else {
                s0 = qlo + (int)((long long)n * part / p.col_parts);
                s1 = qlo + (int)((long long)n * (part + 1) / p.col_parts);
            }
            if (s1 > s0) { flush_ = true; return; }   // (a part of a short item may be empty)
        }
        done = true;
    }

    FCS_HD void cut(const Problem& p) {
        long long n = p.NQB - s0;
        if (n > s_end - s) n = s_end - s;
        s1 = s0 + (int)n;
        const bool end = (s + n >= s_end);
        flush_ = ((s1 >= p.NQB) && (h + 1 >= p.H)) || end;
    }
    FCS_HD void init(const Problem& p, int cta, int grid) {
        b = h = kt = s0 = s1 = qlo = 0;
        flush_ = false;
        s = s_end = 0;
        chunk = cta;
        stride = grid;
        if (p.col_interleave) {
            done = false;
            load_chunk(p);
            return;
        }
        s = p.steps_total * cta / grid;
        s_end = p.steps_total * (cta + 1) / grid;
        done = (s >= s_end);
        if (done) return;
        b = (int)(s / p.steps_per_batch);
        long long r = s % p.steps_per_batch;
        const long long per_kt = (long long)p.H * p.NQB;
        const long long regular = per_kt * p.kreg;
        if (r < regular) {
            kt = (int)(r / per_kt);
            r = r % per_kt;
            qlo = 0;
        } else {
            r -= regular;
            kt = p.kreg;
            qlo = colsum_first_q_block(p, kt);
            for (int guard = 0; guard < p.NKC; ++guard) {
                const long long n = (long long)p.H * (p.NQB - qlo);
                if (r < n) break;
                r -= n;
                ++kt;
                qlo = colsum_first_q_block(p, kt);
            }
        }
        const int nq = p.NQB - qlo;
        h = (int)(r / nq);
        s0 = qlo + (int)(r % nq);
        cut(p);
    }
    FCS_HD void next(const Problem& p) {
        if (p.col_interleave) {
            chunk += stride;
            load_chunk(p);
            return;
        }
        s += s1 - s0;
        if (s >= s_end) { done = true; return; }
        if (h + 1 < p.H) {
            ++h;
        } else {
            h = 0;
            if (kt + 1 < p.NKC) { ++kt; } else { kt = 0; ++b; }
            qlo = colsum_first_q_block(p, kt);
        }
        s0 = qlo;
        cut(p);
    }
    FCS_HD int a_row() const { return kt * TILE; }        // resident = key tile
    FCS_HD int b_row(int st) const { return st * BLOCK; } // streamed = query block
    FCS_HD bool flush() const { return flush_; }
};

// Head-major order of the column pass (a query axis of one block, sixteen or more key
// tiles): the list of (b, h, group of col_pack key tiles) is cut into one contiguous run
// per CTA, so that a CTA stays with one head for as long as possible, keeps that head's
// only query block in shared memory and streams key tiles.  Every item is a single step
// and flushes.  When the queries fill at most half an accumulator (128 of its 256
// columns) an item is two key tiles (`nt`, from `kt` on), computed side by side, so that
// the per-item costs are paid half as often.
struct PackedItems {
    bool done;
    int b, h, kt, nt;
    long long chunk, chunk_end;
    static constexpr int s0 = 0, s1 = 1;

    FCS_HD void init(const Problem& p, int cta, int grid) {
        const int per_head = ceil_div(p.NKC, p.col_pack);
        const long long all = (long long)p.B * p.H * per_head;
        chunk = all * cta / grid;
        chunk_end = all * (cta + 1) / grid;
        done = chunk >= chunk_end;
        b = h = kt = 0;
        nt = 1;
        if (done) return;
        long long item = chunk;
        kt = (int)(item % per_head) * p.col_pack;
        item /= per_head;
        h = (int)(item % p.H);
        b = (int)(item / p.H);
        nt = p.NKC - kt < p.col_pack ? p.NKC - kt : p.col_pack;
    }
    // (no divisions here: a step is short, and every role of the CTA walks the list)
    FCS_HD void next(const Problem& p) {
        if (++chunk >= chunk_end) { done = true; return; }
        kt += p.col_pack;
        if (kt >= p.NKC) {
            kt = 0;
            if (++h >= p.H) { h = 0; ++b; }
        }
        nt = p.NKC - kt < p.col_pack ? p.NKC - kt : p.col_pack;
    }
    FCS_HD int a_row() const { return kt * TILE; }        // resident = key tiles
    FCS_HD int b_row(int) const { return 0; }             // the query block
    FCS_HD bool flush() const { return true; }
};

// The same order for a query axis of two blocks (both stay in shared memory): an item is one
// key tile against the query blocks s0..s1-1 that see it.
struct ResidentItems {
    bool done;
    int b, h, kt, s0, s1;
    long long chunk, chunk_end;
    static constexpr int nt = 1;

    FCS_HD void init(const Problem& p, int cta, int grid) {
        const long long all = (long long)p.B * p.H * p.NKC;
        chunk = all * cta / grid;
        chunk_end = all * (cta + 1) / grid;
        done = chunk >= chunk_end;
        b = h = kt = s0 = 0;
        s1 = p.NQB;
        if (done) return;
        long long item = chunk;
        kt = (int)(item % p.NKC);
        item /= p.NKC;
        h = (int)(item % p.H);
        b = (int)(item / p.H);
        s0 = colsum_first_q_block(p, kt);
    }
    FCS_HD void next(const Problem& p) {
        if (++chunk >= chunk_end) { done = true; return; }
        if (++kt >= p.NKC) {
            kt = 0;
            if (++h >= p.H) { h = 0; ++b; }
        }
        s0 = colsum_first_q_block(p, kt);
    }
    FCS_HD int a_row() const { return kt * TILE; }            // resident = key tile
    FCS_HD int b_row(int st) const { return st * BLOCK; }     // the query blocks
    FCS_HD bool flush() const { return true; }
};

template <int MODE> struct ItemsOf;
template <> struct ItemsOf<MODE_STATS> { typedef StatsItems type; };
template <> struct ItemsOf<MODE_COLSUM> { typedef ColsumItems type; };
template <> struct ItemsOf<MODE_COLSUM_EXT> { typedef ColsumItems type; };
template <> struct ItemsOf<MODE_COLSUM_EXT_SHORT> { typedef PackedItems type; };
template <> struct ItemsOf<MODE_COLSUM_EXT_SHORT2> { typedef ResidentItems type; };
template <> struct ItemsOf<MODE_COLSUM_EXT_SHORT_COMBINE> { typedef PackedItems type; };
template <> struct ItemsOf<MODE_COLSUM_EXT_SHORT2_COMBINE> { typedef ResidentItems type; };

// ---------------------------------------------------------------------------
// Planning (host): fills the shape-derived fields of `p`.
// ---------------------------------------------------------------------------
// Query rows (B * H * Sq) beyond which the column pass deals its work out interleaved:
// the rows and their extension columns (up to 288 bytes each) then exceed what the L2
// keeps for data that every SM reads.
constexpr long long COL_INTERLEAVE_MIN_ROWS = 300000;
constexpr int COL_HEAD_MAJOR_MAX_BLOCKS = 2;   // query blocks that stay in shared memory next to a ring of key tiles
constexpr int COL_HEAD_MAJOR_MIN_TILES = 16;   // key tiles per head from which the head-major order is used

inline void plan(Problem& p, int B, int H, int Sq, int Sk, int causal, int k_past, int sms,
                 long long interleave_min_rows = COL_INTERLEAVE_MIN_ROWS, bool head_major_ok = true) {
    p.B = B; p.H = H; p.Sq = Sq; p.Sk = Sk;
    p.NQ = ceil_div(Sq, TILE);
    p.NKT = ceil_div(Sk, TILE);
    p.NQB = ceil_div(Sq, BLOCK);
    p.NKB = ceil_div(Sk, BLOCK);
    p.lse_rows = (long long)p.NQB * BLOCK;
    p.causal = causal;
    p.k_past = causal ? k_past : 0;
    // statistics pass: split the key range when (b, h, query tile) items are too
    // few to fill the SMs; never into more ranges than the shortest item has blocks
    const long long base_items = (long long)B * H * p.NQ;
    int max_split = stats_key_blocks(p, 0);
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
        // key tiles whose first key is seen by query block 0's ... first block: d < BLOCK
        const long long kr = ((long long)p.k_past + BLOCK - 1) / TILE + 1;
        p.kreg = kr > p.NKC ? p.NKC : (int)kr;
        // keep only tiles with first_q_block == 0
        while (p.kreg > 0 && colsum_first_q_block(p, p.kreg - 1) != 0) --p.kreg;
    } else {
        p.NKC = p.NKT;
        p.kreg = p.NKT;
    }
    long long steps = (long long)p.kreg * H * p.NQB;
    for (int kt = p.kreg; kt < p.NKC; ++kt) steps += (long long)H * (p.NQB - colsum_first_q_block(p, kt));
    p.steps_per_batch = steps;
    p.steps_total = steps * B;
    p.col_interleave = ((long long)B * H * Sq >= interleave_min_rows) ? 1 : 0;
    // enough chunks for a balanced deal: about eight per CTA, by cutting the query blocks
    // of an item into parts when the (b, h, key tile) items alone are too few
    const long long items = (long long)B * H * p.NKC;
    long long parts = items >= 8ll * sms ? 1 : (8ll * sms + items - 1) / items;
    if (parts > p.NQB) parts = p.NQB;
    p.col_parts = (int)parts;
    p.col_pack = 1;
    if (head_major_ok && p.NQB <= COL_HEAD_MAJOR_MAX_BLOCKS && p.NKC >= COL_HEAD_MAJOR_MIN_TILES) {
        p.col_interleave = COL_HEAD_MAJOR;
        p.col_parts = 1;
        if (Sq <= BLOCK / 2) p.col_pack = 2;   // two key tiles side by side in one accumulator
    }
}

// ---------------------------------------------------------------------------
// Single-pass kernel: a cluster's share of the list of (batch, head, query tile)
// triples, ordered with the query tile innermost.  The list is cut evenly over the
// clusters, so a share starts and ends anywhere inside a (batch, head) pair.
// ---------------------------------------------------------------------------
struct TileRange {
    long long g0, g1;   // tiles [g0, g1) of the list
    int u0, u1;         // the (batch, head) pairs they touch: u0 .. u1-1
    int NQ;

    FCS_HD void init(long long units, int nq, int cluster, int clusters) {
        NQ = nq;
        const long long all = units * nq;
        g0 = all * cluster / clusters;
        g1 = all * (cluster + 1) / clusters;
        u0 = (int)(g0 / nq);
        u1 = (int)((g1 + nq - 1) / nq);
    }
    FCS_HD int tiles() const { return (int)(g1 - g0); }
    // query tiles [t_lo, t_hi) of pair u belong to the share
    FCS_HD int t_lo(int u) const { return u == u0 ? (int)(g0 - (long long)u0 * NQ) : 0; }
    FCS_HD int t_hi(int u) const { return u + 1 == u1 ? (int)(g1 - (long long)(u1 - 1) * NQ) : NQ; }
    // query tile of the i-th tile of the share
    FCS_HD int tile_of(int i) const { return (int)((g0 + i) % NQ); }
    // The column sums are written out after pair u: at the end of the share, of a batch entry
    // (H pairs), and every `flush_units` pairs at the latest.
    FCS_HD bool flush_after(int u, int H, int flush_units) const {
        return (u + 1 == u1) || ((u + 1) / H != u / H) || ((u + 1 - u0) % flush_units == 0);
    }
};

// ---------------------------------------------------------------------------
// The one-kernel form for a short query axis over a short key axis: a cluster of `cl` CTAs
// per (batch, head), CTA r walking the r-th run of `bpc` 256-key blocks twice (statistics,
// then columns).  `max_clusters[c]` is how many clusters of c CTAs the device runs at once
// (c = 1..8); `k_past` is the resolved value (>= 0) of a causal call.
//
// The cluster size is the largest with which all (batch, head) pairs run in one wave; with
// more pairs than SMs, one CTA each in several waves.  The form is taken when the query
// rows fit one 128-row tile and a model of the two forms says so.  In units of one key
// block through one phase on one SM (~1.35 us at D = 128): a CTA of this form costs a ramp
// of ~3 and then its blocks, once per wave of CTAs; the three kernels of the streaming form
// cost ~10 in launches, ramps and drains and then the call's blocks spread over all SMs:
//       waves * (3 + bpc)  <=  10 + B * H * nkb / SMs
// (measured per call, 32 heads x 128 queries: 28 against 41 us at 4096 keys, 64 against 79
// at 16384, 107 against 128 at 32768; 8 heads x 32768 keys -- 64 CTAs -- tie at 55 and stay
// with the streaming form; 768 pairs of 197 keys, six waves of one-block CTAs, lose 60 to 50).
// Calls that are bound by memory in either form are also taken while one wave of clusters
// covers four fifths of the SMs, no CTA walks more than 64 blocks and the call holds at
// most 64 blocks per SM (32 heads x 65536 keys: 191 against 211 us; a tie from 131072 on).
// `force`: only the shape limit applies (at most 128 rows).
// ---------------------------------------------------------------------------
constexpr int FUSED_SHORT_MAX_CLUSTER = 8;
constexpr int FUSED_SHORT_MAX_BLOCKS = 64;      // per CTA
constexpr int FUSED_SHORT_RAMP = 3;             // blocks: what a CTA costs before its first block
constexpr int FUSED_SHORT_LAUNCHES = 10;        // blocks: what the three-kernel form costs before its first block
constexpr int FUSED_SHORT_LARGE_WORK = 64;      // blocks per SM in the whole call
FCS_HD inline bool fused_short_plan(int B, int H, int Sq, int Sk, int causal, int k_past, int sms,
                                    const int* max_clusters, bool force, int* cl_out, int* nkb_out, int* bpc_out) {
    if (Sq > TILE) return false;
    long long keys = Sk;
    if (causal && (long long)k_past + Sq < keys) keys = (long long)k_past + Sq;   // keys some row sees
    const long long nkb = (keys + BLOCK - 1) / BLOCK;
    const long long units = (long long)B * H;
    int cl = 1;
    for (int c = nkb < FUSED_SHORT_MAX_CLUSTER ? (int)nkb : FUSED_SHORT_MAX_CLUSTER; c > 1; --c)
        if (units <= max_clusters[c]) { cl = c; break; }
    const long long bpc = (nkb + cl - 1) / cl;
    cl = (int)((nkb + bpc - 1) / bpc);                 // no CTA without a block
    if (bpc > (1 << 20)) return false;
    if (!force) {
        if (bpc > FUSED_SHORT_MAX_BLOCKS) return false;
        const long long at_once = cl > 1 ? max_clusters[cl] : sms;
        const long long waves = (units + at_once - 1) / at_once;
        const long long work = units * nkb;
        const bool model = waves * (FUSED_SHORT_RAMP + bpc) * sms <= (long long)FUSED_SHORT_LAUNCHES * sms + work;
        const bool memory_bound = waves == 1 && units * cl * 5 >= (long long)sms * 4 &&
                                  work <= (long long)FUSED_SHORT_LARGE_WORK * sms;
        if (!model && !memory_bound) return false;
    }
    if (cl_out) *cl_out = cl;
    if (nkb_out) *nkb_out = (int)nkb;
    if (bpc_out) *bpc_out = (int)bpc;
    return true;
}

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Scratch layout: [neg_lse | ext | part]; returns the total and the offsets.
inline size_t workspace_layout(const Problem& p, size_t* part_off, size_t* ext_off = nullptr) {
    size_t off = align_up((size_t)p.B * p.H * (size_t)p.lse_rows * sizeof(float), 256);
    if (ext_off) *ext_off = off;
    off += align_up((size_t)p.B * p.H * (size_t)p.lse_rows * 32, 256);
    if (part_off) *part_off = off;
    if (p.nsplit > 1) off += align_up((size_t)p.B * p.H * p.NQ * TILE * 2 * sizeof(float) * p.nsplit, 256);
    return off;
}

}  // namespace fcs
