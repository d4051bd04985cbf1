// Attention column mean for B200 (sm_100a): kernels and their C ABI.
//
// out[b, k] = 1/(H * R) * sum_h sum_{q < R} softmax_k(scale * Q[b,h,q,:] . K[b,h,k,:])
//
// Two streaming kernels share one warp-specialised skeleton (TMA -> shared
// memory -> tcgen05 MMA -> tensor memory -> consumer warps):
//
//   statistics pass  S  = Q K^T : tensor-memory lane = query row, so the running
//                    row maximum and sum of exp2 stay inside one thread.  It
//                    writes -(log2-sum-exp + log2(H*R)) per query row.
//   column pass      S^T = K Q^T: tensor-memory lane = key, so the reduction
//                    down the query axis stays inside one thread as well.  It
//                    adds exp2(c*s - lse) into a per-key fp32 accumulator and
//                    flushes that with one atomic add per (key tile, CTA range).
//                    -lse/c reaches the accumulator through 16 extra contraction
//                    columns (MODE_COLSUM_EXT); for tiny scales it is staged
//                    through shared memory instead (MODE_COLSUM).  A query axis of
//                    one or two 256-row blocks over sixteen or more key tiles swaps
//                    the roles (MODE_COLSUM_EXT_SHORT / _SHORT2): the head's query
//                    blocks stay in shared memory, the key tiles stream through a
//                    deep ring, and with at most 128 queries two key tiles share
//                    one accumulator buffer.
//
// Both operands are row tiles with the head dimension contiguous, so the same
// shared-memory layout serves as A (128 resident rows) or B (256 streamed rows)
// of the MMA; one step is a 128 x 256 x D MMA into one of two accumulator
// buffers of 256 tensor-memory columns.  Calls with at most four query rows
// take the matrix-vector kernel of colsum_small_q.cuh instead; short non-causal
// key axes at head dimension 64 take the single-pass cluster kernel of
// colsum_single_pass.cuh; a query axis of at most 128 rows over a few thousand keys
// takes the one-kernel cluster form of colsum_fused_short.cuh; select_topk.cuh holds
// the pruning step that callers run on the result.
#include "sm100_ptx.cuh"
#include "schedule.h"
#include "colsum_small_q.cuh"
#include "colsum_math.cuh"

#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include "../../include/flash_colsum_b200.h"

#include "colsum_single_pass.cuh"
#include "select_topk.cuh"

namespace fcs {

constexpr int NUM_TBUF = 2;        // accumulator buffers of 256 tensor-memory columns
constexpr int TMEM_COLS = 512;
constexpr int NUM_LSE = 4;         // per-query-block log-sum-exp vectors in flight (column pass)
// Consumer warps come in groups of four (a group covers the 128 tensor-memory
// lanes); every group takes an equal run of the columns of each accumulator.
constexpr int CONSUMER_GROUPS = 4;
constexpr int GROUP_COLS = BLOCK / CONSUMER_GROUPS;
constexpr int CONSUMER_WARPS = 4 * CONSUMER_GROUPS;
constexpr int CONSUMER_THREADS = 32 * CONSUMER_WARPS;
constexpr int PRODUCER_WARP = CONSUMER_WARPS;
constexpr int MMA_WARP = CONSUMER_WARPS + 1;
constexpr int THREADS = 32 * (CONSUMER_WARPS + 2);
static_assert(GROUP_COLS == 64, "a group consumes one 64-column block per step");

// Item-end partials of the statistics pass wait in one of these slots until a group
// combines them; consumer groups are never more than two steps apart, so four
// slots cannot be overrun.
constexpr int MERGE_SLOTS = 4;
constexpr int EXT_K = 16;                        // extra contraction columns that carry -(lse)/c
constexpr int EXT_ROW_BYTES = EXT_K * 2;
constexpr int EXT_A_BYTES = TILE * EXT_ROW_BYTES;    // the constant key-side columns
constexpr int EXT_B_BYTES = BLOCK * EXT_ROW_BYTES;   // the query-side columns of one block

template <int D, int MODE>
struct Layout {
    static constexpr bool COMBINE = (MODE == MODE_COLSUM_EXT_SHORT_COMBINE) || (MODE == MODE_COLSUM_EXT_SHORT2_COMBINE);
    static constexpr bool SHORT2 = (MODE == MODE_COLSUM_EXT_SHORT2) || (MODE == MODE_COLSUM_EXT_SHORT2_COMBINE);
    static constexpr bool SHORT = (MODE == MODE_COLSUM_EXT_SHORT) || (MODE == MODE_COLSUM_EXT_SHORT_COMBINE) || SHORT2;
    static constexpr int NB = SHORT2 ? 2 : 1;   // (short modes) resident query blocks
    static constexpr bool EXT = (MODE == MODE_COLSUM_EXT) || SHORT;
    static constexpr int SLABS = D / 64;              // 64-element (128-byte) column slabs
    static constexpr int A_SLAB_BYTES = TILE * 128;
    static constexpr int B_SLAB_BYTES = BLOCK * 128;
    static constexpr int A_BYTES = SLABS * A_SLAB_BYTES;
    static constexpr int B_BYTES = SLABS * B_SLAB_BYTES;
    static constexpr int B_STAGE_BYTES = B_BYTES + (EXT ? EXT_B_BYTES : 0);   // block, then its extension
    static constexpr int NS = SHORT ? NB : (D == 64) ? 4 : 2;     // streamed-operand stages
    // resident-operand buffers: two; in the short modes they are what streams -- 128 KiB of them,
    // or what two 128-wide query blocks leave
    static constexpr int NA = !SHORT ? 2 : (NB == 2 && D == 128) ? 2 : 256 / SLABS / 32;
    static constexpr int A_OFF = 0;
    static constexpr int B_OFF = NA * A_BYTES;
    static constexpr int EXTA_OFF = B_OFF + NS * B_STAGE_BYTES;             // 128 rows of the constant
    static constexpr int LSE_OFF = EXTA_OFF + (EXT ? EXT_A_BYTES : 0);      // NUM_LSE slots of 256 floats
    static constexpr int BAR_OFF = LSE_OFF + (MODE == MODE_COLSUM ? NUM_LSE * BLOCK * 4 : 0);
    // barriers: a_full[NA] a_empty[NA] b_full[NS] b_empty[NS] t_full[2] t_empty[2] merge[MERGE_SLOTS]
    //           l_full[NUM_LSE] l_empty[NUM_LSE]
    static constexpr int NUM_BARS = 2 * NA + 2 * NS + 2 * NUM_TBUF + MERGE_SLOTS + 2 * NUM_LSE;
    static constexpr int MISC_OFF = BAR_OFF + NUM_BARS * 8;        // tmem address, abort flag
    static constexpr int MERGE_OFF = (MISC_OFF + 16 + 15) / 16 * 16;  // float2[MERGE_SLOTS][groups][128]
    // (short column modes: float[MERGE_SLOTS][groups][128], the groups' sums of an item before the one add)
    static constexpr int PROB_OFF = MERGE_OFF + (MODE == MODE_STATS ? MERGE_SLOTS * CONSUMER_GROUPS * TILE * 8
                                                                    : COMBINE ? MERGE_SLOTS * CONSUMER_GROUPS * TILE * 4 : 0);
    // a copy of the call's parameters: what is read once per item (the item iterators) is read from
    // here -- in the constant bank those words are cold by the next item, a miss each
    static constexpr int TOTAL = PROB_OFF + (int)((sizeof(Problem) + 15) / 16 * 16);
    static constexpr int DYN_BYTES = TOTAL + 1024;    // slack to align the base to 1024
    static_assert(DYN_BYTES <= 227 * 1024, "shared memory budget");
};

// A group's 64 columns of one accumulator.  `taddr`, `lim`, `thr`, `end` and
// `nl` are relative to the group's first column.
template <bool MASKED>
__device__ __forceinline__ void stats_tile(uint32_t taddr, int lim, float c, float& m, float& l) {
    uint32_t r[32];
    tmem_ld_x32(taddr, r);
    tmem_ld_wait(r);
    stats_block32<MASKED>(r, lim, c, m, l);
    tmem_ld_x32(taddr + 32, r);
    tmem_ld_wait(r);
    stats_block32<MASKED>(r, lim - 32, c, m, l);
}
template <bool MASKED>
__device__ __forceinline__ void colsum_tile_ext(uint32_t taddr, int thr, int end, float c, float (&acc)[4]) {
    if constexpr (!MASKED) {
        // 16 columns at a time, the next 16 in flight from tensor memory while these are in the exp pipes
        uint32_t ra[16], rb[16];
        tmem_ld_16cols(taddr, ra);
        tmem_wait_16cols(ra);
        tmem_ld_16cols(taddr + 16, rb);
        colsum_chunk16_ext<0>(ra, c, acc);
        tmem_wait_16cols(rb);
        tmem_ld_16cols(taddr + 32, ra);
        colsum_chunk16_ext<8>(rb, c, acc);
        tmem_wait_16cols(ra);
        tmem_ld_16cols(taddr + 48, rb);
        colsum_chunk16_ext<0>(ra, c, acc);
        tmem_wait_16cols(rb);
        colsum_chunk16_ext<8>(rb, c, acc);
        return;
    }
    uint32_t r[32];
    tmem_ld_x32(taddr, r);
    tmem_ld_wait(r);
    colsum_chunk_ext<MASKED>(r, thr, end, c, acc);
    tmem_ld_x32(taddr + 32, r);
    tmem_ld_wait(r);
    colsum_chunk_ext<MASKED>(r, thr - 32, end - 32, c, acc);
}
template <bool MASKED>
__device__ __forceinline__ void colsum_tile(uint32_t taddr, const float4* nl, int thr, int end, float c,
                                            float (&acc)[4]) {
    uint32_t r[32];
#pragma unroll
    for (int ch = 0; ch < GROUP_COLS / 32; ++ch) {
        tmem_ld_x32(taddr + 32 * ch, r);
        tmem_ld_wait(r);
        colsum_chunk<MASKED>(r, nl + 8 * ch, thr - 32 * ch, end - 32 * ch, c, acc);
    }
}

// Release stores at system scope, kept out of line: with a system-scope fence or release store
// in its own body the streaming kernel's adds into another GPU's memory run markedly slower
// (measured on the long-context shape: 0.363 against 0.289 ms for the column pass of a rank that
// adds over NVLink, whether or not the store is ever executed).
__device__ __noinline__ void release_store_system(int* const* flags, int n, int value) {
    __threadfence_system();
    for (int i = 0; i < n; ++i)
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(flags[i]), "r"(value) : "memory");
}
__device__ __noinline__ void release_store_system_one(int* flag, int value) {
    __threadfence_system();
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(flag), "r"(value) : "memory");
}

// ---------------------------------------------------------------------------
// The streaming kernel.  tm_a: resident operand (box of 128 rows), tm_b:
// streamed operand (box of 256 rows), tm_ext: the 16 extension columns of the
// query blocks (MODE_COLSUM_EXT only).
// ---------------------------------------------------------------------------
template <int D, int MODE>
__global__ void __launch_bounds__(THREADS, 1)
colsum_stream_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                     const __grid_constant__ CUtensorMap tm_ext, const Problem p) {
    using L = Layout<D, MODE>;
    constexpr bool EXT = L::EXT;
    constexpr int NA = L::NA;
    using Items = typename ItemsOf<MODE>::type;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t a_smem = smem_base + L::A_OFF;
    const uint32_t b_smem = smem_base + L::B_OFF;
    const uint32_t lse_smem = smem_base + L::LSE_OFF;
    const uint32_t bars = smem_base + L::BAR_OFF;
    auto a_full = [&](int i) { return bars + 8u * i; };
    auto a_empty = [&](int i) { return bars + 8u * (NA + i); };
    auto b_full = [&](int i) { return bars + 8u * (2 * NA + i); };
    auto b_empty = [&](int i) { return bars + 8u * (2 * NA + L::NS + i); };
    auto t_full = [&](int i) { return bars + 8u * (2 * NA + 2 * L::NS + i); };
    auto t_empty = [&](int i) { return bars + 8u * (2 * NA + 2 * L::NS + NUM_TBUF + i); };
    auto merge_bar = [&](int i) { return bars + 8u * (2 * NA + 2 * L::NS + 2 * NUM_TBUF + i); };
    auto l_full = [&](int i) { return bars + 8u * (2 * NA + MERGE_SLOTS + 2 * L::NS + 2 * NUM_TBUF + i); };
    auto l_empty = [&](int i) { return bars + 8u * (2 * NA + MERGE_SLOTS + 2 * L::NS + 2 * NUM_TBUF + NUM_LSE + i); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + L::MISC_OFF);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::MISC_OFF + 4);
    float2* merge_buf = reinterpret_cast<float2*>(smem + L::MERGE_OFF);
    // The item iterators take the parameters by reference; taken from the kernel's parameter block
    // that is a copy in local memory, whose lines are cold -- a miss each, 450 cycles per item in all --
    // by the time the next item is decoded.  They read this copy in shared memory instead.  (The mask
    // rules, evaluated every step, keep the local copy: its lines stay in L1, and the long-context
    // column pass was 2 % slower with them on the shared copy.)
    Problem& ps = *reinterpret_cast<Problem*>(smem + L::PROB_OFF);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 32) ps = p;
    if (threadIdx.x == 0) {
        for (int i = 0; i < NA; ++i) { mbar_init(a_full(i), 1); mbar_init(a_empty(i), 1); }
        for (int i = 0; i < L::NS; ++i) { mbar_init(b_full(i), 1); mbar_init(b_empty(i), 1); }
        for (int i = 0; i < NUM_TBUF; ++i) { mbar_init(t_full(i), 1); mbar_init(t_empty(i), CONSUMER_THREADS); }
        for (int i = 0; i < MERGE_SLOTS; ++i) mbar_init(merge_bar(i), CONSUMER_THREADS);
        for (int i = 0; i < NUM_LSE; ++i) { mbar_init(l_full(i), 1); mbar_init(l_empty(i), CONSUMER_THREADS); }
        *abort_flag = 0;
        mbar_fence_init();
    }
    if constexpr (EXT) {
        // the key-side constant of the extension: every 16-byte piece is (k, k, k, 0, 0, 0, 0, 0),
        // which reads the same under any swizzle of the pieces
        const uint32_t k16 = p.ext_bf16 ? 0x3F80u : 0x5C00u;   // bf16 1.0 / fp16 256.0
        uint4* ones = reinterpret_cast<uint4*>(smem + L::EXTA_OFF);
        for (int i = threadIdx.x; i < EXT_A_BYTES / 16; i += THREADS)
            ones[i] = make_uint4(k16 | (k16 << 16), k16, 0u, 0u);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == PRODUCER_WARP && lane == 0) {
        prefetch_tensormap(&tm_a);
        prefetch_tensormap(&tm_b);
        if constexpr (EXT) prefetch_tensormap(&tm_ext);
    }
    if (warp == MMA_WARP) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // everything above touched only this CTA's shared and tensor memory; from here on the
    // results of the kernel before this one in the stream are read
    grid_dependency_wait();
    grid_launch_dependents();
    if (MODE != MODE_STATS && (p.sig_wait || p.sig_post_n > 0)) {
        // head shards on several GPUs adding into one buffer: nothing is added before the owner of
        // the buffer has said that it is clear (a flag in this GPU's memory, written over NVLink;
        // the wait is bounded), and the owner says so for the buffer of the next call once the
        // kernels before this one (its statistics pass cleared that buffer) have completed
        if (threadIdx.x == 0) {
            if (p.sig_wait) {
                const long long t0 = clock64();
                unsigned spins = 0;
                while (true) {
                    int v;
                    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p.sig_wait) : "memory");
                    if (v >= p.sig_wait_value) break;
                    if ((++spins & 63u) == 0u && clock64() - t0 > g_wait_limit_cycles) {
                        if (p.status) atomicCAS(p.status, 0, FCS_STATUS_WAIT_PEER);
                        break;
                    }
                    __nanosleep(200);
                }
            }
            if (blockIdx.x == 0 && p.sig_post_n > 0) {
                // (In the generic modes the flag pointers come from the shared copy, and with that the
                // compiler keeps no copy of the parameter block in local memory at all: the headline
                // shape's column pass is 5 % faster without it.  The short-query modes measured 2.5 %
                // slower without that copy, so there its address is still taken.)
                if constexpr (L::SHORT) release_store_system(p.sig_post, p.sig_post_n, p.sig_post_value);
                else release_store_system(ps.sig_post, p.sig_post_n, p.sig_post_value);
            }
        }
        __syncthreads();
    }

    // The producer and MMA warps run their loops with all 32 lanes converged (so
    // that addresses, descriptors and counters stay in uniform registers) and
    // elect one lane only around the instructions that must be issued once.
    auto wait_all = [&](uint32_t bar, uint32_t parity, int code) -> bool {
        const bool ok = mbar_wait(bar, parity, abort_flag, p.status, code);
        return __all_sync(0xffffffffu, ok);
    };

    if (warp >= CONSUMER_WARPS) {
        if (warp == PRODUCER_WARP) {
            // -------------------------------------------- TMA producer
            Items it;
            it.init(ps, blockIdx.x, gridDim.x);
            int a_cnt = 0, stage = 0, n = 0;
            uint32_t phase = 0;
            bool ok = p.withhold_loads == 0;   // (self-test: nothing is loaded, every wait for data runs out)
            // which streamed block every stage holds: when a (batch, head) has no more blocks
            // than there are stages (short query axes in the column pass, short key axes in the
            // statistics pass), the next item finds its blocks still in shared memory and the
            // stage is handed to the MMA warp again without a copy
            long long held[L::NS];
#pragma unroll
            for (int i = 0; i < L::NS; ++i) held[i] = -1;
            if constexpr (L::SHORT) {
                // Short query axis: an item is one or two key tiles against the head's only query
                // block.  The key tiles run ahead as far as their ring is deep; the query block
                // is loaded when the head changes.
                int cur_bh = -1, b_cnt = 0;
                for (; ok && !it.done; it.next(ps)) {
                    for (int t = 0; t < it.nt; ++t, ++a_cnt) {
                        const int ab = a_cnt % NA;
                        if (!wait_all(a_empty(ab), ((a_cnt / NA) & 1) ^ 1, FCS_STATUS_WAIT_PRODUCER)) { ok = false; break; }
                        if (elect_one_sync()) {
                            mbar_arrive_expect_tx(a_full(ab), L::A_BYTES);
#pragma unroll
                            for (int sl = 0; sl < L::SLABS; ++sl)
                                tma_load_4d(a_smem + ab * L::A_BYTES + sl * L::A_SLAB_BYTES, &tm_a, a_full(ab),
                                            sl * 64, it.a_row() + t * TILE, it.h, it.b);
                        }
                    }
                    if (!ok) break;
                    const int bh = it.b * p.H + it.h;
                    if (bh != cur_bh) {
                        if (!wait_all(b_empty(0), (b_cnt & 1) ^ 1, FCS_STATUS_WAIT_PRODUCER)) break;
                        if (elect_one_sync()) {
                            mbar_arrive_expect_tx(b_full(0), (uint32_t)p.NQB * L::B_STAGE_BYTES);
                            for (int qb = 0; qb < p.NQB; ++qb) {
#pragma unroll
                                for (int sl = 0; sl < L::SLABS; ++sl)
                                    tma_load_4d(b_smem + qb * L::B_STAGE_BYTES + sl * L::B_SLAB_BYTES, &tm_b, b_full(0),
                                                sl * 64, qb * BLOCK, it.h, it.b);
                                tma_load_3d(b_smem + qb * L::B_STAGE_BYTES + L::B_BYTES, &tm_ext, b_full(0), 0,
                                            qb * BLOCK, bh);
                            }
                        }
                        __syncwarp();
                        ++b_cnt;
                        cur_bh = bh;
                    }
                }
            } else {
            for (; ok && !it.done; it.next(ps), ++a_cnt) {
                const int ab = a_cnt & 1;
                if (!wait_all(a_empty(ab), ((a_cnt >> 1) & 1) ^ 1, FCS_STATUS_WAIT_PRODUCER)) break;
                if (elect_one_sync()) {
                    mbar_arrive_expect_tx(a_full(ab), L::A_BYTES);
#pragma unroll
                    for (int sl = 0; sl < L::SLABS; ++sl)
                        tma_load_4d(a_smem + ab * L::A_BYTES + sl * L::A_SLAB_BYTES, &tm_a, a_full(ab),
                                    sl * 64, it.a_row(), it.h, it.b);
                }
                const float* lse_src = nullptr;
                if constexpr (MODE == MODE_COLSUM)
                    lse_src = p.neg_lse + ((long long)it.b * p.H + it.h) * p.lse_rows;
                const int bh = it.b * p.H + it.h;
                for (int st = it.s0; st < it.s1; ++st, ++n) {
                    if (!wait_all(b_empty(stage), phase ^ 1, FCS_STATUS_WAIT_PRODUCER)) { ok = false; break; }
                    const long long block_id = ((long long)bh << 32) | (unsigned)st;
                    bool reuse = false;
#pragma unroll
                    for (int i = 0; i < L::NS; ++i)
                        if (i == stage) { reuse = held[i] == block_id; held[i] = block_id; }
                    if (reuse) {
                        if (elect_one_sync()) mbar_arrive(b_full(stage));
                    } else if (elect_one_sync()) {
                        mbar_arrive_expect_tx(b_full(stage), L::B_STAGE_BYTES);
#pragma unroll
                        for (int sl = 0; sl < L::SLABS; ++sl)
                            tma_load_4d(b_smem + stage * L::B_STAGE_BYTES + sl * L::B_SLAB_BYTES, &tm_b,
                                        b_full(stage), sl * 64, it.b_row(st), it.h, it.b);
                        if constexpr (EXT)
                            tma_load_3d(b_smem + stage * L::B_STAGE_BYTES + L::B_BYTES, &tm_ext, b_full(stage),
                                        0, it.b_row(st), bh);
                    }
                    if constexpr (MODE == MODE_COLSUM) {
                        // -(lse) of the 256 queries of this block, for the consumers
                        const int ls = n & (NUM_LSE - 1);
                        if (!wait_all(l_empty(ls), ((n / NUM_LSE) & 1) ^ 1, FCS_STATUS_WAIT_PRODUCER)) {
                            ok = false; break;
                        }
                        if (elect_one_sync()) {
                            mbar_arrive_expect_tx(l_full(ls), BLOCK * 4);
                            bulk_load(lse_smem + ls * BLOCK * 4, lse_src + (long long)st * BLOCK, BLOCK * 4,
                                      l_full(ls));
                        }
                    }
                    __syncwarp();
                    if (++stage == L::NS) { stage = 0; phase ^= 1; }
                }
            }
            }
        } else if (warp == MMA_WARP) {
            // -------------------------------------------- MMA issuer
            Items it;
            it.init(ps, blockIdx.x, gridDim.x);
            int a_cnt = 0, stage = 0, n = 0;
            uint32_t phase = 0;
            bool ok = true;
            if constexpr (L::SHORT) {
                int cur_bh = -1, b_cnt = 0;
                for (; ok && !it.done; it.next(ps)) {
                    const int bh = it.b * p.H + it.h;
                    if (bh != cur_bh) {
                        // the MMAs of the head before this one have read its query block: hand
                        // the buffer back, then wait for this head's block
                        if (cur_bh >= 0 && elect_one_sync()) umma_commit(b_empty(0));
                        __syncwarp();
                        if (!wait_all(b_full(0), b_cnt & 1, FCS_STATUS_WAIT_MMA)) break;
                        ++b_cnt;
                        cur_bh = bh;
                    }
                    if constexpr (L::SHORT2) {
                        // one key tile against the head's resident query blocks, a step each
                        const int ab = a_cnt % NA;
                        if (!wait_all(a_full(ab), (a_cnt / NA) & 1, FCS_STATUS_WAIT_MMA)) break;
                        const uint64_t da = umma_desc_k_sw128(a_smem + ab * L::A_BYTES);
                        for (int st = it.s0; st < it.s1; ++st, ++n) {
                            const int buf = n & (NUM_TBUF - 1);
                            if (!wait_all(t_empty(buf), ((n >> 1) & 1) ^ 1, FCS_STATUS_WAIT_MMA)) { ok = false; break; }
                            tc_fence_after();
                            const uint64_t db = umma_desc_k_sw128(b_smem + st * L::B_STAGE_BYTES);
                            const uint32_t d_tmem = tmem_base + buf * BLOCK;
                            if (elect_one_sync()) {
#pragma unroll
                                for (int ks = 0; ks < D / 16; ++ks) {
                                    const uint64_t oa = (uint64_t)(((ks >> 2) * L::A_SLAB_BYTES + (ks & 3) * 32) >> 4);
                                    const uint64_t ob = (uint64_t)(((ks >> 2) * L::B_SLAB_BYTES + (ks & 3) * 32) >> 4);
                                    umma_f16(d_tmem, da + oa, db + ob, p.idesc, ks > 0 ? 1u : 0u);
                                }
                                umma_f16(d_tmem, umma_desc_k_sw32(smem_base + L::EXTA_OFF),
                                         umma_desc_k_sw32(b_smem + st * L::B_STAGE_BYTES + L::B_BYTES), p.idesc, 1u);
                                umma_commit(t_full(buf));
                                if (st + 1 == it.s1) umma_commit(a_empty(ab));
                            }
                            __syncwarp();
                        }
                        ++a_cnt;
                        continue;
                    }
                    // one step: the item's key tiles side by side in one accumulator buffer
                    const int buf = n & (NUM_TBUF - 1);
                    if (!wait_all(t_empty(buf), ((n >> 1) & 1) ^ 1, FCS_STATUS_WAIT_MMA)) break;
                    const uint64_t db = umma_desc_k_sw128(b_smem);
                    for (int t = 0; t < it.nt; ++t, ++a_cnt) {
                        const int ab = a_cnt % NA;
                        if (!wait_all(a_full(ab), (a_cnt / NA) & 1, FCS_STATUS_WAIT_MMA)) { ok = false; break; }
                        tc_fence_after();
                        const uint64_t da = umma_desc_k_sw128(a_smem + ab * L::A_BYTES);
                        const uint32_t d_tmem = tmem_base + buf * BLOCK + t * (BLOCK / 2);
                        if (elect_one_sync()) {
#pragma unroll
                            for (int ks = 0; ks < D / 16; ++ks) {
                                const uint64_t oa = (uint64_t)(((ks >> 2) * L::A_SLAB_BYTES + (ks & 3) * 32) >> 4);
                                const uint64_t ob = (uint64_t)(((ks >> 2) * L::B_SLAB_BYTES + (ks & 3) * 32) >> 4);
                                umma_f16(d_tmem, da + oa, db + ob, p.idesc, ks > 0 ? 1u : 0u);
                            }
                            umma_f16(d_tmem, umma_desc_k_sw32(smem_base + L::EXTA_OFF),
                                     umma_desc_k_sw32(b_smem + L::B_BYTES), p.idesc, 1u);
                            umma_commit(a_empty(ab));
                            if (t + 1 == it.nt) umma_commit(t_full(buf));
                        }
                        __syncwarp();
                    }
                    ++n;
                }
            } else {
            for (; ok && !it.done; it.next(ps), ++a_cnt) {
                const int ab = a_cnt & 1;
                if (!wait_all(a_full(ab), (a_cnt >> 1) & 1, FCS_STATUS_WAIT_MMA)) break;
                const uint64_t da = umma_desc_k_sw128(a_smem + ab * L::A_BYTES);
                for (int st = it.s0; st < it.s1; ++st, ++n) {
                    if (!wait_all(b_full(stage), phase, FCS_STATUS_WAIT_MMA)) { ok = false; break; }
                    const int buf = n & (NUM_TBUF - 1);
                    if (!wait_all(t_empty(buf), ((n >> 1) & 1) ^ 1, FCS_STATUS_WAIT_MMA)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t db = umma_desc_k_sw128(b_smem + stage * L::B_STAGE_BYTES);
                    const uint32_t d_tmem = tmem_base + buf * BLOCK;
                    if (elect_one_sync()) {
#pragma unroll
                        for (int ks = 0; ks < D / 16; ++ks) {
                            // 32 bytes per 16-element step inside a slab
                            const uint64_t oa = (uint64_t)(((ks >> 2) * L::A_SLAB_BYTES + (ks & 3) * 32) >> 4);
                            const uint64_t ob = (uint64_t)(((ks >> 2) * L::B_SLAB_BYTES + (ks & 3) * 32) >> 4);
                            umma_f16(d_tmem, da + oa, db + ob, p.idesc, ks > 0 ? 1u : 0u);
                        }
                        if constexpr (EXT)   // + (key-side constant) x (-(lse)/c parts of the queries)
                            umma_f16(d_tmem, umma_desc_k_sw32(smem_base + L::EXTA_OFF),
                                     umma_desc_k_sw32(b_smem + stage * L::B_STAGE_BYTES + L::B_BYTES), p.idesc, 1u);
                        umma_commit(b_empty(stage));
                        umma_commit(t_full(buf));
                        if (st + 1 == it.s1) umma_commit(a_empty(ab));
                    }
                    __syncwarp();
                    if (++stage == L::NS) { stage = 0; phase ^= 1; }
                }
            }
            }
        }
    } else {
        // ------------------------------------------------ consumers
        const int wg = warp >> 2;                  // consumer group
        const int col0 = wg * GROUP_COLS;          // its first column of every accumulator
        const int row = ((warp & 3) << 5) | lane;  // tensor-memory lane of this thread
        const uint32_t lane_addr = tmem_base + ((uint32_t)((warp & 3) << 5) << 16) + col0;
        const float c = p.c;
        bool ok = true;

        if (MODE == MODE_STATS && p.clear_out) {
            // the output is accumulated by the column pass: clear it here
            const long long n_out = (long long)p.B * p.Sk;
            for (long long idx = (long long)blockIdx.x * CONSUMER_THREADS + threadIdx.x; idx < n_out;
                 idx += (long long)gridDim.x * CONSUMER_THREADS) {
                const long long bb = idx / p.Sk;
                p.out[bb * p.out_ld + (idx - bb * p.Sk)] = 0.f;
            }
        }

        if (MODE == MODE_STATS && p.clear_extra) {
            // a buffer the caller wants zeroed alongside this call (the target of its next call)
            for (long long idx = (long long)blockIdx.x * CONSUMER_THREADS + threadIdx.x; idx < p.clear_extra_n;
                 idx += (long long)gridDim.x * CONSUMER_THREADS)
                p.clear_extra[idx] = 0.f;
        }

        Items it;
        it.init(ps, blockIdx.x, gridDim.x);
        float m_run = -INFINITY, l_run = 0.f;      // statistics pass state
        float acc[4] = {0.f, 0.f, 0.f, 0.f};       // column pass state
        int item_cnt = 0, n = 0;
        // statistics pass: the item whose partials this group still has to combine
        bool pending = false;
        int pend_cnt = 0, pend_b = 0, pend_h = 0, pend_qt = 0, pend_sp = 0;
        auto finish_item = [&]() -> bool {
            const int slot = pend_cnt & (MERGE_SLOTS - 1);
            bool good = mbar_wait(merge_bar(slot), (pend_cnt / MERGE_SLOTS) & 1, abort_flag, p.status,
                                  FCS_STATUS_WAIT_CONSUMER);
            good = __all_sync(0xffffffffu, good);
            pending = false;
            if (!good) return false;
            const float2* mb = merge_buf + slot * CONSUMER_GROUPS * TILE;
            float mm = -INFINITY;
#pragma unroll
            for (int g = 0; g < CONSUMER_GROUPS; ++g) mm = fmaxf(mm, mb[g * TILE + row].x);
            const float ms = (mm == -INFINITY) ? 0.f : mm;
            float ll = 0.f;
#pragma unroll
            for (int g = 0; g < CONSUMER_GROUPS; ++g) {
                const float2 o = mb[g * TILE + row];
                ll += o.y * exp2f(o.x - ms);
            }
            const long long bh = (long long)pend_b * p.H + pend_h;
            const int q_abs = pend_qt * TILE + row;
            if (p.nsplit == 1) {
                const float nlv = (q_abs < p.Sq) ? -(mm + log2f(ll) + p.log2_norm) : -INFINITY;
                p.neg_lse[bh * p.lse_rows + q_abs] = nlv;
                uint4 e0, e1;
                make_ext_row(nlv, p.inv_c, p.ext_bf16 != 0, e0, e1);
                uint4* er = reinterpret_cast<uint4*>(p.ext) + (bh * p.lse_rows + q_abs) * 2;
                er[0] = e0;
                er[1] = e1;
            } else {
                const long long rows = (long long)p.NQ * TILE;
                reinterpret_cast<float2*>(p.part)[((long long)pend_sp * p.B * p.H + bh) * rows + q_abs] =
                    make_float2(mm, ll);
            }
            return true;
        };
        // short column modes: every item ends a key tile, and its sums sit in four groups.  When
        // `out` may be another GPU's memory (the _COMBINE modes) they meet in shared memory and one group,
        // a different one every item, adds them into the output after its next step -- one add per
        // key over NVLink instead of four, nobody waits.  (With a local `out` the four adds are
        // cheaper than the meeting: measured +2 % on the long-context shape.)
        float* colbuf = reinterpret_cast<float*>(smem + L::MERGE_OFF);
        bool cpend = false;
        int cp_cnt = 0, cp_b = 0, cp_kt = 0, cp_nt = 0;
        auto finish_cols = [&]() -> bool {
            const int slot = cp_cnt & (MERGE_SLOTS - 1);
            bool good = mbar_wait(merge_bar(slot), (cp_cnt / MERGE_SLOTS) & 1, abort_flag, p.status,
                                  FCS_STATUS_WAIT_CONSUMER);
            good = __all_sync(0xffffffffu, good);
            cpend = false;
            if (!good) return false;
            const float* cb = colbuf + slot * CONSUMER_GROUPS * TILE + row;
            // system scope: `out` may live on another GPU and take adds from several
            float* dst = p.out + (long long)cp_b * p.out_ld;
            const int k0 = cp_kt * TILE + row;
            if (p.col_pack == 2) {   // groups 0, 1 hold the first key tile, groups 2, 3 the second
                if (k0 < p.Sk) atomicAdd_system(dst + k0, cb[0] + cb[TILE]);
                if (cp_nt == 2 && k0 + TILE < p.Sk) atomicAdd_system(dst + k0 + TILE, cb[2 * TILE] + cb[3 * TILE]);
            } else if (k0 < p.Sk) {
                atomicAdd_system(dst + k0, (cb[0] + cb[TILE]) + (cb[2 * TILE] + cb[3 * TILE]));
            }
            return true;
        };
        for (; ok && !it.done; it.next(ps), ++item_cnt) {
            // steps f_lo <= st < f_hi need no masks: their per-step work is kept minimal
            int f_lo, f_hi;
            if constexpr (MODE == MODE_STATS) stats_full_range(ps, it.qt, f_lo, f_hi);
            else colsum_full_range(ps, it.kt, f_lo, f_hi);
            for (int st = it.s0; st < it.s1; ++st, ++n) {
                const int buf = n & (NUM_TBUF - 1);
                ok = mbar_wait(t_full(buf), (n >> 1) & 1, abort_flag, p.status, FCS_STATUS_WAIT_CONSUMER);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                const uint32_t taddr = lane_addr + buf * BLOCK;
                const bool full = (st >= f_lo) && (st < f_hi);
                if constexpr (MODE == MODE_STATS) {
                    if (full) {
                        stats_tile<false>(taddr, GROUP_COLS, c, m_run, l_run);
                    } else {
                        const int lim = stats_last_visible(p, it.qt, st, row) - col0;
                        // skip the block when no row of the tile sees any of its columns
                        const int lim_last_row = stats_last_visible(p, it.qt, st, TILE - 1) - col0;
                        if (lim_last_row >= 0) stats_tile<true>(taddr, lim, c, m_run, l_run);
                    }
                } else if constexpr (EXT) {
                    // the accumulator already holds s - lse/c
                    if (full) {
                        colsum_tile_ext<false>(taddr, 0, GROUP_COLS, c, acc);
                    } else {
                        bool done_short = false;
                        if constexpr (L::SHORT) {
                            if (p.col_pack == 2) {
                                // two key tiles in this accumulator buffer, 128 query columns each: groups
                                // 0, 1 take the halves of the first tile's columns, groups 2, 3 the second's
                                done_short = true;
                                const int tg = wg >> 1;
                                if (tg < it.nt) {
                                    const int ktg = it.kt + tg;
                                    const int q0 = (wg & 1) * GROUP_COLS;
                                    const int end = colsum_end_visible(p, st) - q0;
                                    const int thr = colsum_first_visible(p, ktg, st, row) - q0;
                                    const int thr_first_row = colsum_first_visible(p, ktg, st, 0) - q0;
                                    const int thr_last_row = colsum_first_visible(p, ktg, st, TILE - 1) - q0;
                                    if (end > 0 && thr_first_row < GROUP_COLS) {
                                        if (end >= GROUP_COLS && thr_last_row <= 0)
                                            colsum_tile_ext<false>(taddr, 0, GROUP_COLS, c, acc);
                                        else
                                            colsum_tile_ext<true>(taddr, thr, end, c, acc);
                                    }
                                }
                            } else if (colsum_end_visible(p, st) <= BLOCK / 2) {
                                // at most 128 query columns, one key tile per item: the four groups take
                                // 32 columns each, not two of them 64
                                done_short = true;
                                const int c0 = wg * (GROUP_COLS / 2);
                                const int end = colsum_end_visible(p, st) - c0;
                                const int thr = colsum_first_visible(p, it.kt, st, row) - c0;
                                const int thr_first_row = colsum_first_visible(p, it.kt, st, 0) - c0;
                                const int thr_last_row = colsum_first_visible(p, it.kt, st, TILE - 1) - c0;
                                if (end > 0 && thr_first_row < GROUP_COLS / 2) {
                                    uint32_t r[32];
                                    tmem_ld_x32(taddr - col0 + c0, r);
                                    tmem_ld_wait(r);
                                    if (end >= GROUP_COLS / 2 && thr_last_row <= 0) colsum_chunk_ext<false>(r, 0, 32, c, acc);
                                    else colsum_chunk_ext<true>(r, thr, end, c, acc);
                                }
                            }
                        }
                        if (!done_short) {
                            const int thr = colsum_first_visible(p, it.kt, st, row) - col0;
                            const int end = colsum_end_visible(p, st) - col0;
                            // skip the block when no key of the tile is seen by any of its queries
                            const int thr_first_row = colsum_first_visible(p, it.kt, st, 0) - col0;
                            if (end > 0 && thr_first_row < GROUP_COLS) colsum_tile_ext<true>(taddr, thr, end, c, acc);
                        }
                    }
                } else {
                    const int ls = n & (NUM_LSE - 1);
                    ok = mbar_wait(l_full(ls), (n / NUM_LSE) & 1, abort_flag, p.status, FCS_STATUS_WAIT_CONSUMER);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    const float4* nl = reinterpret_cast<const float4*>(smem + L::LSE_OFF + ls * BLOCK * 4) + col0 / 4;
                    if (full) {
                        colsum_tile<false>(taddr, nl, 0, GROUP_COLS, c, acc);
                    } else {
                        const int thr = colsum_first_visible(p, it.kt, st, row) - col0;
                        const int end = colsum_end_visible(p, st) - col0;
                        // skip the block when no key of the tile is seen by any of its queries
                        const int thr_first_row = colsum_first_visible(p, it.kt, st, 0) - col0;
                        if (end > 0 && thr_first_row < GROUP_COLS) colsum_tile<true>(taddr, nl, thr, end, c, acc);
                    }
                    mbar_arrive(l_empty(ls));
                }
                tc_fence_before();
                mbar_arrive(t_empty(buf));
                if constexpr (MODE == MODE_STATS) {
                    if (pending) { ok = finish_item(); if (!ok) break; }
                }
                if constexpr (L::COMBINE) {
                    if (cpend) { ok = finish_cols(); if (!ok) break; }
                }
            }
            if (!ok) break;
            if constexpr (MODE == MODE_STATS) {
                // post this group's partial (max, sum); one group, a different one every
                // item, combines the four partials after its next step, when the others
                // have long since posted -- nobody stands waiting at the end of an item
                if (pending) { ok = finish_item(); if (!ok) break; }
                const int slot = item_cnt & (MERGE_SLOTS - 1);
                merge_buf[(slot * CONSUMER_GROUPS + wg) * TILE + row] = make_float2(m_run, l_run);
                mbar_arrive(merge_bar(slot));
                if ((item_cnt % CONSUMER_GROUPS) == wg) {
                    pending = true;
                    pend_cnt = item_cnt; pend_b = it.b; pend_h = it.h; pend_qt = it.qt; pend_sp = it.sp;
                }
                m_run = -INFINITY; l_run = 0.f;
            } else if constexpr (L::SHORT) {
                if constexpr (!L::COMBINE) {
                    // four adds per key, straight from the groups: cheapest when `out` is local
                    int tg = 0;
                    bool mine = true;
                    if (p.col_pack == 2) { tg = wg >> 1; mine = tg < it.nt; }
                    const int k_abs = (it.kt + tg) * TILE + row;
                    if (k_abs < p.Sk && mine)
                        atomicAdd_system(p.out + (long long)it.b * p.out_ld + k_abs,
                                         (acc[0] + acc[1]) + (acc[2] + acc[3]));
                    acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
                } else {
                    if (cpend) { ok = finish_cols(); if (!ok) break; }
                    const int slot = item_cnt & (MERGE_SLOTS - 1);
                    colbuf[(slot * CONSUMER_GROUPS + wg) * TILE + row] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
                    mbar_arrive(merge_bar(slot));
                    if ((item_cnt % CONSUMER_GROUPS) == wg) {
                        cpend = true;
                        cp_cnt = item_cnt; cp_b = it.b; cp_kt = it.kt; cp_nt = it.nt;
                    }
                    acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
                }
            } else {
                if (it.flush()) {
                    const int k_abs = it.kt * TILE + row;
                    if (k_abs < p.Sk)
                        // system scope: `out` may live on another GPU and take adds from several
                        atomicAdd_system(p.out + (long long)it.b * p.out_ld + k_abs,
                                         (acc[0] + acc[1]) + (acc[2] + acc[3]));
                    acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
                }
            }
        }
        if constexpr (MODE == MODE_STATS) {
            if (ok && pending) finish_item();
        }
        if constexpr (L::COMBINE) {
            if (ok && cpend) finish_cols();
        }
    }

    // ---------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (MODE != MODE_STATS && p.sig_done && threadIdx.x == 0) {
        // every add of this CTA was issued before the barrier above; the last CTA to get here tells
        // the owner of the output (release, system scope) that this GPU's share of the call is in.
        // One system-scope fence per grid, by that last CTA: a system-scope fence in every CTA cost
        // 67 us on the long-context shape (they are served one after the other); the CTAs hand
        // their writes on to it through device-scope fences and the counter.
        __threadfence();
        const int arrived = atomicAdd(p.sig_counter, 1);
        if (arrived == (int)gridDim.x - 1) {
            *p.sig_counter = 0;
            release_store_system_one(p.sig_done, p.sig_done_value);
        }
    }
    if (warp == MMA_WARP) {
        if (*abort_flag) __nanosleep(1000000);   // let copies and MMAs in flight land
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// Combine the key-range partials of the statistics pass into the per-row value
// the column pass subtracts.
__global__ void merge_stats_kernel(const Problem p) {
    grid_dependency_wait();
    grid_launch_dependents();
    const long long rows = (long long)p.NQ * TILE;
    const long long n = (long long)p.B * p.H * rows;
    const float2* part = reinterpret_cast<const float2*>(p.part);
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long bh = idx / rows;
        const int q_abs = (int)(idx - bh * rows);
        float v = -INFINITY;
        if (q_abs < p.Sq) {
            float mm = -INFINITY;
            for (int s = 0; s < p.nsplit; ++s) mm = fmaxf(mm, part[s * n + idx].x);
            float ll = 0.f;
            for (int s = 0; s < p.nsplit; ++s) {
                const float2 t = part[s * n + idx];
                ll += t.y * exp2f(t.x - mm);
            }
            v = -(mm + log2f(ll) + p.log2_norm);
        }
        p.neg_lse[bh * p.lse_rows + q_abs] = v;
        uint4 e0, e1;
        make_ext_row(v, p.inv_c, p.ext_bf16 != 0, e0, e1);
        uint4* er = reinterpret_cast<uint4*>(p.ext) + (bh * p.lse_rows + q_abs) * 2;
        er[0] = e0;
        er[1] = e1;
    }
}

// ---------------------------------------------------------------------------
// Flags between the GPUs of a node (peer-mapped memory), for callers that order their
// kernels across ranks without a collective: a release store per flag, and a bounded wait
// until every flag has reached a value.
// ---------------------------------------------------------------------------
}  // namespace fcs

#include "colsum_fused_short.cuh"

namespace fcs {

constexpr int PEER_FLAGS_MAX = 16;
struct PeerFlagPointers { int* p[PEER_FLAGS_MAX]; };

__global__ void peer_post_kernel(const PeerFlagPointers flags, int n, int value) {
    if ((int)threadIdx.x < n) {
        // everything the kernels before this one in the stream wrote (to any GPU) is visible to
        // whoever reads this value with an acquire load
        __threadfence_system();
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(flags.p[threadIdx.x]), "r"(value) : "memory");
    }
}

__global__ void peer_wait_kernel(const int* flags, int n, int value, int* status) {
    if ((int)threadIdx.x < n) {
        const long long t0 = clock64();
        unsigned spins = 0;
        while (true) {
            int v;
            asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flags + threadIdx.x) : "memory");
            if (v >= value) break;
            if ((++spins & 63u) == 0u && clock64() - t0 > g_wait_limit_cycles) {
                if (status) atomicCAS(status, 0, FCS_STATUS_WAIT_PEER);
                break;
            }
            __nanosleep(100);
        }
    }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
static thread_local char g_err[512] = "";

static int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

static int num_sms() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

// (D, S, H, B) view of a [B, H, S, D] tensor, boxes of `box_rows` rows x 64
// elements, 128-byte swizzle, out-of-range rows read as zero -- and so do the columns
// from D on when D is not a multiple of 64: the kernels contract 64 or 128 columns, the
// padding adds nothing to a score.
static int make_tensor_map(CUtensorMap* m, const void* base, int dtype, int B, int H, int S, int D,
                           int64_t sb, int64_t sh, int64_t ss, int box_rows) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return fail(FCS_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)S, (cuuint64_t)H, (cuuint64_t)B};
    cuuint64_t strides[3] = {(cuuint64_t)ss * 2, (cuuint64_t)sh * 2, (cuuint64_t)sb * 2};
    cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(m, dtype == FCS_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                     4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(FCS_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return FCS_OK;
}

// Optional per-pass timing: when enabled, events are recorded on the caller's
// stream around each kernel of a call.
struct PassTimers {
    bool ready = false;
    bool recorded = false;
    cudaEvent_t ev[4];
};
static bool g_profiling = false;
static PassTimers g_timers[64];

static PassTimers* timers_for_current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    PassTimers& t = g_timers[dev];
    if (!t.ready) {
        for (int i = 0; i < 4; ++i)
            if (cudaEventCreate(&t.ev[i]) != cudaSuccess) return nullptr;
        t.ready = true;
    }
    return &t;
}

// (16, rows, planes) view of the [planes][rows][16] extension columns: boxes of 256
// rows x 16 elements (32 bytes), 32-byte swizzle.
static int make_ext_tensor_map(CUtensorMap* m, const void* base, int dtype, long long planes, long long rows) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return fail(FCS_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[3] = {(cuuint64_t)EXT_K, (cuuint64_t)rows, (cuuint64_t)planes};
    cuuint64_t strides[2] = {(cuuint64_t)EXT_ROW_BYTES, (cuuint64_t)rows * EXT_ROW_BYTES};
    cuuint32_t box[3] = {(cuuint32_t)EXT_K, (cuuint32_t)BLOCK, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(m, dtype == FCS_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                     3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(FCS_ERR_CUDA, "cuTensorMapEncodeTiled (extension) failed with CUresult %d", (int)r);
    return FCS_OK;
}

template <int D, int MODE>
static cudaError_t launch_stream(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& text,
                                 const Problem& p, int grid, cudaStream_t stream, bool after_own_kernel) {
    using LayoutT = Layout<D, MODE>;
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kern = colsum_stream_kernel<D, MODE>;
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             LayoutT::DYN_BYTES);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = LayoutT::DYN_BYTES;
    cfg.stream = stream;
    // a pass that follows another kernel of the same call starts its set-up (barriers, tensor
    // memory) while that kernel drains; it waits for it inside (grid_dependency_wait)
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = after_own_kernel ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, ta, tb, text, p);
}

static long long sms_for_clear() { return num_sms(); }

// Rows of 16-byte multiples (what a tensor map and a bulk copy can address), at most two
// 64-column slabs.
static bool head_dim_ok(int D) { return D >= 8 && D <= 128 && D % 8 == 0; }

static int check_operand(const char* name, const void* ptr, int64_t sb, int64_t sh, int64_t ss) {
    if (!ptr) return fail(FCS_ERR_INVALID_ARGUMENT, "%s is NULL", name);
    if (reinterpret_cast<uintptr_t>(ptr) % 16)
        return fail(FCS_ERR_INVALID_ARGUMENT, "%s must be 16-byte aligned", name);
    if (sb <= 0 || sh <= 0 || ss <= 0 || sb % 8 || sh % 8 || ss % 8)
        return fail(FCS_ERR_INVALID_ARGUMENT,
                    "%s strides must be positive multiples of 8 elements (got b=%lld h=%lld s=%lld)", name,
                    (long long)sb, (long long)sh, (long long)ss);
    return FCS_OK;
}

// Few query rows: the matrix-vector kernel (a kernel that clears the output, then the
// clustered kernel as its programmatic dependent).
template <int D, bool BF16, int RMAX, int W>
static cudaError_t launch_small_q_w(const SmallQParams& sp, int grid, size_t smem, cudaStream_t stream,
                                    bool after_clear) {
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kern = colsum_small_q_kernel<D, BF16, RMAX, W>;
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMALLQ_MAX_SMEM);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(32 * (W + 1));
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    // The cluster attribute is given for clusters of one as well: the kernel's cluster instructions
    // (barrier.cluster, mapa, st.async) are illegal in a launch without it.
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = (unsigned)sp.CL;
    attrs[0].val.clusterDim.y = 1;
    attrs[0].val.clusterDim.z = 1;
    // behind the clearing kernel: start at once, wait for it only before the adds
    attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = after_clear ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kern, sp);
}

template <int D, bool BF16, int RMAX>
static cudaError_t launch_small_q_r(const SmallQParams& sp, int grid, size_t smem, cudaStream_t stream,
                                    bool after_clear) {
    if (sp.wide) return launch_small_q_w<D, BF16, RMAX, SMALLQ_WIDE_WARPS>(sp, grid, smem, stream, after_clear);
    return launch_small_q_w<D, BF16, RMAX, SMALLQ_CONSUMER_WARPS>(sp, grid, smem, stream, after_clear);
}

template <int D, bool BF16>
static cudaError_t launch_small_q_t(const SmallQParams& sp, int grid, size_t smem, cudaStream_t stream,
                                    bool after_clear) {
    if (sp.R == 1) return launch_small_q_r<D, BF16, 1>(sp, grid, smem, stream, after_clear);
    if (sp.R == 2) return launch_small_q_r<D, BF16, 2>(sp, grid, smem, stream, after_clear);
    return launch_small_q_r<D, BF16, 4>(sp, grid, smem, stream, after_clear);
}

static int launch_small_q(const void* q, const void* k, float* out, int64_t out_ld, int B, int H, int R, int Sk,
                          int D, int dtype, int64_t qsb, int64_t qsh, int64_t qss, int64_t ksb, int64_t ksh,
                          int64_t kss, float scale, int causal, int k_past, int h_norm, bool clear_out,
                          int* status, cudaStream_t stream) {
    const int sms = num_sms();
    if (clear_out) {
        long long blocks = ((long long)B * Sk + 1023) / 1024;
        if (blocks > sms) blocks = sms;
        clear_rows_kernel<<<(unsigned)blocks, 256, 0, stream>>>(out, (long long)out_ld, B, Sk);
        const cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return fail(FCS_ERR_CUDA, "clearing the output failed: %s", cudaGetErrorString(e));
    }
    SmallQParams sp;
    memset(&sp, 0, sizeof(sp));
    sp.q = q; sp.k = k; sp.out = out; sp.out_ld = out_ld;
    sp.H = H; sp.R = R; sp.Sk = Sk;
    sp.qsb = qsb; sp.qsh = qsh; sp.qss = qss; sp.ksb = ksb; sp.ksh = ksh; sp.kss = kss;
    sp.c = scale * 1.4426950408889634f;
    sp.causal = causal; sp.k_past = causal ? k_past : 0;
    sp.inv_norm = 1.0f / ((float)h_norm * (float)R);
    sp.status = status;
    // keys past the last query's horizon are seen by no row: not read, their columns stay zero
    long long keys = Sk;
    if (causal && (long long)k_past + R < keys) keys = (long long)k_past + R;
    sp.keys = (int)keys;
    size_t smem = 0;
    sp.units = B * H;
    if (!smallq_plan(sp.units, R, sp.keys, D, sms, &sp.CL, &sp.clusters, &sp.range_rows, &sp.stages, &sp.bufs, &sp.wide, &smem))
        return fail(FCS_ERR_UNSUPPORTED, "few-row kernel: %d keys do not fit", Sk);
    const int grid = sp.clusters * sp.CL;
    const bool bf16 = dtype == FCS_DTYPE_BF16;
    const cudaError_t e =
        (D == 64) ? (bf16 ? launch_small_q_t<64, true>(sp, grid, smem, stream, clear_out)
                          : launch_small_q_t<64, false>(sp, grid, smem, stream, clear_out))
                  : (bf16 ? launch_small_q_t<128, true>(sp, grid, smem, stream, clear_out)
                          : launch_small_q_t<128, false>(sp, grid, smem, stream, clear_out));
    if (e != cudaSuccess) return fail(FCS_ERR_CUDA, "few-row kernel launch failed: %s", cudaGetErrorString(e));
    return FCS_OK;
}

// Short key axes (non-causal, head dimension 64, S_k <= 2048): the single-pass
// cluster kernel.  g_single_pass: 0 = where it is the faster of the two (see
// single_pass_applies), 1 = never, 2 = whenever the shape allows.
static int g_single_pass = 0;

static int single_pass_cluster_size(int Sk) {
    return (Sk + 255) / 256;   // one CTA per 256 keys; any size up to eight is a legal cluster
}

static bool single_pass_applies(int B, int H, int Sq, int Sk, int D, int causal) {
    if (g_single_pass == 1 || causal || D > 64 || Sk > 256 * sp::MAX_CL) return false;   // (D < 64: zero-filled columns)
    if (g_single_pass == 2) return true;
    const int cl = single_pass_cluster_size(Sk);
    // measured at B=32 H=16 against the two passes: 1.2-1.3x at 400-1024 keys, 1.07-1.14x at
    // 1152-1536, 1.02x at 577 (75 % of three slices); clusters of 7 and 8 fit only 15 at a time
    // (105 / 120 of 148 SMs) and lose on large calls (0.84x / 0.95x) but win on small ones,
    // where the fixed costs of two launches and partial waves weigh more
    if (cl <= 6) return (long long)Sk * 100 >= (long long)cl * 256 * 75;
    if ((long long)Sk * 100 < (long long)cl * 256 * 85) return false;
    const long long tiles = (long long)B * H * ((Sq + TILE - 1) / TILE);
    return tiles <= 512;
}

// Clusters of `cl` CTAs that can be resident at once (0 if the query fails).
static int single_pass_max_clusters(int cl) {
    static int cached[64][sp::MAX_CL + 1] = {{0}};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || cl < 1 || cl > sp::MAX_CL) return 0;
    const int idx = cl;
    if (cached[dev][idx] == 0) {
        if (cudaFuncSetAttribute(colsum_single_pass_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 sp::DYN_BYTES) != cudaSuccess)
            return 0;
        cudaLaunchConfig_t cfg;
        memset(&cfg, 0, sizeof(cfg));
        cfg.gridDim = dim3((unsigned)(cl * 64));
        cfg.blockDim = dim3(sp::THREADS);
        cfg.dynamicSmemBytes = sp::DYN_BYTES;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = (unsigned)cl;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, colsum_single_pass_kernel, &cfg) != cudaSuccess || n <= 0) {
            cudaGetLastError();
            return 0;
        }
        cached[dev][idx] = n;
    }
    return cached[dev][idx];
}

static int launch_single_pass(const CUtensorMap& tq, const CUtensorMap& tk, float* out, int64_t out_ld, int B,
                              int H, int Sq, int Sk, float scale, int h_norm, int dtype, bool clear_out,
                              int max_clusters, int* status, cudaStream_t stream) {
    cudaError_t e = cudaSuccess;
    if (clear_out)
        e = cudaMemset2DAsync(out, (size_t)out_ld * sizeof(float), 0, (size_t)Sk * sizeof(float), (size_t)B, stream);
    if (e != cudaSuccess) return fail(FCS_ERR_CUDA, "clearing the output failed: %s", cudaGetErrorString(e));
    SinglePassParams sp_;
    memset(&sp_, 0, sizeof(sp_));
    sp_.B = B; sp_.H = H; sp_.Sq = Sq; sp_.Sk = Sk;
    sp_.NQ = (Sq + TILE - 1) / TILE;
    sp_.CL = single_pass_cluster_size(Sk);
    sp_.units = B * H;
    // the (batch, head, query tile) list is cut evenly over the clusters, through pairs if need be
    {
        const long long tiles = (long long)sp_.units * sp_.NQ;
        sp_.clusters = tiles < max_clusters ? (int)tiles : max_clusters;
    }
    // at most ~1024 accumulations (16 query rows each) per flush
    sp_.flush_units = 128 / sp_.NQ > 1 ? 128 / sp_.NQ : 1;
    sp_.c = fabsf(scale) * 1.4426950408889634f;
    sp_.out_scale = 1.0f / ((float)h_norm * (float)Sq * 1024.0f);
    sp_.out = out;
    sp_.out_ld = out_ld;
    sp_.status = status;
    const uint32_t fmt = dtype == FCS_DTYPE_BF16 ? 1u : 0u;
    // one score MMA covers the 256 keys of the slice: M = 128, N = 256
    sp_.idesc_scores = (1u << 4) | (fmt << 7) | (fmt << 10) | ((scale < 0.f ? 1u : 0u) << 13) |
                       ((uint32_t)(BLOCK >> 3) << 17) | ((uint32_t)(TILE >> 4) << 24);
    // fp16 x fp16 -> fp32, A stored with the M index contiguous, B K-major, M = 128, N = 16
    sp_.idesc_colsum = (1u << 4) | (1u << 15) | ((uint32_t)(sp::W_N >> 3) << 17) | ((uint32_t)(TILE >> 4) << 24);
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)(sp_.clusters * sp_.CL));
    cfg.blockDim = dim3(sp::THREADS);
    cfg.dynamicSmemBytes = sp::DYN_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = (unsigned)sp_.CL;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, colsum_single_pass_kernel, tq, tk, sp_);
    if (e != cudaSuccess) return fail(FCS_ERR_CUDA, "single-pass kernel launch failed: %s", cudaGetErrorString(e));
    return FCS_OK;
}

// Short query axis over a short key axis: the one-kernel cluster form.
// g_short_fused: 0 = where fused_short_plan says so, 1 = never, 2 = whenever the query
// rows fit one tile.
static int g_short_fused = 0;

// Clusters of 1..8 CTAs of the one-kernel form that the current device runs at once
// (table[c]; fewer than SMs / c: a cluster stays inside one GPC).  Without a device to ask,
// seven eighths of SMs / c, which is what a B200 answers for clusters of four and of eight.
template <int D>
static const int* fused_short_max_clusters() {
    static int cached[64][fused::MAX_CL + 1] = {{0}};
    static int fallback[fused::MAX_CL + 1];
    int dev = 0;
    const bool have_dev = cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64;
    if (!have_dev) cudaGetLastError();
    const int sms = num_sms();
    int* table = have_dev ? cached[dev] : fallback;
    if (have_dev && table[1] != 0) return table;
    auto kern = fused::colsum_fused_short_kernel<D>;
    bool ask = have_dev && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                fused::FLayout<D>::DYN_BYTES) == cudaSuccess;
    for (int cl = 1; cl <= fused::MAX_CL; ++cl) {
        int n = 0;
        if (ask) {
            cudaLaunchConfig_t cfg;
            memset(&cfg, 0, sizeof(cfg));
            cfg.gridDim = dim3((unsigned)(cl * 64));
            cfg.blockDim = dim3(THREADS);
            cfg.dynamicSmemBytes = fused::FLayout<D>::DYN_BYTES;
            cudaLaunchAttribute attr;
            attr.id = cudaLaunchAttributeClusterDimension;
            attr.val.clusterDim.x = (unsigned)cl;
            attr.val.clusterDim.y = 1;
            attr.val.clusterDim.z = 1;
            cfg.attrs = &attr;
            cfg.numAttrs = 1;
            if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
                cudaGetLastError();
                n = 0;
            }
        }
        if (n <= 0) n = cl == 1 ? sms : (sms / cl) * 7 / 8;
        table[cl] = n > 0 ? n : 1;
    }
    return table;
}

static bool short_fused_applies(int B, int H, int Sq, int Sk, int D, int causal, int k_past, int* cl_out,
                                int* nkb_out, int* bpc_out) {
    if (g_short_fused == 1) return false;
    if (causal && k_past < 0) k_past = Sk > Sq ? Sk - Sq : 0;
    const int* table = D <= 64 ? fused_short_max_clusters<64>() : fused_short_max_clusters<128>();
    return fused_short_plan(B, H, Sq, Sk, causal, causal ? k_past : 0, num_sms(), table, g_short_fused == 2, cl_out,
                            nkb_out, bpc_out);
}

// Whether all (batch, head) pairs of a call the one-kernel form takes run at once: such a call
// goes there even where the single-pass kernel would take it (B=4 H=16, 100 CLS rows over 577
// keys: 19 against 23.5 us); with several waves of CTAs the single-pass kernel keeps it (B=32:
// 50 against 58 us).
static bool short_fused_one_wave(int B, int H, int D, int cl) {
    const int* table = D <= 64 ? fused_short_max_clusters<64>() : fused_short_max_clusters<128>();
    return (long long)B * H <= (cl > 1 ? table[cl] : num_sms());
}

template <int D>
static cudaError_t launch_fused_short_d(const CUtensorMap& tq, const CUtensorMap& tk, const fused::Params& fp,
                                        cudaStream_t stream, bool after_clear) {
    using LayoutT = fused::FLayout<D>;
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kern = fused::colsum_fused_short_kernel<D>;
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, LayoutT::DYN_BYTES);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)((long long)fp.p.B * fp.p.H * fp.CL));
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = LayoutT::DYN_BYTES;
    cfg.stream = stream;
    // (the cluster attribute also for clusters of one: the kernel uses cluster instructions)
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = (unsigned)fp.CL;
    attrs[0].val.clusterDim.y = 1;
    attrs[0].val.clusterDim.z = 1;
    // behind the clearing kernel: start at once, wait for it only before the adds
    attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = after_clear ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kern, tq, tk, fp);
}

// `p` carries the sizes, the mask rule, the scale and the output; tq: boxes of 128 query rows,
// tk: boxes of 256 key rows.
static int launch_fused_short(const CUtensorMap& tq, const CUtensorMap& tk, const Problem& p, int DK, float scale,
                              bool use_ext, int cl, int nkb, int bpc, bool clear_out, float* clear_extra,
                              long long clear_extra_n, cudaStream_t stream) {
    if (clear_extra && clear_extra_n > 0) {
        long long blocks = (clear_extra_n + 1023) / 1024;
        if (blocks > sms_for_clear()) blocks = sms_for_clear();
        clear_rows_kernel<<<(unsigned)blocks, 256, 0, stream>>>(clear_extra, clear_extra_n, 1, (int)clear_extra_n);
    }
    if (clear_out) {
        long long blocks = ((long long)p.B * p.Sk + 1023) / 1024;
        if (blocks > num_sms()) blocks = num_sms();
        clear_rows_kernel<<<(unsigned)blocks, 256, 0, stream>>>(p.out, p.out_ld, p.B, p.Sk);
        const cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return fail(FCS_ERR_CUDA, "clearing the output failed: %s", cudaGetErrorString(e));
    }
    fused::Params fp;
    memset(&fp, 0, sizeof(fp));
    fp.p = p;
    fp.CL = cl;
    fp.nkb = nkb;
    fp.blocks_per_cta = bpc;
    fp.use_ext = use_ext ? 1 : 0;
    const uint32_t fmt = p.ext_bf16 ? 1u : 0u;
    const uint32_t common = (1u << 4) | (fmt << 7) | (fmt << 10) | ((scale < 0.f ? 1u : 0u) << 13) |
                            ((uint32_t)(TILE >> 4) << 24);
    fp.idesc_scores = common | ((uint32_t)(BLOCK >> 3) << 17);
    fp.idesc_cols = common | ((uint32_t)((BLOCK / 2) >> 3) << 17);
    const cudaError_t e = (DK == 64) ? launch_fused_short_d<64>(tq, tk, fp, stream, clear_out)
                                     : launch_fused_short_d<128>(tq, tk, fp, stream, clear_out);
    if (e != cudaSuccess) return fail(FCS_ERR_CUDA, "one-kernel short form launch failed: %s", cudaGetErrorString(e));
    return FCS_OK;
}

enum : int { PASSES_BOTH = 0, PASSES_STATS = 1, PASSES_COLUMNS = 2 };

// -(log-sum-exp) per query row -> the 16 extension columns the column pass contracts with.
__global__ void ext_from_lse_kernel(const Problem p) {
    const long long n = (long long)p.B * p.H * p.lse_rows;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
         idx += (long long)gridDim.x * blockDim.x) {
        uint4 e0, e1;
        make_ext_row(p.neg_lse[idx], p.inv_c, p.ext_bf16 != 0, e0, e1);
        uint4* er = reinterpret_cast<uint4*>(p.ext) + idx * 2;
        er[0] = e0;
        er[1] = e1;
    }
}

// The one implementation behind the three entry points.
static int colsum_impl(const void* q, const void* k, float* out, int64_t out_ld, int B, int H, int Sq_full,
                       int Sk, int D, int dtype, int64_t qsb, int64_t qsh, int64_t qss, int64_t ksb,
                       int64_t ksh, int64_t kss, float scale, int causal, int k_past, int cls_n, int h_norm,
                       void* workspace, size_t workspace_bytes, int* status, void* stream_v,
                       bool clear_out = true, int passes = PASSES_BOTH, float* shared_lse = nullptr,
                       long long norm_rows = 0, float* clear_extra = nullptr, long long clear_extra_n = 0,
                       const FcsPeerSignals* sig = nullptr) {
    // passes: both, or one of the two for work split over devices (non-causal only) --
    // PASSES_STATS writes -(log-sum-exp + log2(h_norm * norm_rows)) of the given query rows to
    // `shared_lse`; PASSES_COLUMNS takes that vector for ALL query rows and the given keys.
    g_err[0] = 0;
    if (B <= 0 || H <= 0 || Sq_full <= 0 || Sk <= 0)
        return fail(FCS_ERR_INVALID_ARGUMENT, "sizes must be positive (B=%d H=%d Sq=%d Sk=%d)", B, H, Sq_full, Sk);
    if (!head_dim_ok(D))
        return fail(FCS_ERR_UNSUPPORTED, "head dimension must be a multiple of 8 from 8 to 128, got %d", D);
    if (dtype != FCS_DTYPE_FP16 && dtype != FCS_DTYPE_BF16)
        return fail(FCS_ERR_UNSUPPORTED, "dtype must be FCS_DTYPE_FP16 or FCS_DTYPE_BF16, got %d", dtype);
    const int DK = D <= 64 ? 64 : 128;   // columns the streaming kernels contract (zero-filled beyond D)
    if (passes != PASSES_STATS) {
        if (!out) return fail(FCS_ERR_INVALID_ARGUMENT, "out is NULL");
        if (out_ld < Sk)
            return fail(FCS_ERR_INVALID_ARGUMENT, "out_ld (%lld) is smaller than the key length", (long long)out_ld);
    }
    if (passes != PASSES_BOTH) {
        if (causal) return fail(FCS_ERR_UNSUPPORTED, "the passes can be run apart for non-causal calls only");
        if (!shared_lse || reinterpret_cast<uintptr_t>(shared_lse) % 16)
            return fail(FCS_ERR_INVALID_ARGUMENT, "the statistics vector must be a 16-byte aligned device pointer");
    }
    if (!isfinite(scale)) return fail(FCS_ERR_INVALID_ARGUMENT, "scale must be finite");
    if (!causal && cls_n != -1 && cls_n <= 0)
        return fail(FCS_ERR_INVALID_ARGUMENT, "cls_n must be -1 or positive, got %d", cls_n);
    int rc;
    if ((rc = check_operand("q", q, qsb, qsh, qss)) != FCS_OK) return rc;
    if ((rc = check_operand("k", k, ksb, ksh, kss)) != FCS_OK) return rc;
    if (h_norm <= 0) h_norm = H;

    int Sq = Sq_full;                       // rows that enter the mean
    if (!causal && cls_n > 0 && cls_n < Sq_full) Sq = cls_n;
    if (causal && k_past < 0) k_past = Sk > Sq ? Sk - Sq : 0;

    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
    if (sig && passes == PASSES_BOTH && smallq_fits(Sq, Sk, D, B * H, num_sms()))
        return fail(FCS_ERR_UNSUPPORTED, "calls with at most four query rows take the few-row kernel, which does not "
                                         "signal other GPUs; order them with a barrier");
    if (passes == PASSES_BOTH && smallq_fits(Sq, Sk, D, B * H, num_sms())) {
        // reported as a call whose statistics and merge passes take no time
        PassTimers* tms = g_profiling ? timers_for_current_device() : nullptr;
        if (tms) {
            tms->recorded = false;
            for (int i = 0; i < 3; ++i) cudaEventRecord(tms->ev[i], stream);
        }
        if (clear_extra && clear_extra_n > 0) {
            clear_rows_kernel<<<(unsigned)((clear_extra_n + 1023) / 1024 < sms_for_clear() ? (clear_extra_n + 1023) / 1024
                                                                                          : sms_for_clear()),
                                256, 0, stream>>>(clear_extra, clear_extra_n, 1, (int)clear_extra_n);
        }
        rc = launch_small_q(q, k, out, out_ld, B, H, Sq, Sk, D, dtype, qsb, qsh, qss, ksb, ksh, kss, scale,
                            causal, k_past, h_norm, clear_out, status, stream);
        if (rc == FCS_OK && tms) { cudaEventRecord(tms->ev[3], stream); tms->recorded = true; }
        return rc;
    }

    const int sms = num_sms();
    // -(lse) rides in the MMA of the column pass unless the scale is so small that
    // -(lse)/c leaves the range of its 16-bit parts
    const bool use_ext = fabsf(scale) * 1.4426950408889634f >= 1e-4f;
    Problem p;
    memset(&p, 0, sizeof(p));
    plan(p, B, H, Sq, Sk, causal, k_past, sms, COL_INTERLEAVE_MIN_ROWS, /*head_major_ok=*/use_ext);
    p.ext_bf16 = dtype == FCS_DTYPE_BF16 ? 1 : 0;
    p.out = out;
    p.out_ld = out_ld;
    p.clear_out = (clear_out && passes == PASSES_BOTH) ? 1 : 0;   // (the statistics pass does the clearing)
    p.col_combine = clear_out ? 0 : 1;   // accumulating into a caller's buffer: it may be peer-mapped
    p.clear_extra = clear_extra_n > 0 ? clear_extra : nullptr;
    p.clear_extra_n = clear_extra_n;
    p.status = status;
    p.c = fabsf(scale) * 1.4426950408889634f;
    p.inv_c = use_ext ? (scale < 0.f ? -1.0f : 1.0f) / p.c : 0.f;
    p.log2_norm = log2f((float)h_norm * (float)(norm_rows > 0 ? norm_rows : Sq));
    const uint32_t fmt = dtype == FCS_DTYPE_BF16 ? 1u : 0u;
    // fp32 accumulate, K-major A and B, M = 128, N = 256; a negative scale negates A
    p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((scale < 0.f ? 1u : 0u) << 13) |
              ((uint32_t)(BLOCK >> 3) << 17) | ((uint32_t)(TILE >> 4) << 24);

    // each tensor is the resident operand (128-row boxes) of one pass and the
    // streamed operand (256-row boxes) of the other
    // (the two cluster kernels take queries in 128-row and keys in 256-row boxes only: the other two
    // maps are encoded once it is known that the streaming passes run -- an encode is a microsecond
    // of host time, and the calls the cluster kernels take are bound by the host when issued back to back)
    CUtensorMap tq_a, tq_b, tk_a, tk_b;
    if ((rc = make_tensor_map(&tq_a, q, dtype, B, H, Sq, D, qsb, qsh, qss, TILE)) != FCS_OK) return rc;
    if ((rc = make_tensor_map(&tk_b, k, dtype, B, H, Sk, D, ksb, ksh, kss, BLOCK)) != FCS_OK) return rc;
    int fcl = 0, fnkb = 0, fbpc = 0;
    const bool fused_ok = passes == PASSES_BOTH && !sig && short_fused_applies(B, H, Sq, Sk, D, causal, k_past, &fcl, &fnkb, &fbpc);
    const bool fused_first = fused_ok && short_fused_one_wave(B, H, D, fcl);
    if (passes == PASSES_BOTH && !fused_first && single_pass_applies(B, H, Sq, Sk, D, causal)) {
        const int max_clusters = single_pass_max_clusters(single_pass_cluster_size(Sk));
        if (max_clusters > 0) {
            // reported as a call whose statistics and merge passes take no time
            PassTimers* tms = g_profiling ? timers_for_current_device() : nullptr;
            if (tms) {
                tms->recorded = false;
                for (int i = 0; i < 3; ++i) cudaEventRecord(tms->ev[i], stream);
            }
            rc = launch_single_pass(tq_a, tk_b, out, out_ld, B, H, Sq, Sk, scale, h_norm, dtype, clear_out,
                                    max_clusters, status, stream);
            if (rc == FCS_OK && tms) { cudaEventRecord(tms->ev[3], stream); tms->recorded = true; }
            return rc;
        }
    }
    {
        if (fused_ok) {
            // reported as a call whose statistics and merge passes take no time
            PassTimers* tms = g_profiling ? timers_for_current_device() : nullptr;
            if (tms) {
                tms->recorded = false;
                for (int i = 0; i < 3; ++i) cudaEventRecord(tms->ev[i], stream);
            }
            rc = launch_fused_short(tq_a, tk_b, p, DK, scale, use_ext, fcl, fnkb, fbpc, clear_out, clear_extra,
                                    clear_extra_n, stream);
            if (rc == FCS_OK && tms) { cudaEventRecord(tms->ev[3], stream); tms->recorded = true; }
            return rc;
        }
    }
    if ((rc = make_tensor_map(&tq_b, q, dtype, B, H, Sq, D, qsb, qsh, qss, BLOCK)) != FCS_OK) return rc;
    if ((rc = make_tensor_map(&tk_a, k, dtype, B, H, Sk, D, ksb, ksh, kss, TILE)) != FCS_OK) return rc;
    // the two streaming passes are the only kernels that use scratch memory
    size_t part_off = 0, ext_off = 0;
    const size_t need = workspace_layout(p, &part_off, &ext_off);
    if (!workspace || workspace_bytes < need)
        return fail(FCS_ERR_WORKSPACE, "workspace too small: need %zu bytes, got %zu", need, workspace_bytes);
    if (reinterpret_cast<uintptr_t>(workspace) % 256)
        return fail(FCS_ERR_WORKSPACE, "workspace must be 256-byte aligned");
    p.neg_lse = passes == PASSES_BOTH ? reinterpret_cast<float*>(workspace) : shared_lse;
    p.part = reinterpret_cast<uint8_t*>(workspace) + part_off;
    p.ext = reinterpret_cast<uint8_t*>(workspace) + ext_off;
    CUtensorMap text = tq_b;   // placeholder when the extension is not used
    if (use_ext && (rc = make_ext_tensor_map(&text, p.ext, dtype, (long long)B * H, p.lse_rows)) != FCS_OK) return rc;

    const int grid1 = (int)(p.stats_items < sms ? p.stats_items : sms);
    stats_set_grid(p, grid1);
    long long col_items = p.steps_total;
    if (p.col_interleave == COL_HEAD_MAJOR) col_items = (long long)B * H * ceil_div(p.NKC, p.col_pack);
    const int grid2 = (int)(col_items < sms ? col_items : sms);
    PassTimers* tm = g_profiling ? timers_for_current_device() : nullptr;
    if (tm) { tm->recorded = false; cudaEventRecord(tm->ev[0], stream); }
    cudaError_t e = cudaSuccess;
    if (passes == PASSES_COLUMNS) {
        // the caller's statistics -> the column pass's operand form; the output starts from zero
        int blocks = (int)(((long long)B * H * p.lse_rows + 255) / 256);
        if (blocks > sms * 8) blocks = sms * 8;
        ext_from_lse_kernel<<<blocks, 256, 0, stream>>>(p);
        e = cudaGetLastError();
        if (e == cudaSuccess && clear_out)
            e = cudaMemset2DAsync(out, (size_t)out_ld * sizeof(float), 0, (size_t)Sk * sizeof(float), (size_t)B, stream);
        if (e != cudaSuccess) return fail(FCS_ERR_CUDA, "preparing the column pass failed: %s", cudaGetErrorString(e));
    } else {
        e = (DK == 64) ? launch_stream<64, MODE_STATS>(tq_a, tk_b, text, p, grid1, stream, false)
                      : launch_stream<128, MODE_STATS>(tq_a, tk_b, text, p, grid1, stream, false);
    }
    if (e != cudaSuccess) return fail(FCS_ERR_CUDA, "statistics pass launch failed: %s", cudaGetErrorString(e));
    if (tm) cudaEventRecord(tm->ev[1], stream);
    if (p.nsplit > 1 && passes != PASSES_COLUMNS) {
        const long long n = (long long)B * H * p.NQ * TILE;
        int blocks = (int)((n + 255) / 256);
        if (blocks > sms * 8) blocks = sms * 8;
        cudaLaunchConfig_t cfg;
        memset(&cfg, 0, sizeof(cfg));
        cfg.gridDim = dim3((unsigned)blocks);
        cfg.blockDim = dim3(256);
        cfg.stream = stream;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr.val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = tm ? 0 : 1;   // (event records between the kernels when timing is on)
        e = cudaLaunchKernelEx(&cfg, merge_stats_kernel, p);
        if (e != cudaSuccess) return fail(FCS_ERR_CUDA, "statistics merge launch failed: %s", cudaGetErrorString(e));
    }
    if (tm) cudaEventRecord(tm->ev[2], stream);
    if (passes == PASSES_STATS) {
        if (tm) { cudaEventRecord(tm->ev[3], stream); tm->recorded = true; }
        return FCS_OK;
    }
    const bool chained = !tm && passes == PASSES_BOTH;   // directly behind a kernel of this call
    // a query axis of at most 128 rows fills half a streamed block: the MMAs need N = 128 only
    if (Sq <= BLOCK / 2)
        p.idesc = (p.idesc & ~(0x3Fu << 17)) | ((uint32_t)((BLOCK / 2) >> 3) << 17);
    if (sig) {   // the column pass orders itself against the other GPUs of a head-sharded call
        p.sig_wait = sig->wait_flag;
        p.sig_wait_value = sig->wait_value;
        p.sig_post_n = sig->post_n;
        p.sig_post_value = sig->post_value;
        for (int i = 0; i < sig->post_n; ++i) p.sig_post[i] = sig->post[i];
        p.sig_counter = sig->counter;
        p.sig_done = sig->done_flag;
        p.sig_done_value = sig->done_value;
    }
    const bool head_major = use_ext && p.col_interleave == COL_HEAD_MAJOR;
    if (head_major && p.col_combine && p.NQB == 2)
        e = (DK == 64) ? launch_stream<64, MODE_COLSUM_EXT_SHORT2_COMBINE>(tk_a, tq_b, text, p, grid2, stream, chained)
                      : launch_stream<128, MODE_COLSUM_EXT_SHORT2_COMBINE>(tk_a, tq_b, text, p, grid2, stream, chained);
    else if (head_major && p.col_combine)
        e = (DK == 64) ? launch_stream<64, MODE_COLSUM_EXT_SHORT_COMBINE>(tk_a, tq_b, text, p, grid2, stream, chained)
                      : launch_stream<128, MODE_COLSUM_EXT_SHORT_COMBINE>(tk_a, tq_b, text, p, grid2, stream, chained);
    else if (head_major && p.NQB == 2)   // two resident query blocks per head
        e = (DK == 64) ? launch_stream<64, MODE_COLSUM_EXT_SHORT2>(tk_a, tq_b, text, p, grid2, stream, chained)
                      : launch_stream<128, MODE_COLSUM_EXT_SHORT2>(tk_a, tq_b, text, p, grid2, stream, chained);
    else if (head_major)   // one query block per head, many key tiles: the key tiles stream
        e = (DK == 64) ? launch_stream<64, MODE_COLSUM_EXT_SHORT>(tk_a, tq_b, text, p, grid2, stream, chained)
                      : launch_stream<128, MODE_COLSUM_EXT_SHORT>(tk_a, tq_b, text, p, grid2, stream, chained);
    else if (use_ext)
        e = (DK == 64) ? launch_stream<64, MODE_COLSUM_EXT>(tk_a, tq_b, text, p, grid2, stream, chained)
                      : launch_stream<128, MODE_COLSUM_EXT>(tk_a, tq_b, text, p, grid2, stream, chained);
    else
        e = (DK == 64) ? launch_stream<64, MODE_COLSUM>(tk_a, tq_b, text, p, grid2, stream, chained)
                      : launch_stream<128, MODE_COLSUM>(tk_a, tq_b, text, p, grid2, stream, chained);
    if (e != cudaSuccess) return fail(FCS_ERR_CUDA, "column pass launch failed: %s", cudaGetErrorString(e));
    if (tm) { cudaEventRecord(tm->ev[3], stream); tm->recorded = true; }
    return FCS_OK;
}

// ---------------------------------------------------------------------------
// Built-in scratch for callers that have no device allocator to draw from.
// One copy lives in every device that loads this library, for the life of the
// process.  The name below is a host-side handle in host code, not a device
// address: the address is looked up per device with cudaGetSymbolAddress.
// ---------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_static_scratch[FCS_STATIC_SCRATCH_BYTES];

static int static_scratch_address(void** out_ptr) {
    static void* cached[64] = {nullptr};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(FCS_ERR_CUDA, "cudaGetDevice failed: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= 64) return fail(FCS_ERR_UNSUPPORTED, "device ordinal %d is out of range", dev);
    if (!cached[dev]) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess || !ptr)
            return fail(FCS_ERR_CUDA, "cudaGetSymbolAddress(static scratch) failed: %s", cudaGetErrorString(e));
        cached[dev] = ptr;
    }
    *out_ptr = cached[dev];
    return FCS_OK;
}

}  // namespace fcs

// ---------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------
extern "C" {

int fcs_version(void) { return 202; }

const char* fcs_last_error(void) { return fcs::g_err; }

int fcs_set_profiling(int enabled) {
    fcs::g_profiling = enabled != 0;
    return FCS_OK;
}

int fcs_set_single_pass(int mode) {
    if (mode < 0 || mode > 2) return FCS_ERR_INVALID_ARGUMENT;
    fcs::g_single_pass = mode;
    return FCS_OK;
}

int fcs_set_short_fused(int mode) {
    if (mode < 0 || mode > 2) return FCS_ERR_INVALID_ARGUMENT;
    fcs::g_short_fused = mode;
    return FCS_OK;
}

int fcs_short_fused_applies(int B, int H, int sq_rows, int Sk, int D, int is_causal, int k_past, int* cluster_size,
                            int* blocks_per_cta) {
    if (B <= 0 || H <= 0 || sq_rows <= 0 || Sk <= 0 || !fcs::head_dim_ok(D)) return 0;
    int cl = 0, nkb = 0, bpc = 0;
    if (!fcs::short_fused_applies(B, H, sq_rows, Sk, D, is_causal ? 1 : 0, k_past, &cl, &nkb, &bpc)) return 0;
    if (cluster_size) *cluster_size = cl;
    if (blocks_per_cta) *blocks_per_cta = bpc;
    return 1;
}

int fcs_single_pass_applies(int B, int H, int sq_rows, int Sk, int D, int is_causal) {
    if (B <= 0 || H <= 0 || sq_rows <= 0 || Sk <= 0) return 0;
    return fcs::single_pass_applies(B, H, sq_rows, Sk, D, is_causal ? 1 : 0) ? 1 : 0;
}

int fcs_single_pass_info(int Sk, int* cluster_size, int* max_clusters) {
    if (Sk <= 0 || Sk > 256 * fcs::sp::MAX_CL) return FCS_ERR_UNSUPPORTED;
    const int cl = fcs::single_pass_cluster_size(Sk);
    if (cluster_size) *cluster_size = cl;
    if (max_clusters) *max_clusters = fcs::single_pass_max_clusters(cl);
    return FCS_OK;
}

int fcs_last_pass_ms(float* stats_ms, float* merge_ms, float* colsum_ms) {
    fcs::g_err[0] = 0;
    fcs::PassTimers* tm = fcs::timers_for_current_device();
    if (!tm || !tm->recorded)
        return fcs::fail(FCS_ERR_INVALID_ARGUMENT, "no profiled call has been made on this device");
    cudaError_t e = cudaEventSynchronize(tm->ev[3]);
    if (e != cudaSuccess) return fcs::fail(FCS_ERR_CUDA, "event synchronize failed: %s", cudaGetErrorString(e));
    float a = 0.f, b = 0.f, c = 0.f;
    cudaEventElapsedTime(&a, tm->ev[0], tm->ev[1]);
    cudaEventElapsedTime(&b, tm->ev[1], tm->ev[2]);
    cudaEventElapsedTime(&c, tm->ev[2], tm->ev[3]);
    if (stats_ms) *stats_ms = a;
    if (merge_ms) *merge_ms = b;
    if (colsum_ms) *colsum_ms = c;
    return FCS_OK;
}

int fcs_plan_info(int B, int H, int sq_rows, int Sk, int is_causal, int* nsplit, long long* stats_items,
                  long long* colsum_steps, int* sms) {
    if (B <= 0 || H <= 0 || sq_rows <= 0 || Sk <= 0) return FCS_ERR_INVALID_ARGUMENT;
    fcs::Problem p;
    memset(&p, 0, sizeof(p));
    const int k_past = Sk > sq_rows ? Sk - sq_rows : 0;
    const int n_sm = fcs::num_sms();
    fcs::plan(p, B, H, sq_rows, Sk, is_causal ? 1 : 0, k_past, n_sm);
    if (nsplit) *nsplit = p.nsplit;
    if (stats_items) *stats_items = p.stats_items;
    if (colsum_steps) *colsum_steps = p.steps_total;
    if (sms) *sms = n_sm;
    return FCS_OK;
}

size_t fcs_workspace_bytes(int B, int H, int sq_rows, int Sk, int D, int is_causal) {
    if (B <= 0 || H <= 0 || sq_rows <= 0 || Sk <= 0 || !fcs::head_dim_ok(D)) return 0;
    // An upper bound for every k_past and every kernel choice: the layout of the two streaming
    // passes with the key range of the statistics pass split as far as any k_past allows (the
    // split grows with the keys the first query tile sees, and k_past = Sk shows it all of them).
    fcs::Problem p;
    memset(&p, 0, sizeof(p));
    fcs::plan(p, B, H, sq_rows, Sk, is_causal ? 1 : 0, is_causal ? Sk : 0, fcs::num_sms());
    return fcs::workspace_layout(p, nullptr);
}

int fcs_call_workspace_bytes(int B, int H, int sq_rows, int Sk, int D, int is_causal, int k_past,
                             size_t* bytes) {
    fcs::g_err[0] = 0;
    if (!bytes) return fcs::fail(FCS_ERR_INVALID_ARGUMENT, "bytes is NULL");
    *bytes = 0;
    if (B <= 0 || H <= 0 || sq_rows <= 0 || Sk <= 0)
        return fcs::fail(FCS_ERR_INVALID_ARGUMENT, "sizes must be positive (B=%d H=%d Sq=%d Sk=%d)", B, H, sq_rows, Sk);
    if (!fcs::head_dim_ok(D))
        return fcs::fail(FCS_ERR_UNSUPPORTED, "head dimension must be a multiple of 8 from 8 to 128, got %d", D);
    const int causal = is_causal ? 1 : 0;
    // the same decisions, in the same order, as the call itself
    if (fcs::smallq_fits(sq_rows, Sk, D, B * H, fcs::num_sms()))
        return FCS_OK;   // few-row kernel: no scratch
    if (fcs::single_pass_applies(B, H, sq_rows, Sk, D, causal) &&
        fcs::single_pass_max_clusters(fcs::single_pass_cluster_size(Sk)) > 0)
        return FCS_OK;   // single-pass kernel: no scratch
    if (causal && k_past < 0) k_past = Sk > sq_rows ? Sk - sq_rows : 0;
    if (fcs::short_fused_applies(B, H, sq_rows, Sk, D, causal, k_past, nullptr, nullptr, nullptr))
        return FCS_OK;   // one-kernel short form: no scratch
    fcs::Problem p;
    memset(&p, 0, sizeof(p));
    fcs::plan(p, B, H, sq_rows, Sk, causal, causal ? k_past : 0, fcs::num_sms());
    *bytes = fcs::workspace_layout(p, nullptr);
    return FCS_OK;
}

int fcs_colsum_batched(const void* q, const void* k, float* out, int64_t out_ld, int B, int H, int S, int D,
                       int dtype, int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
                       int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_s, float scale, int cls_n,
                       int h_norm, void* workspace, size_t workspace_bytes, int* status, void* stream) {
    return fcs::colsum_impl(q, k, out, out_ld, B, H, S, S, D, dtype, q_stride_b, q_stride_h, q_stride_s,
                            k_stride_b, k_stride_h, k_stride_s, scale, 0, 0, cls_n, h_norm, workspace,
                            workspace_bytes, status, stream);
}

int fcs_colsum_non_batched(const void* q, const void* k, float* out, int H, int S, int D, int dtype,
                           int64_t q_stride_h, int64_t q_stride_s, int64_t k_stride_h, int64_t k_stride_s,
                           float scale, int cls_n, int h_norm, void* workspace, size_t workspace_bytes,
                           int* status, void* stream) {
    return fcs::colsum_impl(q, k, out, S, 1, H, S, S, D, dtype, q_stride_h * H, q_stride_h, q_stride_s,
                            k_stride_h * H, k_stride_h, k_stride_s, scale, 0, 0, cls_n, h_norm, workspace,
                            workspace_bytes, status, stream);
}

int fcs_colsum_causal(const void* q, const void* k, float* out, int H, int q_len, int k_len, int D, int dtype,
                      int64_t q_stride_h, int64_t q_stride_s, int64_t k_stride_h, int64_t k_stride_s,
                      float scale, int k_past, int h_norm, void* workspace, size_t workspace_bytes,
                      int* status, void* stream) {
    return fcs::colsum_impl(q, k, out, k_len, 1, H, q_len, k_len, D, dtype, q_stride_h * H, q_stride_h,
                            q_stride_s, k_stride_h * H, k_stride_h, k_stride_s, scale, 1, k_past, -1, h_norm,
                            workspace, workspace_bytes, status, stream);
}

int fcs_colsum_causal_batched(const void* q, const void* k, float* out, int64_t out_ld, int B, int H, int q_len,
                              int k_len, int D, int dtype, int64_t q_stride_b, int64_t q_stride_h,
                              int64_t q_stride_s, int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_s,
                              float scale, int k_past, int h_norm, void* workspace, size_t workspace_bytes,
                              int* status, void* stream) {
    return fcs::colsum_impl(q, k, out, out_ld, B, H, q_len, k_len, D, dtype, q_stride_b, q_stride_h, q_stride_s,
                            k_stride_b, k_stride_h, k_stride_s, scale, 1, k_past, -1, h_norm, workspace,
                            workspace_bytes, status, stream);
}

size_t fcs_statistics_rows(int q_rows) {
    return q_rows > 0 ? (size_t)fcs::ceil_div(q_rows, fcs::BLOCK) * fcs::BLOCK : 0;
}

int fcs_colsum_statistics(const void* q, const void* k, float* neg_lse, int B, int H, int q_rows, int Sk, int D,
                          int dtype, int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
                          int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_s, float scale,
                          int64_t norm_rows, int h_norm, void* workspace, size_t workspace_bytes, int* status,
                          void* stream) {
    if (norm_rows < q_rows) {
        fcs::g_err[0] = 0;
        return fcs::fail(FCS_ERR_INVALID_ARGUMENT, "norm_rows (%lld) is smaller than the rows given (%d)",
                         (long long)norm_rows, q_rows);
    }
    return fcs::colsum_impl(q, k, nullptr, 0, B, H, q_rows, Sk, D, dtype, q_stride_b, q_stride_h, q_stride_s,
                            k_stride_b, k_stride_h, k_stride_s, scale, 0, 0, -1, h_norm, workspace,
                            workspace_bytes, status, stream, false, fcs::PASSES_STATS, neg_lse, norm_rows);
}

int fcs_colsum_columns(const void* q, const void* k, const float* neg_lse, float* out, int64_t out_ld, int B, int H,
                       int q_rows, int k_rows, int D, int dtype, int64_t q_stride_b, int64_t q_stride_h,
                       int64_t q_stride_s, int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_s,
                       float scale, void* workspace, size_t workspace_bytes, int* status, void* stream) {
    return fcs::colsum_impl(q, k, out, out_ld, B, H, q_rows, k_rows, D, dtype, q_stride_b, q_stride_h, q_stride_s,
                            k_stride_b, k_stride_h, k_stride_s, scale, 0, 0, -1, 0, workspace, workspace_bytes,
                            status, stream, true, fcs::PASSES_COLUMNS, const_cast<float*>(neg_lse), 0);
}

int fcs_select_topk(const float* colsum, int64_t ld, int B, int S, int k, int* indices, float* values,
                    void* stream) {
    fcs::g_err[0] = 0;
    if (!colsum || !indices) return fcs::fail(FCS_ERR_INVALID_ARGUMENT, "colsum and indices must not be NULL");
    if (B <= 0 || S <= 0 || ld < S)
        return fcs::fail(FCS_ERR_INVALID_ARGUMENT, "bad sizes (B=%d S=%d ld=%lld)", B, S, (long long)ld);
    if (k <= 0 || k > S) return fcs::fail(FCS_ERR_INVALID_ARGUMENT, "k must be in 1..S, got %d (S=%d)", k, S);
    fcs::select_topk_kernel<<<B, fcs::TOPK_THREADS, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        colsum, (long long)ld, S, k, indices, values);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fcs::fail(FCS_ERR_CUDA, "top-k selection launch failed: %s", cudaGetErrorString(e));
    return FCS_OK;
}

int fcs_peer_post(int* const* flags, int n_flags, int value, void* stream) {
    fcs::g_err[0] = 0;
    if (!flags || n_flags <= 0 || n_flags > fcs::PEER_FLAGS_MAX)
        return fcs::fail(FCS_ERR_INVALID_ARGUMENT, "1 to %d flag pointers are expected, got %d", fcs::PEER_FLAGS_MAX, n_flags);
    fcs::PeerFlagPointers fp;
    memset(&fp, 0, sizeof(fp));
    for (int i = 0; i < n_flags; ++i) {
        if (!flags[i] || reinterpret_cast<uintptr_t>(flags[i]) % 4)
            return fcs::fail(FCS_ERR_INVALID_ARGUMENT, "flag %d is NULL or misaligned", i);
        fp.p[i] = flags[i];
    }
    fcs::peer_post_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(fp, n_flags, value);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fcs::fail(FCS_ERR_CUDA, "flag post launch failed: %s", cudaGetErrorString(e));
    return FCS_OK;
}

int fcs_peer_wait(const int* flags, int n_flags, int value, int* status, void* stream) {
    fcs::g_err[0] = 0;
    if (!flags || n_flags <= 0 || n_flags > 32 || reinterpret_cast<uintptr_t>(flags) % 4)
        return fcs::fail(FCS_ERR_INVALID_ARGUMENT, "1 to 32 consecutive, aligned flags are expected, got %d", n_flags);
    fcs::peer_wait_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(flags, n_flags, value, status);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fcs::fail(FCS_ERR_CUDA, "flag wait launch failed: %s", cudaGetErrorString(e));
    return FCS_OK;
}

int fcs_selftest_wait_expiry(const void* q, const void* k, void* workspace, size_t workspace_bytes, int* status,
                              double limit_seconds, void* stream_v) {
    fcs::g_err[0] = 0;
    using namespace fcs;
    if (!q || !k || !workspace || !status)
        return fail(FCS_ERR_INVALID_ARGUMENT, "q, k, workspace and status must not be NULL");
    if (!(limit_seconds > 0.0) || limit_seconds > 2.0)
        return fail(FCS_ERR_INVALID_ARGUMENT, "limit_seconds must be in (0, 2]");
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
    // a statistics pass over one 128 x 256 tile of fp16 inputs with D = 64
    const int B = 1, H = 1, Sq = TILE, Sk = BLOCK, D = 64;
    Problem p;
    memset(&p, 0, sizeof(p));
    plan(p, B, H, Sq, Sk, 0, 0, num_sms());
    size_t part_off = 0, ext_off = 0;
    const size_t need = workspace_layout(p, &part_off, &ext_off);
    if (workspace_bytes < need || reinterpret_cast<uintptr_t>(workspace) % 256)
        return fail(FCS_ERR_WORKSPACE, "workspace too small or misaligned: need %zu bytes", need);
    p.neg_lse = reinterpret_cast<float*>(workspace);
    p.part = reinterpret_cast<uint8_t*>(workspace) + part_off;
    p.ext = reinterpret_cast<uint8_t*>(workspace) + ext_off;
    p.status = status;
    p.c = 0.125f * 1.4426950408889634f;
    p.inv_c = 1.0f / p.c;
    p.log2_norm = log2f((float)Sq);
    p.idesc = (1u << 4) | ((uint32_t)(BLOCK >> 3) << 17) | ((uint32_t)(TILE >> 4) << 24);
    p.withhold_loads = 1;
    CUtensorMap tq, tk;
    int rc;
    if ((rc = make_tensor_map(&tq, q, FCS_DTYPE_FP16, B, H, Sq, D, (int64_t)Sq * D, (int64_t)Sq * D, D, TILE)) != FCS_OK) return rc;
    if ((rc = make_tensor_map(&tk, k, FCS_DTYPE_FP16, B, H, Sk, D, (int64_t)Sk * D, (int64_t)Sk * D, D, BLOCK)) != FCS_OK) return rc;
    static long long short_limit, full_limit = kWaitLimitCycles;
    short_limit = (long long)(limit_seconds * 1.9e9);
    cudaError_t e = cudaMemcpyToSymbolAsync(g_wait_limit_cycles, &short_limit, sizeof(long long), 0,
                                            cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess) e = launch_stream<64, MODE_STATS>(tq, tk, tq, p, 1, stream, false);
    const cudaError_t e2 = cudaMemcpyToSymbolAsync(g_wait_limit_cycles, &full_limit, sizeof(long long), 0,
                                                   cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess || e2 != cudaSuccess)
        return fail(FCS_ERR_CUDA, "wait-expiry self-test failed to launch: %s",
                    cudaGetErrorString(e != cudaSuccess ? e : e2));
    return FCS_OK;
}

int fcs_selftest_wait_expiry_cluster(const void* q, const void* k, float* out, int* status, double limit_seconds,
                                     void* stream_v) {
    fcs::g_err[0] = 0;
    using namespace fcs;
    if (!q || !k || !out || !status)
        return fail(FCS_ERR_INVALID_ARGUMENT, "q, k, out and status must not be NULL");
    if (!(limit_seconds > 0.0) || limit_seconds > 2.0)
        return fail(FCS_ERR_INVALID_ARGUMENT, "limit_seconds must be in (0, 2]");
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
    // the one-kernel form on one head: 128 queries, two blocks of 256 keys, a cluster of two CTAs
    const int B = 1, H = 1, Sq = TILE, Sk = 2 * BLOCK, D = 64;
    Problem p;
    memset(&p, 0, sizeof(p));
    p.B = B; p.H = H; p.Sq = Sq; p.Sk = Sk;
    p.out = out;
    p.out_ld = Sk;
    p.status = status;
    p.c = 0.125f * 1.4426950408889634f;
    p.inv_c = 1.0f / p.c;
    p.log2_norm = log2f((float)Sq);
    p.withhold_loads = 1;
    CUtensorMap tq, tk;
    int rc;
    if ((rc = make_tensor_map(&tq, q, FCS_DTYPE_FP16, B, H, Sq, D, (int64_t)Sq * D, (int64_t)Sq * D, D, TILE)) != FCS_OK) return rc;
    if ((rc = make_tensor_map(&tk, k, FCS_DTYPE_FP16, B, H, Sk, D, (int64_t)Sk * D, (int64_t)Sk * D, D, BLOCK)) != FCS_OK) return rc;
    static long long short_limit, full_limit = kWaitLimitCycles;
    short_limit = (long long)(limit_seconds * 1.9e9);
    cudaError_t e = cudaMemcpyToSymbolAsync(g_wait_limit_cycles, &short_limit, sizeof(long long), 0,
                                            cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess)
        rc = launch_fused_short(tq, tk, p, 64, 0.125f, true, /*cl=*/2, /*nkb=*/2, /*bpc=*/1, /*clear_out=*/true, nullptr, 0,
                                stream);
    const cudaError_t e2 = cudaMemcpyToSymbolAsync(g_wait_limit_cycles, &full_limit, sizeof(long long), 0,
                                                   cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess || e2 != cudaSuccess)
        return fail(FCS_ERR_CUDA, "wait-expiry self-test failed to launch: %s",
                    cudaGetErrorString(e != cudaSuccess ? e : e2));
    return rc;
}

int fcs_select_threshold(const float* colsum, int64_t ld, int B, int S, float threshold, int relative, int* indices,
                         int* counts, void* stream) {
    fcs::g_err[0] = 0;
    if (!colsum || !indices || !counts)
        return fcs::fail(FCS_ERR_INVALID_ARGUMENT, "colsum, indices and counts must not be NULL");
    if (B <= 0 || S <= 0 || ld < S)
        return fcs::fail(FCS_ERR_INVALID_ARGUMENT, "bad sizes (B=%d S=%d ld=%lld)", B, S, (long long)ld);
    if (!(threshold == threshold)) return fcs::fail(FCS_ERR_INVALID_ARGUMENT, "threshold is not a number");
    fcs::select_threshold_kernel<<<B, fcs::TOPK_THREADS, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        colsum, (long long)ld, S, threshold, relative ? 1 : 0, indices, counts);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fcs::fail(FCS_ERR_CUDA, "threshold selection launch failed: %s", cudaGetErrorString(e));
    return FCS_OK;
}

int fcs_colsum_batched_static_scratch(const void* q, const void* k, float* out, int64_t out_ld, int B, int H,
                                      int S, int D, int dtype, int64_t q_stride_b, int64_t q_stride_h,
                                      int64_t q_stride_s, int64_t k_stride_b, int64_t k_stride_h,
                                      int64_t k_stride_s, float scale, int cls_n, int h_norm, int* status,
                                      void* stream) {
    fcs::g_err[0] = 0;
    if (B <= 0 || H <= 0 || S <= 0 || !fcs::head_dim_ok(D))
        return fcs::fail(FCS_ERR_INVALID_ARGUMENT, "bad sizes (B=%d H=%d S=%d D=%d)", B, H, S, D);
    const int rows = (cls_n > 0 && cls_n < S) ? cls_n : S;
    // what this call will really use: nothing when it takes the few-row or the single-pass kernel
    size_t need = 0;
    const int qrc = fcs_call_workspace_bytes(B, H, rows, S, D, 0, 0, &need);
    if (qrc != FCS_OK) return qrc;
    if (need > (size_t)FCS_STATIC_SCRATCH_BYTES)
        return fcs::fail(FCS_ERR_WORKSPACE,
                         "this call needs %zu bytes of scratch but the built-in scratch holds %zu; "
                         "use fcs_colsum_batched with a caller-provided workspace",
                         need, (size_t)FCS_STATIC_SCRATCH_BYTES);
    void* scratch = nullptr;
    const int rc = fcs::static_scratch_address(&scratch);
    if (rc != FCS_OK) return rc;
    return fcs::colsum_impl(q, k, out, out_ld, B, H, S, S, D, dtype, q_stride_b, q_stride_h, q_stride_s,
                            k_stride_b, k_stride_h, k_stride_s, scale, 0, 0, cls_n, h_norm, scratch,
                            (size_t)FCS_STATIC_SCRATCH_BYTES, status, stream);
}

int fcs_colsum_causal_accumulate(const void* q, const void* k, float* out, int H, int q_len, int k_len, int D,
                                 int dtype, int64_t q_stride_h, int64_t q_stride_s, int64_t k_stride_h,
                                 int64_t k_stride_s, float scale, int k_past, int h_norm, void* workspace,
                                 size_t workspace_bytes, int* status, void* stream) {
    return fcs::colsum_impl(q, k, out, k_len, 1, H, q_len, k_len, D, dtype, q_stride_h * H, q_stride_h,
                            q_stride_s, k_stride_h * H, k_stride_h, k_stride_s, scale, 1, k_past, -1, h_norm,
                            workspace, workspace_bytes, status, stream, /*clear_out=*/false);
}

int fcs_colsum_causal_accumulate_and_clear(const void* q, const void* k, float* out, float* clear_buf, int H,
                                           int q_len, int k_len, int D, int dtype, int64_t q_stride_h,
                                           int64_t q_stride_s, int64_t k_stride_h, int64_t k_stride_s, float scale,
                                           int k_past, int h_norm, void* workspace, size_t workspace_bytes,
                                           int* status, void* stream) {
    return fcs::colsum_impl(q, k, out, k_len, 1, H, q_len, k_len, D, dtype, q_stride_h * H, q_stride_h,
                            q_stride_s, k_stride_h * H, k_stride_h, k_stride_s, scale, 1, k_past, -1, h_norm,
                            workspace, workspace_bytes, status, stream, /*clear_out=*/false, fcs::PASSES_BOTH, nullptr,
                            0, clear_buf, clear_buf ? (long long)k_len : 0);
}

int fcs_colsum_causal_accumulate_signalled(const void* q, const void* k, float* out, float* clear_buf, int H,
                                           int q_len, int k_len, int D, int dtype, int64_t q_stride_h,
                                           int64_t q_stride_s, int64_t k_stride_h, int64_t k_stride_s, float scale,
                                           int k_past, int h_norm, void* workspace, size_t workspace_bytes,
                                           int* status, void* stream, const FcsPeerSignals* signals) {
    fcs::g_err[0] = 0;
    if (!signals) return fcs::fail(FCS_ERR_INVALID_ARGUMENT, "signals is NULL");
    if (signals->post_n < 0 || signals->post_n > 15)
        return fcs::fail(FCS_ERR_INVALID_ARGUMENT, "at most 15 flags can be posted, got %d", signals->post_n);
    if (signals->done_flag && !signals->counter)
        return fcs::fail(FCS_ERR_INVALID_ARGUMENT, "a done flag needs a counter");
    return fcs::colsum_impl(q, k, out, k_len, 1, H, q_len, k_len, D, dtype, q_stride_h * H, q_stride_h,
                            q_stride_s, k_stride_h * H, k_stride_h, k_stride_s, scale, 1, k_past, -1, h_norm,
                            workspace, workspace_bytes, status, stream, /*clear_out=*/false, fcs::PASSES_BOTH, nullptr,
                            0, clear_buf, clear_buf ? (long long)k_len : 0, signals);
}

}  // extern "C"
