// Attention column mean of a short query axis (at most 128 rows: the causal query
// suffix of a prompt, a long CLS prefix) in one kernel instead of the statistics
// kernel, the merge kernel and the column kernel.  Over a few thousand keys such a
// call takes tens of microseconds and was bound by its three launches, each with its
// own ramp (barriers, tensor memory, first tiles) and drain; which calls take this
// form is decided by fused_short_plan (schedule.h).
//
// One thread-block cluster per (batch, head); CTA r of the cluster owns the r-th run
// of 256-key blocks.  The head's query block is loaded once and serves both phases:
//
//   phase 1  S   = Q K_blk^T   128 queries x 256 keys per step, tensor-memory lane = query:
//                              running (maximum, sum of exp2) per row over the CTA's blocks
//   exchange                   the four consumer groups' values meet in shared memory, the
//                              CTA's (maximum, sum) per row goes to every CTA of the cluster
//                              (st.async counted on the receiver's mbarrier); each CTA then
//                              holds -(log-sum-exp) of all 128 rows and writes it, split into
//                              16-bit parts, into 16 extra contraction columns of the query
//                              block in shared memory (32-byte swizzled rows)
//   phase 2  S^T = K_blk Q^T   two MMAs of 128 keys x 128 queries per block (+ the 16
//                              extra columns, so that the accumulator holds s - lse/c),
//                              tensor-memory lane = key: exp2 summed down the query axis
//                              in the thread, one add per key and consumer group
//
// The key blocks are fetched again for phase 2, last block first: what phase 1 read last is
// what L2 still holds when the call's keys do not all fit it.  The copy warp runs ahead
// across the exchange.  The output is
// cleared by a small kernel in front, of which this kernel is a programmatic dependent:
// it waits for it only before its first add.
//
// Included by flash_colsum_sm100.cu below the streaming kernel, whose consumer-group
// constants and per-tile functions (stats_tile, colsum_tile_ext, colsum_tile) it uses.
#pragma once

namespace fcs {
namespace fused {

constexpr int MAX_CL = FUSED_SHORT_MAX_CLUSTER;   // CTAs per cluster (the portable limit of eight)

struct Params {
    Problem p;              // sizes, mask rule, scale, output (the scratch fields stay unused)
    int CL;                 // CTAs per (batch, head)
    int nkb;                // 256-key blocks that hold a key some row sees
    int blocks_per_cta;
    int use_ext;            // -(lse) rides in the MMA of phase 2 (0: tiny scales, it is applied per element)
    uint32_t idesc_scores;  // 128 x 256 x 16
    uint32_t idesc_cols;    // 128 x 128 x 16
};

template <int D>
struct FLayout {
    static constexpr int SLABS = D / 64;
    static constexpr int Q_SLAB_BYTES = TILE * 128;
    static constexpr int K_SLAB_BYTES = BLOCK * 128;
    static constexpr int Q_BYTES = SLABS * Q_SLAB_BYTES;
    static constexpr int K_BYTES = SLABS * K_SLAB_BYTES;
    static constexpr int NS = 128 * 1024 / K_BYTES;                     // key-block stages: 2 at D = 128, 4 at D = 64
    static constexpr int Q_OFF = 0;
    static constexpr int K_OFF = Q_BYTES;
    static constexpr int EXTA_OFF = K_OFF + NS * K_BYTES;               // key-side constant of the extra columns
    static constexpr int EXTB_OFF = EXTA_OFF + EXT_A_BYTES;             // query-side extra columns, 128 rows
    static constexpr int LSE_OFF = EXTB_OFF + TILE * EXT_ROW_BYTES;     // float[256]: -(lse) per query (tiny scales)
    static constexpr int MERGE_OFF = LSE_OFF + BLOCK * 4;               // float2[groups][128]
    static constexpr int XCH_OFF = MERGE_OFF + CONSUMER_GROUPS * TILE * 8;   // float2[MAX_CL][128]
    static constexpr int BAR_OFF = XCH_OFF + MAX_CL * TILE * 8;
    // q_full, k_full[NS], k_empty[NS], t_full[2], t_empty[2], exchange, ext_ready
    static constexpr int NUM_BARS = 1 + 2 * NS + 2 * NUM_TBUF + 2;
    static constexpr int MISC_OFF = BAR_OFF + NUM_BARS * 8;             // tensor-memory address, abort flag
    static constexpr int TOTAL = MISC_OFF + 16;
    static constexpr int DYN_BYTES = TOTAL + 1024;                      // slack to align the base to 1024
    static_assert(DYN_BYTES <= 227 * 1024, "shared memory budget");
};

template <int D>
__global__ void __launch_bounds__(THREADS, 1)
colsum_fused_short_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                          const Params fp) {
    using L = FLayout<D>;
    const Problem& p = fp.p;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t q_smem = smem_base + L::Q_OFF;
    const uint32_t k_smem = smem_base + L::K_OFF;
    const uint32_t bars = smem_base + L::BAR_OFF;
    const uint32_t q_full = bars;
    auto k_full = [&](int i) { return bars + 8u * (1 + i); };
    auto k_empty = [&](int i) { return bars + 8u * (1 + L::NS + i); };
    auto t_full = [&](int i) { return bars + 8u * (1 + 2 * L::NS + i); };
    auto t_empty = [&](int i) { return bars + 8u * (1 + 2 * L::NS + NUM_TBUF + i); };
    const uint32_t xch_bar = bars + 8u * (1 + 2 * L::NS + 2 * NUM_TBUF);
    const uint32_t ext_ready = xch_bar + 8u;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + L::MISC_OFF);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::MISC_OFF + 4);
    float2* merge_buf = reinterpret_cast<float2*>(smem + L::MERGE_OFF);
    float2* xch = reinterpret_cast<float2*>(smem + L::XCH_OFF);
    float* lse_buf = reinterpret_cast<float*>(smem + L::LSE_OFF);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t cr = smallq_cluster_rank();
    const int unit = (int)smallq_cluster_id();
    const int b = unit / p.H, h = unit % p.H;
    int kb0 = (int)cr * fp.blocks_per_cta;
    if (kb0 > fp.nkb) kb0 = fp.nkb;
    int kb1 = kb0 + fp.blocks_per_cta;
    if (kb1 > fp.nkb) kb1 = fp.nkb;
    const int nblk = kb1 - kb0;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < L::NS; ++i) { mbar_init(k_full(i), 1); mbar_init(k_empty(i), 1); }
        for (int i = 0; i < NUM_TBUF; ++i) { mbar_init(t_full(i), 1); mbar_init(t_empty(i), CONSUMER_THREADS); }
        mbar_init(xch_bar, 1);
        mbar_init(ext_ready, TILE);
        *abort_flag = 0;
        mbar_fence_init();
        // every CTA of the cluster sends its 128 (maximum, sum) pairs here
        mbar_arrive_expect_tx(xch_bar, (uint32_t)fp.CL * TILE * 8);
    }
    {
        // the key-side constant of the extra columns: every 16-byte piece is (k, k, k, 0, 0, 0, 0, 0),
        // which reads the same under any swizzle of the pieces
        const uint32_t k16 = p.ext_bf16 ? 0x3F80u : 0x5C00u;   // bf16 1.0 / fp16 256.0
        uint4* ones = reinterpret_cast<uint4*>(smem + L::EXTA_OFF);
        for (int i = threadIdx.x; i < EXT_A_BYTES / 16; i += THREADS)
            ones[i] = make_uint4(k16 | (k16 << 16), k16, 0u, 0u);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == PRODUCER_WARP && lane == 0) {
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_k);
    }
    if (warp == MMA_WARP) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // every CTA of the cluster has set up its barriers once this completes; it is waited for
    // before the first store into another CTA's shared memory
    smallq_cluster_arrive();

    auto wait_all = [&](uint32_t bar, uint32_t parity, int code) -> bool {
        const bool ok = mbar_wait(bar, parity, abort_flag, p.status, code);
        return __all_sync(0xffffffffu, ok);
    };

    if (warp == PRODUCER_WARP) {
        // -------------------------------------------- copies: the query block, then the key blocks twice
        bool ok = p.withhold_loads == 0;   // (self-test: nothing is loaded, every wait for data runs out)
        if (ok && elect_one_sync()) {
            mbar_arrive_expect_tx(q_full, L::Q_BYTES);
#pragma unroll
            for (int sl = 0; sl < L::SLABS; ++sl)
                tma_load_4d(q_smem + sl * L::Q_SLAB_BYTES, &tm_q, q_full, sl * 64, 0, h, b);
        }
        __syncwarp();
        for (int n = 0; ok && n < 2 * nblk; ++n) {
            const int stage = n % L::NS;
            const int kb = n < nblk ? kb0 + n : kb1 - 1 - (n - nblk);   // phase 2 walks back: the last blocks are the ones still in L2
            if (n >= L::NS && !wait_all(k_empty(stage), ((n / L::NS) & 1) ^ 1, FCS_STATUS_WAIT_PRODUCER)) break;
            if (elect_one_sync()) {
                mbar_arrive_expect_tx(k_full(stage), L::K_BYTES);
#pragma unroll
                for (int sl = 0; sl < L::SLABS; ++sl)
                    tma_load_4d(k_smem + stage * L::K_BYTES + sl * L::K_SLAB_BYTES, &tm_k, k_full(stage), sl * 64,
                                kb * BLOCK, h, b);
            }
            __syncwarp();
        }
        smallq_cluster_wait();      // (pairs with the arrive above; this warp stores nothing into other CTAs)
    } else if (warp == MMA_WARP) {
        // -------------------------------------------- MMA issuer
        bool ok = wait_all(q_full, 0, FCS_STATUS_WAIT_MMA);
        const uint64_t dq = umma_desc_k_sw128(q_smem);
        int n = 0;
        for (; ok && n < nblk; ++n) {          // phase 1: queries x 256 keys
            const int stage = n % L::NS, buf = n & (NUM_TBUF - 1);
            if (!wait_all(k_full(stage), (n / L::NS) & 1, FCS_STATUS_WAIT_MMA)) { ok = false; break; }
            if (n >= NUM_TBUF && !wait_all(t_empty(buf), ((n >> 1) & 1) ^ 1, FCS_STATUS_WAIT_MMA)) { ok = false; break; }
            tc_fence_after();
            const uint64_t dk = umma_desc_k_sw128(k_smem + stage * L::K_BYTES);
            const uint32_t d_tmem = tmem_base + buf * BLOCK;
            if (elect_one_sync()) {
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint64_t oq = (uint64_t)(((ks >> 2) * L::Q_SLAB_BYTES + (ks & 3) * 32) >> 4);
                    const uint64_t ok_ = (uint64_t)(((ks >> 2) * L::K_SLAB_BYTES + (ks & 3) * 32) >> 4);
                    umma_f16(d_tmem, dq + oq, dk + ok_, fp.idesc_scores, ks > 0 ? 1u : 0u);
                }
                umma_commit(k_empty(stage));
                umma_commit(t_full(buf));
            }
            __syncwarp();
        }
        smallq_cluster_wait();      // (pairs with the arrive above)
        // phase 2: two tiles of 128 keys x 128 queries per block.  The score MMAs of the first two
        // blocks do not need the statistics: they are issued while the exchange is under way, and only
        // the MMAs of the extra columns (and the hand-over to the consumers) wait for it.
        auto score_mmas = [&](int stage, int buf) {
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                // rows 128 t .. 128 t + 127 of the block: 16 KiB into each 32 KiB slab
                const uint64_t dk = umma_desc_k_sw128(k_smem + stage * L::K_BYTES + t * (TILE * 128));
                const uint32_t d_tmem = tmem_base + buf * BLOCK + t * (BLOCK / 2);
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint64_t oq = (uint64_t)(((ks >> 2) * L::Q_SLAB_BYTES + (ks & 3) * 32) >> 4);
                    const uint64_t ok_ = (uint64_t)(((ks >> 2) * L::K_SLAB_BYTES + (ks & 3) * 32) >> 4);
                    umma_f16(d_tmem, dk + ok_, dq + oq, fp.idesc_cols, ks > 0 ? 1u : 0u);
                }
            }
        };
        auto extra_mmas = [&](int buf) {
            if (!fp.use_ext) return;
#pragma unroll
            for (int t = 0; t < 2; ++t)
                umma_f16(tmem_base + buf * BLOCK + t * (BLOCK / 2), umma_desc_k_sw32(smem_base + L::EXTA_OFF),
                         umma_desc_k_sw32(smem_base + L::EXTB_OFF), fp.idesc_cols, 1u);
        };
        const int early = nblk < NUM_TBUF ? nblk : NUM_TBUF;
        for (int e = 0; ok && e < early; ++e) {
            const int m = n + e, stage = m % L::NS, buf = m & (NUM_TBUF - 1);
            if (!wait_all(k_full(stage), (m / L::NS) & 1, FCS_STATUS_WAIT_MMA)) { ok = false; break; }
            if (m >= NUM_TBUF && !wait_all(t_empty(buf), ((m >> 1) & 1) ^ 1, FCS_STATUS_WAIT_MMA)) { ok = false; break; }
            tc_fence_after();
            if (elect_one_sync()) {
                score_mmas(stage, buf);
                umma_commit(k_empty(stage));
            }
            __syncwarp();
        }
        // the extra columns of the query block are in shared memory
        if (ok) ok = wait_all(ext_ready, 0, FCS_STATUS_WAIT_MMA);
        tc_fence_after();
        for (int e = 0; ok && e < early; ++e, ++n) {
            const int buf = n & (NUM_TBUF - 1);
            if (elect_one_sync()) {
                extra_mmas(buf);
                umma_commit(t_full(buf));
            }
            __syncwarp();
        }
        for (; ok && n < 2 * nblk; ++n) {
            const int stage = n % L::NS, buf = n & (NUM_TBUF - 1);
            if (!wait_all(k_full(stage), (n / L::NS) & 1, FCS_STATUS_WAIT_MMA)) { ok = false; break; }
            if (n >= NUM_TBUF && !wait_all(t_empty(buf), ((n >> 1) & 1) ^ 1, FCS_STATUS_WAIT_MMA)) { ok = false; break; }
            tc_fence_after();
            if (elect_one_sync()) {
                score_mmas(stage, buf);
                extra_mmas(buf);
                umma_commit(k_empty(stage));
                umma_commit(t_full(buf));
            }
            __syncwarp();
        }
    } else {
        // ------------------------------------------------ consumers
        const int wg = warp >> 2;                  // consumer group
        const int col0 = wg * GROUP_COLS;          // its first column of every accumulator
        const int row = ((warp & 3) << 5) | lane;  // tensor-memory lane of this thread
        const uint32_t lane_addr = tmem_base + ((uint32_t)((warp & 3) << 5) << 16) + col0;
        const float c = p.c;
        // A wait that runs out raises the abort flag (later waits give up at once) but does not end
        // the flow: all consumer warps keep meeting at the named barrier, the results are void and
        // the status word says so.
        bool ok = true;
        int n = 0;

        // phase 1: running (maximum, sum) of this thread's query row over the group's columns
        float m_run = -INFINITY, l_run = 0.f;
        int f_lo, f_hi;
        stats_full_range(p, 0, f_lo, f_hi);
        for (int i = 0; i < nblk; ++i, ++n) {
            const int kb = kb0 + i, buf = n & (NUM_TBUF - 1);
            ok = ok && mbar_wait(t_full(buf), (n >> 1) & 1, abort_flag, p.status, FCS_STATUS_WAIT_CONSUMER);
            ok = __all_sync(0xffffffffu, ok);
            tc_fence_after();
            const uint32_t taddr = lane_addr + buf * BLOCK;
            if (ok) {
                if (kb >= f_lo && kb < f_hi) {
                    stats_tile<false>(taddr, GROUP_COLS, c, m_run, l_run);
                } else {
                    const int lim = stats_last_visible(p, 0, kb, row) - col0;
                    const int lim_last_row = stats_last_visible(p, 0, kb, TILE - 1) - col0;
                    if (lim_last_row >= 0) stats_tile<true>(taddr, lim, c, m_run, l_run);
                }
            }
            tc_fence_before();
            mbar_arrive(t_empty(buf));
        }
        merge_buf[wg * TILE + row] = make_float2(m_run, l_run);
        asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_THREADS) : "memory");
        smallq_cluster_wait();      // the other CTAs' barriers are set up
        if (wg == 0) {
            float mm = -INFINITY;
#pragma unroll
            for (int g = 0; g < CONSUMER_GROUPS; ++g) mm = fmaxf(mm, merge_buf[g * TILE + row].x);
            const float ms = (mm == -INFINITY) ? 0.f : mm;
            float ll = 0.f;
#pragma unroll
            for (int g = 0; g < CONSUMER_GROUPS; ++g) {
                const float2 o = merge_buf[g * TILE + row];
                ll += o.y * exp2f(o.x - ms);
            }
            const uint32_t slot = smem_u32(xch + (size_t)cr * TILE + row);
            for (int d = 0; d < fp.CL; ++d) smallq_post(slot, xch_bar, (uint32_t)d, mm, ll);
        }
        ok = ok && mbar_wait(xch_bar, 0, abort_flag, p.status, FCS_STATUS_WAIT_CONSUMER);
        ok = __all_sync(0xffffffffu, ok);
        if (wg == 0) {
            // -(log-sum-exp) of this query row over the whole key axis, in the form phase 2 takes
            float mm = -INFINITY;
            for (int i = 0; i < fp.CL; ++i) mm = fmaxf(mm, xch[i * TILE + row].x);
            const float ms = (mm == -INFINITY) ? 0.f : mm;
            float ll = 0.f;
            for (int i = 0; i < fp.CL; ++i) {
                const float2 o = xch[i * TILE + row];
                ll += o.y * exp2f(o.x - ms);
            }
            const float nlv = (ok && row < p.Sq) ? -(mm + log2f(ll) + p.log2_norm) : -INFINITY;
            lse_buf[row] = nlv;
            lse_buf[TILE + row] = -INFINITY;
            uint4 e0, e1;
            make_ext_row(nlv, p.inv_c, p.ext_bf16 != 0, e0, e1);
            // rows of 32 bytes under the 32-byte swizzle: the two 16-byte halves of a row
            // change places in rows 4..7 of every eight
            const int sw = (row >> 2) & 1;
            uint4* er = reinterpret_cast<uint4*>(smem + L::EXTB_OFF) + row * 2;
            er[sw] = e0;
            er[sw ^ 1] = e1;
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(ext_ready);
        }
        if (!fp.use_ext) asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_THREADS) : "memory");   // lse_buf is read by all

        // phase 2: lane = key; groups 0, 1 take the query halves of the block's first 128 keys,
        // groups 2, 3 those of its second
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        const int tg = wg >> 1;
        const int q0 = (wg & 1) * GROUP_COLS;
        const int end = colsum_end_visible(p, 0) - q0;
        const float4* nl = reinterpret_cast<const float4*>(lse_buf) + q0 / 4;
        float* dst = p.out + (long long)b * p.out_ld;
        bool out_clear = false;
        for (int i = 0; i < nblk; ++i, ++n) {
            const int kb = kb1 - 1 - i, buf = n & (NUM_TBUF - 1);
            ok = ok && mbar_wait(t_full(buf), (n >> 1) & 1, abort_flag, p.status, FCS_STATUS_WAIT_CONSUMER);
            ok = __all_sync(0xffffffffu, ok);
            tc_fence_after();
            const uint32_t taddr = lane_addr + buf * BLOCK;
            const int ktg = kb * 2 + tg;
            const int thr = colsum_first_visible(p, ktg, 0, row) - q0;
            const int thr_first_row = colsum_first_visible(p, ktg, 0, 0) - q0;
            const int thr_last_row = colsum_first_visible(p, ktg, 0, TILE - 1) - q0;
            if (ok && end > 0 && thr_first_row < GROUP_COLS) {
                const bool whole = end >= GROUP_COLS && thr_last_row <= 0;
                if (fp.use_ext) {
                    if (whole) colsum_tile_ext<false>(taddr, 0, GROUP_COLS, c, acc);
                    else colsum_tile_ext<true>(taddr, thr, end, c, acc);
                } else {
                    if (whole) colsum_tile<false>(taddr, nl, 0, GROUP_COLS, c, acc);
                    else colsum_tile<true>(taddr, nl, thr, end, c, acc);
                }
            }
            tc_fence_before();
            mbar_arrive(t_empty(buf));
            if (!out_clear) { grid_dependency_wait(); out_clear = true; }   // the output has been cleared
            const int k_abs = ktg * TILE + row;
            const float v = (acc[0] + acc[1]) + (acc[2] + acc[3]);
            // system scope: `out` may live on another GPU and take adds from several
            if (ok && k_abs < p.Sk && v != 0.f) atomicAdd_system(dst + k_abs, v);
            acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
        }
    }

    // ---------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) {
        if (*abort_flag) __nanosleep(1000000);   // let copies and MMAs in flight land
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
    // nobody leaves while a peer may still store into its shared memory: a CTA whose flow was
    // intact has waited for every such store on its exchange barrier; one that gave up a wait
    // has not, and lingers until stores issued before the peers' arrival have landed
    smallq_cluster_arrive();
    smallq_cluster_wait();
    if (*abort_flag) __nanosleep(100000);
}

}  // namespace fused
}  // namespace fcs
