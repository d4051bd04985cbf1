/*
 * flash_colsum_b200 -- C ABI of the B200 (sm_100a) attention column-mean library.
 *
 * For attention A = softmax(scale * Q K^T [+ causal mask]) the library returns,
 * per key position, the mean of A over heads and query rows without forming A.
 * The entry points are what a binding of the reference's three kernel
 * launchers would call; the Python operator `flash_colsum` binds them with
 * ctypes.  Plain pointers and sizes only: device pointers are raw addresses,
 * the stream is a cudaStream_t passed as void*.
 *
 * Common conventions
 *   - q, k: device pointers to 16-bit elements (dtype: FCS_DTYPE_*), innermost
 *     (head-dim) stride 1; the other strides are given in elements and must be
 *     multiples of 8 (16 bytes); base addresses 16-byte aligned.  D is a multiple
 *     of 8 from 8 to 128 (the kernels contract 64 or 128 columns; what lies
 *     beyond D reads as zero).
 *   - out: device pointer to fp32, row stride `out_ld` elements.  It is
 *     overwritten (zeroed by the library, then accumulated).
 *   - h_norm: number of heads the mean is taken over.  Pass H, or the global
 *     head count when this call sees only a shard of the heads and the partial
 *     results are summed afterwards.
 *   - workspace: device scratch of at least fcs_call_workspace_bytes(...) bytes
 *     (fcs_workspace_bytes(...) is an upper bound that needs no k_past),
 *     256-byte aligned, owned by the caller, not preserved between calls.
 *   - status: optional device int (may be NULL), zeroed by the caller once.  A
 *     device-side wait that ran out of time stores a non-zero code there; the
 *     caller reads it after synchronising the stream.
 *   - All calls are asynchronous on `stream`, never synchronise and never
 *     allocate.  Return value: FCS_OK or a negative FCS_ERR_* code;
 *     fcs_last_error() gives the message for the calling thread.
 *   - The first call that takes a given kernel on a device sets that kernel's
 *     shared-memory limit (and, for the cluster kernels, asks the device how many
 *     clusters it runs at once): make the first call of each shape outside any
 *     stream capture.  Later calls of the entries that take a caller's workspace
 *     have been captured in CUDA graphs and replayed (few-row, short-axis and
 *     streaming shapes); fcs_colsum_batched_static_scratch makes no statement on
 *     capture.
 */
#ifndef FLASH_COLSUM_B200_H_
#define FLASH_COLSUM_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FCS_OK 0
#define FCS_ERR_INVALID_ARGUMENT (-1)
#define FCS_ERR_UNSUPPORTED (-2)
#define FCS_ERR_WORKSPACE (-3)
#define FCS_ERR_CUDA (-4)

#define FCS_DTYPE_FP16 0
#define FCS_DTYPE_BF16 1

/* Device status codes (written to *status by a kernel whose bounded wait expired). */
#define FCS_STATUS_WAIT_PRODUCER 1
#define FCS_STATUS_WAIT_MMA 2
#define FCS_STATUS_WAIT_CONSUMER 3
#define FCS_STATUS_WAIT_PEER 4

/* Library version, as major * 10000 + minor * 100 + patch. */
int fcs_version(void);

/* Message of the last failing call made by this thread ("" if none). */
const char *fcs_last_error(void);

/*
 * Scratch bytes that are enough for ANY call with these sizes on the current
 * device: every k_past a causal call may pass, and whichever kernel the call
 * takes.  `sq_rows` is the number of query rows that enter the mean (S, or
 * min(cls_len, S)).  Returns 0 on invalid sizes.  The reference's launchers
 * allocate their own scratch with torch (flash_colsum/kernel_causal.py:104);
 * here the caller owns it.
 */
size_t fcs_workspace_bytes(int B, int H, int sq_rows, int Sk, int D, int is_causal);

/*
 * Scratch bytes the call with exactly these arguments will use, written to
 * *bytes: 0 when it takes the few-row kernel (at most four query rows), the
 * single-pass kernel (see fcs_set_single_pass) or the one-kernel form for short
 * query axes (see fcs_set_short_fused), which use none -- such a call
 * may pass workspace = NULL -- otherwise the layout of the two streaming passes
 * for this k_past (k_past < 0: the inferred max(0, Sk - sq_rows); ignored when
 * not causal).  The answer follows the kernel choice in force when it is asked:
 * ask again after fcs_set_single_pass or fcs_set_short_fused.  Never more than fcs_workspace_bytes().
 * Returns FCS_OK or an FCS_ERR_* code for sizes no call accepts.
 */
int fcs_call_workspace_bytes(int B, int H, int sq_rows, int Sk, int D, int is_causal, int k_past,
                             size_t *bytes);

/*
 * Batched non-causal column mean: out[b, k] = mean over h and over the first
 * `rows` query positions of softmax_k(scale * q[b,h,s,:] . k[b,h,k,:]), where
 * rows = S if cls_n == -1, else min(cls_n, S).
 * Replaces _flash_colsum_batched(Q, K, scale, CLS_N=-1)
 * (reference flash_colsum/kernel_noncausal_batched.py:102-125 and its kernel
 * :9-97); unlike that launcher it writes fp32 and normalises by min(cls_n, S).
 */
int fcs_colsum_batched(const void *q, const void *k, float *out, int64_t out_ld,
                       int B, int H, int S, int D, int dtype,
                       int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
                       int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_s,
                       float scale, int cls_n, int h_norm,
                       void *workspace, size_t workspace_bytes, int *status, void *stream);

/*
 * Single-sample non-causal column mean (B == 1), out has S elements.
 * Replaces _flash_colsum_non_batched(Q, K, scale, CLS_N=-1)
 * (reference flash_colsum/kernel_noncausal.py:95-117 and its kernel :9-93).
 */
int fcs_colsum_non_batched(const void *q, const void *k, float *out,
                           int H, int S, int D, int dtype,
                           int64_t q_stride_h, int64_t q_stride_s,
                           int64_t k_stride_h, int64_t k_stride_s,
                           float scale, int cls_n, int h_norm,
                           void *workspace, size_t workspace_bytes, int *status, void *stream);

/*
 * Causal suffix-query column mean (B == 1): q_len queries aligned to the end of
 * k_len keys; key j is visible to query i iff j <= k_past + i.  k_past < 0
 * means "infer": max(0, k_len - q_len).  out has k_len elements.
 * Replaces _flash_colsum_causal(Q, K, scale, K_past=None)
 * (reference flash_colsum/kernel_causal.py:94-125 and its kernel :7-92); unlike
 * that kernel it contracts the full head dimension and accepts any q_len.
 */
int fcs_colsum_causal(const void *q, const void *k, float *out,
                      int H, int q_len, int k_len, int D, int dtype,
                      int64_t q_stride_h, int64_t q_stride_s,
                      int64_t k_stride_h, int64_t k_stride_s,
                      float scale, int k_past, int h_norm,
                      void *workspace, size_t workspace_bytes, int *status, void *stream);

/*
 * Causal column mean of a batch: q [B, H, q_len, D], k [B, H, k_len, D], out (B, k_len)
 * with row stride out_ld.  The reference's operator refuses causal calls with B > 1
 * (flash_colsum/ops.py:79-82) although its naive_colsum defines them
 * (flash_colsum/baselines.py:45-63, which this entry follows), and never passes the
 * launcher's K_past (flash_colsum/kernel_causal.py:94-113; ops.py:89): here k_past >= 0
 * sets the number of keys every query sees before its own position (key j is visible to
 * query i iff j <= k_past + i, clipped to the key axis), k_past < 0 infers
 * max(0, k_len - q_len) -- which also covers k_len < q_len (baselines.py:58-62).
 */
int fcs_colsum_causal_batched(const void *q, const void *k, float *out, int64_t out_ld,
                              int B, int H, int q_len, int k_len, int D, int dtype,
                              int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
                              int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_s,
                              float scale, int k_past, int h_norm,
                              void *workspace, size_t workspace_bytes, int *status, void *stream);

/*
 * Causal column mean ADDED into `out`: same arguments and arithmetic as
 * fcs_colsum_causal, but `out` is not cleared first.  It exists for head-sharded
 * calls that flush into one buffer: every shard passes the global head count as
 * h_norm, the caller clears the buffer once, and each shard's column pass adds
 * its fp32 per-key sums with system-scope atomics -- so `out` may be a
 * peer-mapped address on another GPU of the node (the reduce over NVLink then
 * happens inside the kernel, with no separate collective).  The caller orders
 * the clear before, and the read after, all shards' calls.  No counterpart in
 * the reference, which has no multi-GPU path (its single-GPU launcher is
 * flash_colsum/kernel_causal.py:94).
 */
int fcs_colsum_causal_accumulate(const void *q, const void *k, float *out,
                                 int H, int q_len, int k_len, int D, int dtype,
                                 int64_t q_stride_h, int64_t q_stride_s,
                                 int64_t k_stride_h, int64_t k_stride_s,
                                 float scale, int k_past, int h_norm,
                                 void *workspace, size_t workspace_bytes, int *status, void *stream);

/*
 * fcs_colsum_causal_accumulate that also zeroes `clear_buf` (k_len floats, local device
 * memory, may be NULL) while it runs.  For a reduce target that alternates between two
 * buffers: the rank that owns them passes the buffer of the NEXT call here, so that the
 * clear costs no kernel of its own and one barrier per call (after the adds) is enough --
 * every rank has passed that barrier before anyone adds into the freshly cleared buffer.
 * No counterpart in the reference (single GPU only, flash_colsum/kernel_causal.py:94).
 */
int fcs_colsum_causal_accumulate_and_clear(const void *q, const void *k, float *out, float *clear_buf,
                                           int H, int q_len, int k_len, int D, int dtype,
                                           int64_t q_stride_h, int64_t q_stride_s,
                                           int64_t k_stride_h, int64_t k_stride_s,
                                           float scale, int k_past, int h_norm,
                                           void *workspace, size_t workspace_bytes, int *status, void *stream);

/*
 * fcs_colsum_causal_accumulate_and_clear whose column pass orders itself against the other GPUs
 * of a head-sharded call through flags in peer-mapped memory, so that the ranks need no barrier
 * kernel around it (one process per GPU; no counterpart in the reference):
 *   wait_flag / wait_value   (ranks that do not own `out`) local flag; nothing is added into `out`
 *                            before it has reached wait_value -- the owner stores the number of
 *                            the call during which it cleared the buffer this call adds into.
 *                            The wait is bounded (FCS_STATUS_WAIT_PEER on expiry).
 *   post / post_n / post_value  (the owner) flags on the other ranks, stored once the owner's
 *                            statistics pass -- which clears `clear_buf`, the target of the next
 *                            call -- has completed.
 *   counter / done_flag / done_value  (ranks that do not own `out`) `counter`: a local int, zero
 *                            between calls; the last CTA of the column pass stores done_value to
 *                            done_flag (on the owner) with release semantics at system scope: the
 *                            owner waits for it with fcs_peer_wait and then holds this rank's share.
 * Unused parts are NULL / 0.  Calls with at most four query rows (the few-row kernel) are
 * refused with FCS_ERR_UNSUPPORTED: order those with a barrier.
 */
typedef struct FcsPeerSignals {
    const int *wait_flag;
    int wait_value;
    int *post[15];
    int post_n;
    int post_value;
    int *counter;
    int *done_flag;
    int done_value;
} FcsPeerSignals;
int fcs_colsum_causal_accumulate_signalled(const void *q, const void *k, float *out, float *clear_buf,
                                           int H, int q_len, int k_len, int D, int dtype,
                                           int64_t q_stride_h, int64_t q_stride_s,
                                           int64_t k_stride_h, int64_t k_stride_s,
                                           float scale, int k_past, int h_norm,
                                           void *workspace, size_t workspace_bytes, int *status, void *stream,
                                           const FcsPeerSignals *signals);

/*
 * Flags between the GPUs of a node, for ordering the calls above across ranks without a
 * collective (one process per GPU; the flags live in peer-mapped memory).  fcs_peer_post
 * stores `value` to each of the n_flags (at most 16) addresses with release semantics at system
 * scope, on `stream`: everything the kernels before it in that stream wrote -- adds into another
 * GPU's buffer included -- is visible to a rank that has seen the value.  fcs_peer_wait holds
 * `stream` until each of the n_flags (at most 32) consecutive ints at `flags` (local memory) is
 * at least `value`, reading with acquire semantics; the wait is bounded (about two seconds), after
 * which FCS_STATUS_WAIT_PEER is stored to *status and the stream moves on.  A rank that waits
 * never runs on the same GPU as the rank it waits for.  No counterpart in the reference.
 */
int fcs_peer_post(int *const *flags, int n_flags, int value, void *stream);
int fcs_peer_wait(const int *flags, int n_flags, int value, int *status, void *stream);

/*
 * Batched non-causal column mean for callers that cannot give the library a
 * workspace.  It has no counterpart in the reference.
 *
 * Some hosts of this library have no device allocator to call: a plugin inside
 * an inference server that handed all device memory to its own arena at start
 * up, or a service bound through FFI (C, Go, Rust) that only ever holds the
 * input and output buffers it was given.  For them the scratch of this entry
 * point is a fixed array of FCS_STATIC_SCRATCH_BYTES built into the library's
 * device image, so the call allocates nothing: no cudaMalloc, no cudaFree, no
 * allocating library routine.  Every device that loads the library holds that
 * array until the process exits.
 *
 * Same arguments and result as fcs_colsum_batched, minus the workspace.
 *   - Limit: the call must need no more than FCS_STATIC_SCRATCH_BYTES of
 *     scratch (fcs_call_workspace_bytes(B, H, rows, S, D, 0, 0, &n): calls
 *     that take the few-row kernel, the single-pass kernel or the one-kernel
 *     form for short query axes need none and are never refused); larger problems are rejected with FCS_ERR_WORKSPACE and a
 *     message, nothing is launched.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current) and caches it.  Make
 *     that first call outside any stream capture.
 *   - All calls on a device share the one array, and it keeps whatever the
 *     previous call left there.  Each call rewrites every scratch value it
 *     later reads and clears `out` itself, so back-to-back calls on one stream
 *     are independent; two calls that overlap on the GPU (different streams,
 *     or different host threads without ordering) race on the array and give
 *     wrong results.
 */
#define FCS_STATIC_SCRATCH_BYTES (4u << 20)
int fcs_colsum_batched_static_scratch(const void *q, const void *k, float *out, int64_t out_ld,
                                      int B, int H, int S, int D, int dtype,
                                      int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
                                      int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_s,
                                      float scale, int cls_n, int h_norm,
                                      int *status, void *stream);

/*
 * The two passes apart, for splitting the WORK of one non-causal call over several devices
 * that all hold the inputs (the reference has no multi-device path; its single-sample
 * launcher is flash_colsum/kernel_noncausal.py:95).  Device r runs fcs_colsum_statistics on
 * its share of the query rows (a view of q) against all keys, the devices exchange the
 * resulting vectors, and device r runs fcs_colsum_columns on its share of the keys (a view
 * of k) against all query rows -- the output columns of the shares are final, there is
 * nothing to reduce.
 *
 * neg_lse    fp32 [B*H][fcs_statistics_rows(q_rows)]: per query row minus (log2-sum-exp of
 *            its scores + log2(h_norm * norm_rows)); rows past q_rows are not written by
 *            fcs_colsum_statistics (fill them with -inf) and are ignored by fcs_colsum_columns.
 * norm_rows  query rows that enter the mean over the whole call (>= q_rows of a share).
 * Shares of query rows must start at multiples of 256 for the vectors to concatenate.
 */
size_t fcs_statistics_rows(int q_rows);
int fcs_colsum_statistics(const void *q, const void *k, float *neg_lse,
                          int B, int H, int q_rows, int Sk, int D, int dtype,
                          int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
                          int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_s,
                          float scale, int64_t norm_rows, int h_norm,
                          void *workspace, size_t workspace_bytes, int *status, void *stream);
int fcs_colsum_columns(const void *q, const void *k, const float *neg_lse, float *out, int64_t out_ld,
                       int B, int H, int q_rows, int k_rows, int D, int dtype,
                       int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
                       int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_s,
                       float scale,
                       void *workspace, size_t workspace_bytes, int *status, void *stream);

/*
 * Token pruning on top of the column means (the operator's use in the reference's
 * README: keep the most-attended visual tokens): for each of the B rows of `colsum`
 * (fp32, S valid entries, row stride ld) the k positions with the largest value, written
 * to indices[B][k] in ascending position order (ties go to the lower position) and, if
 * `values` is not NULL, their values in the same order.  Runs on `stream`, after the
 * call that produced `colsum`; no host synchronisation, no allocation.  No counterpart in
 * the reference, which leaves the selection to its callers.
 */
int fcs_select_topk(const float *colsum, int64_t ld, int B, int S, int k,
                    int *indices, float *values, void *stream);

/*
 * The threshold form of the same step: per row the positions whose column mean is at least
 * `threshold` (relative == 0), or at least `threshold` times the row's average value
 * (relative != 0: the means of a row sum to one, so 1.0 keeps the keys that get more than a
 * uniform share of the attention).  indices[B][S]: the kept positions of row b, ascending, in
 * its first counts[b] entries, -1 in the rest.  Same stream rules as fcs_select_topk; no
 * counterpart in the reference.
 */
int fcs_select_threshold(const float *colsum, int64_t ld, int B, int S, float threshold, int relative,
                         int *indices, int *counts, void *stream);

/*
 * Measurement aids.  No counterpart in the reference, which times whole calls
 * with a host clock (benchmarks/benchmark_colsum.py:42-56).
 *
 * fcs_set_profiling(1) makes every later fcs_colsum_* call record CUDA events
 * on its stream around each of its kernels; fcs_last_pass_ms() waits for the
 * last such call on the current device and returns the duration of the
 * statistics pass, of the key-range merge (0 when the call needed none) and of
 * the column pass.  Off by default; not thread-safe.
 */
int fcs_set_profiling(int enabled);
int fcs_last_pass_ms(float *stats_ms, float *merge_ms, float *colsum_ms);

/*
 * Kernel choice for non-causal calls with head dimension 64 and at most 2048
 * keys, which can run as one pass on thread-block clusters instead of the two
 * streaming passes.  No counterpart in the reference.  mode 0 (default): the
 * single pass where it is the faster one (up to 1536 keys that fill their
 * 256-key slices to 75 % or more, or up to 2048 when the call is small);
 * 1: never; 2: whenever the shape allows.  Process-wide; not
 * thread-safe.  A single-pass call reports its whole duration as the column
 * pass in fcs_last_pass_ms().  Its results agree with the two-pass kernels to
 * ~1e-4 relative (P~ is rounded to fp16 before the second MMA).
 */
int fcs_set_single_pass(int mode);
/* 1 if a call with these sizes (sq_rows = query rows that enter the mean) takes the
 * single pass under the current mode (host arithmetic only; calls with at most four query rows take the few-row kernel
 * before this choice is made, and so do calls of at most 128 query rows that the one-kernel form of
 * fcs_set_short_fused runs in one wave of clusters). */
int fcs_single_pass_applies(int B, int H, int sq_rows, int Sk, int D, int is_causal);
/* CTAs per cluster the single pass uses for `Sk` keys (one per 256 keys) and how many
 * such clusters the current device runs at once. */
int fcs_single_pass_info(int Sk, int *cluster_size, int *max_clusters);

/*
 * Kernel choice for a query axis of at most 128 rows (the causal query suffix of a
 * prompt, a CLS prefix of more than four rows) over a short key axis.  Such calls take
 * tens of microseconds and are bound by their launches; the one-kernel form runs a
 * thread-block cluster per (batch, head): every CTA finds the row statistics of its
 * run of 256-key blocks, the CTAs exchange them through distributed shared memory, and
 * every CTA then sums its keys' columns -- one kernel behind a small clearing kernel
 * instead of three, and no scratch.  No counterpart in the reference, whose causal
 * launcher (flash_colsum/kernel_causal_batched.py:106-136) is one Triton kernel per
 * call with atomics over key blocks.
 * mode 0 (default): the cluster size is the largest with which all (batch, head) pairs
 * run at once (32 heads on 148 SMs: clusters of four); the form is taken when a cost
 * model says it is the faster one -- per wave of CTAs a ramp and the blocks one CTA
 * walks, against the three launches of the streaming form and the call's blocks spread
 * over all SMs -- and for calls bound by memory (up to 64 blocks per SM) while the
 * clusters cover four fifths of the SMs; 1: never; 2: whenever the query rows fit one tile.
 * Process-wide; not thread-safe.  The call reports its whole duration as the column
 * pass in fcs_last_pass_ms(); fcs_call_workspace_bytes() follows the mode in force.
 */
int fcs_set_short_fused(int mode);
/* 1 if a call with these sizes takes the one-kernel form under the current mode (host
 * arithmetic only; k_past < 0: the inferred value).  Calls the few-row kernel takes are
 * decided before this one; so are calls the single-pass kernel takes, unless this form
 * runs all their (batch, head) pairs in one wave of clusters.  Writes the CTAs per cluster and the key
 * blocks each walks when the pointers are not NULL. */
int fcs_short_fused_applies(int B, int H, int sq_rows, int Sk, int D, int is_causal, int k_past, int *cluster_size,
                            int *blocks_per_cta);

/*
 * Self-test of the device status path.  Every wait inside the kernels (on an mbarrier that a
 * copy, an MMA or another warp completes) is bounded: when it runs out, the CTA raises an abort
 * flag, stores an FCS_STATUS_* code to *status, all its roles fall through to the teardown,
 * tensor memory is freed and the kernel returns -- the context stays usable.  This entry runs one
 * statistics pass (one 128 x 256 tile; q: 128 x 64 fp16, k: 256 x 64 fp16, both readable) whose
 * producer issues no copies, with the limit lowered to `limit_seconds` (at most 2) for that
 * launch, so that the waits for data do run out: afterwards *status is FCS_STATUS_WAIT_MMA or
 * FCS_STATUS_WAIT_CONSUMER, and ordinary calls on the same stream work as before.  Nothing
 * faults, traps or spins without bound.  workspace: fcs_workspace_bytes(1, 1, 128, 256, 64, 0)
 * bytes.  No counterpart in the reference, whose kernels cannot fail softly.
 */
int fcs_selftest_wait_expiry(const void *q, const void *k, void *workspace, size_t workspace_bytes,
                             int *status, double limit_seconds, void *stream);
/*
 * The same for the kernels that run on thread-block clusters: one launch of the one-kernel form
 * for short query axes (one head, 128 queries, 512 keys: a cluster of two CTAs; q: 128 x 64 fp16,
 * k: 512 x 64 fp16, out: 512 floats, cleared) whose copy warp issues nothing.  Every CTA's waits
 * run out, the CTAs still meet at their barriers, exchange what they have and leave together;
 * *status is FCS_STATUS_WAIT_MMA or FCS_STATUS_WAIT_CONSUMER afterwards and `out` holds zeros.
 */
int fcs_selftest_wait_expiry_cluster(const void *q, const void *k, float *out, int *status, double limit_seconds,
                                     void *stream);

/*
 * How a call with these sizes is decomposed on the current device: key ranges
 * per query tile in the statistics pass, its work items, the 128x128 score
 * tiles of the column pass, and the SM count used for planning.  Host
 * arithmetic only.
 */
int fcs_plan_info(int B, int H, int sq_rows, int Sk, int is_causal, int *nsplit,
                  long long *stats_items, long long *colsum_steps, int *sms);

#ifdef __cplusplus
}
#endif

#endif /* FLASH_COLSUM_B200_H_ */
