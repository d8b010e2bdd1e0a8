/*
 * texb_scatter.h -- C ABI of the B200 (sm_100a) segmented scatter-reduction library.
 *
 * The library replaces the native half of TorchEx's scatter operators
 * (scatter_sum / scatter_mean / scatter_max over feats[N, C] grouped by
 * unq_inv[N]).  Every entry point takes plain device pointers and sizes, an
 * explicit CUDA stream (a cudaStream_t passed as void*; NULL = legacy default
 * stream) and returns an int status.  Nothing here allocates device memory
 * unless a comment says otherwise: scratch is a caller-provided workspace
 * whose size comes from the matching *_workspace_bytes query.  Nothing calls
 * exit() or throws.  All pointers refer to the CUDA device that is current on
 * the calling thread.
 *
 * Vocabulary: a "point" is one row of feats; a "segment" is the set of points
 * that share one id (one voxel / one pooled group); "sid" is the segment id of
 * a point; "offsets" is TorchEx's preSum array (offsets[s] .. offsets[s+1] is
 * the range of segment s in segment-sorted order); "perm" maps a position in
 * segment-sorted order to the row of feats it came from.
 */
#ifndef TEXB_SCATTER_H_
#define TEXB_SCATTER_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes --------------------------------------------------------- */
#define TEXB_OK 0
#define TEXB_ERR_INVALID_ARGUMENT 1 /* null pointer, negative size, bad enum   */
#define TEXB_ERR_UNSUPPORTED 2      /* size beyond a documented limit           */
#define TEXB_ERR_WORKSPACE 3        /* workspace smaller than *_workspace_bytes */
#define TEXB_ERR_CUDA 4             /* a CUDA runtime call or launch failed     */

/* reduce operators of texb_segment_reduce */
#define TEXB_OP_SUM 0
#define TEXB_OP_MEAN 1
#define TEXB_OP_MAX 2

/* bits of the plan_flags argument of the reduce entry points (0 and 1 keep the
 * meaning of the former has_empty argument) */
#define TEXB_PLAN_HAS_EMPTY 1 /* some segment may have no rows: fill their output rows */
#define TEXB_PLAN_SETTLED 2   /* the plan arrays were complete, and the host had synchronised
                                 with their stream, before this call (see "Stream order") */
#define TEXB_PLAN_NO_SPLIT 4  /* every cut of the balance table is a segment start (largest segment
                                 <= 128 rows, table built with the plan statistics): the reduce is
                                 then a single launch, nothing is left for a fix-up */
#define TEXB_PLAN_NO_SPLIT_MAX_CNT 128
/* Sequences: several reductions of the SAME feats with the SAME plan issued back to back
 * on one stream (a pooling layer that wants sum, mean and max of its point features).
 * Mark the first call TEXB_SEQUENCE_FIRST and the following ones TEXB_SEQUENCE_NEXT, and
 * give every call of the sequence outputs and a workspace of its own.  The first call
 * waits for the earlier work of the stream like any call; a following call does not wait
 * at its start -- its CTAs take over the SMs one by one as the CTAs of the call before it
 * retire, so the ramp-down of one reduction, the finishing of its long segments and the
 * ramp-up of the next overlap -- and waits at its end instead, so that the calls still
 * complete in order.  Every call of a sequence is a single launch (long segments are
 * finished inside the reduce kernel).  TEXB_SEQUENCE_NEXT requires TEXB_PLAN_SETTLED, and
 * nothing else may be put on the stream between the calls of a sequence. */
#define TEXB_SEQUENCE_FIRST 8
#define TEXB_SEQUENCE_NEXT 16

/* Library version (major * 100 + minor). */
int texb_version(void);

/* Message for the last non-zero status returned on the calling thread.
 * The pointer stays valid until the next failing call on that thread.
 * TorchEx has no counterpart: its CHECK_CALL prints and calls exit(1)
 * (torchex/src/utils/error.cuh:4-18) and the scatter launchers check nothing
 * (torchex/src/scatter/scatter_kernel.cu:173-192). */
const char* texb_last_error(void);

/* Health counters of the current device since the library was loaded (both 0
 * in a healthy process; either pointer may be NULL).  Synchronises with the
 * device.  No counterpart in the reference.
 *   wait_timeouts: bounded device-side waits that expired.  The reduce kernels
 *     wait for their bulk copies with an iteration limit; when it runs out they
 *     count the event and return instead of hanging.
 *   bad_indices: indices found outside their range in a plan handed to the
 *     reduce kernels (a perm entry outside [0, n), a segment id outside
 *     [0, num_segments), a balance cut outside [0, n]).  The access is skipped or
 *     redirected and counted instead of faulting; the output is then wrong. */
int texb_device_status(int* wait_timeouts, int* bad_indices);

/* Tuning knobs for experiments: "rows_per_cta" (0 = one wave of CTAs),
 * "staged" (0 register kernel, 1 cp.async ring, 2 bulk-copy ring),
 * "compensated" (1 = error-free sums), "fixup_pdl", "balanced", "end_cost_x4"
 * (cost of closing a segment in quarter rows, used by texb_plan_balance),
 * "l2_stream_hint" (1 = feature rows are copied with an L2 evict-first policy),
 * "chain_inline" (1 = segments that span several CTAs are finished inside the reduce
 * kernel by the CTA where they end, which looks back over its neighbours' records
 * with bounded waits; 0 = by a second, dependent launch).
 * Process-wide; returns TEXB_ERR_INVALID_ARGUMENT for unknown keys or values
 * out of range.  texb_tune_get returns the current value or -1. */
int texb_tune_set(const char* key, int value);
int texb_tune_get(const char* key);

/* ---- segment-offset builder ------------------------------------------------
 * Replaces ScatterData.__init__ / GetPreSumFunction
 * (torchex/operator_py/scatter_op.py:7-21, 114-135) and getPreSum_launcher
 * (torchex/src/scatter/scatter_kernel.cu:85-100, 173-175), and lifts their
 * "ids must already be sorted and dense" requirement. */

/* One pass over ids[n] (id_bytes = 4 for int32, 8 for int64).
 * Writes stats_dev[0..3] (device int32): [0] 1 if ids are non-decreasing else
 * 0, [1] minimum id, [2] maximum id, [3] number of distinct runs (equals the
 * number of distinct ids when sorted).  n == 0 gives {1, INT32_MAX, INT32_MIN, 0}. */
int texb_ids_inspect(const void* ids, int id_bytes, int64_t n,
                     int32_t* stats_dev, void* stream);

/* Workspace for texb_plan_build. */
size_t texb_plan_workspace_bytes(int64_t n, int64_t num_segments, int sorted);

/* Builds the segment plan for ids[n] with ids in [0, num_segments).
 *   sorted != 0: ids are non-decreasing.  sid_out receives the ids as int32,
 *                perm_out is not touched (may be NULL), no sort runs.
 *   sorted == 0: a stable LSD radix sort (per-digit histogram -> exclusive scan
 *                -> scatter) orders the points by id; sid_out[p] is the id at
 *                sorted position p and perm_out[p] the original row, rows of
 *                one segment in increasing row order.
 * offsets_out[num_segments + 1] is TorchEx's preSum.  plan_stats_dev[0..3]
 * (device int32): [0] largest segment size, [1] number of empty segments,
 * [2] number of ids outside [0, num_segments) (the plan is unusable if not 0),
 * [3] reserved.  Limits: n < 2^31, num_segments < 2^31. */
int texb_plan_build(const void* ids, int id_bytes, int64_t n,
                    int64_t num_segments, int sorted, int32_t* sid_out,
                    int32_t* perm_out, int32_t* offsets_out,
                    int32_t* plan_stats_dev, void* workspace,
                    size_t workspace_bytes, void* stream);

/* Optional part of the plan: balance_out[balance_len] (balance_len = K + 1,
 * K >= 1) receives increasing positions, balance_out[0] = 0 and
 * balance_out[K] = n, that cut the segment-sorted rows sid[n] into K pieces of
 * equal estimated cost (a row costs 1, closing a segment costs the
 * "end_cost_x4" knob / 4).  texb_segment_reduce hands each group of lanes a
 * run of consecutive pieces, so regions full of tiny segments do not finish
 * later than regions inside one huge segment.  K around 50 times the number
 * of groups in flight (131072 is plenty for a B200) keeps the cut fine enough.
 * A cut that falls inside a segment is moved forward to the start of the next
 * segment when that is near.  plan_stats_dev (optional, may be NULL) is the
 * statistics array that texb_plan_build / texb_unique_fill wrote in the same
 * stream: when it says that the largest segment has at most 128 rows, every cut
 * is moved to a segment start, so that no segment is split between two groups;
 * a caller who knows this on the host (largest segment <= 128 rows and the table
 * built with the statistics) may then pass TEXB_PLAN_NO_SPLIT to the reduce
 * entry points.  Without the statistics cuts move by at most 8 positions.
 * No counterpart in the reference, whose grid is one block per segment. */
int texb_plan_balance(const int32_t* sid, int64_t n, int32_t* balance_out,
                      int balance_len, const int32_t* plan_stats_dev, void* stream);

/* ---- plan straight from keys (the caller's torch.unique step) ----------------
 * TorchEx's callers obtain unq_inv / unq_cnts with
 * torch.unique(coors, dim=0, return_inverse=True, return_counts=True) before
 * they build ScatterData (torchex/operator_py/scatter_op.py:7-21 takes both as
 * inputs).  These two calls fold that step into the plan builder: keys[n]
 * (int32 or int64, any order, values in [0, key_bound), key_bound <= 2^31;
 * typically the linearised voxel coordinate) are sorted once by the same radix
 * sort, and the dense ids, counts, offsets and permutation all come out of that
 * one sort.  Dense ids follow increasing key, as torch.unique orders them.
 *
 * Call texb_unique_count, read stats_dev[0] (= number of distinct keys M) on
 * the host to size the outputs, then texb_unique_fill with the SAME workspace
 * (texb_unique_workspace_bytes(n)), untouched in between.
 *   texb_unique_count: sorted != 0 means keys are already non-decreasing (no
 *     sort runs, perm_out is not written and may be NULL).
 *   texb_unique_fill: perm = perm_out of the first call (NULL if sorted);
 *     writes sid_out[n] (dense id per sorted position), offsets_out[M + 1],
 *     unq_inv_out[n] (dense id per row, the "inverse"), unique_keys_out[M], and
 *     plan_stats_dev[0..3] as texb_plan_build does ([0] largest count). */
size_t texb_unique_workspace_bytes(int64_t n);
int texb_unique_count(const void* keys, int key_bytes, int64_t n,
                      int64_t key_bound, int sorted, int32_t* sorted_keys_out,
                      int32_t* perm_out, int32_t* stats_dev, void* workspace,
                      size_t workspace_bytes, void* stream);
int texb_unique_fill(const int32_t* sorted_keys, const int32_t* perm, int64_t n,
                     int64_t num_segments, int32_t* sid_out,
                     int32_t* offsets_out, int32_t* unq_inv_out,
                     int32_t* unique_keys_out, int32_t* plan_stats_dev,
                     void* workspace, size_t workspace_bytes, void* stream);

/* rank_out[row] = index of the point inside its segment, counted in increasing
 * row order, from a plan (sid, perm or NULL, offsets).  The deterministic form of
 * TorchEx's ingroup_inds, whose kernel hands out the indices with an atomic
 * counter in arrival order (torchex/src/ingroup_inds/ingroup_inds_kernel.cu:17-30):
 * both give each segment the set {0 .. count-1}.  A segment id outside
 * [0, num_segments) or a perm entry outside [0, n) is skipped and counted
 * (texb_device_status) instead of being used as an address. */
int texb_segment_rank(const int32_t* sid, const int32_t* perm,
                      const int32_t* offsets, int64_t n, int64_t num_segments,
                      int64_t* rank_out, void* stream);

/* Drop-in for getPreSum_launcher(unq_inv, preSum, num_total)
 * (torchex/src/scatter/scatter.cpp:18, scatter_kernel.cu:173-175): sorted
 * int32 ids -> pre_sum[num_unq + 1].  Unlike the reference every entry is
 * written (pre_sum need not be zero-filled) and skipped ids give empty
 * segments instead of corrupt offsets. */
int texb_get_pre_sum(const int32_t* unq_inv, int32_t* pre_sum,
                     int64_t num_total, int64_t num_unq, void* stream);

/* ---- forward reduce ----------------------------------------------------------
 * Replaces scatter_sum_launcher / scatter_max_launcher
 * (torchex/src/scatter/scatter.cpp:12-16, scatter_kernel.cu:102-171, 177-192)
 * and the separate mean divide (torchex/operator_py/scatter_op.py:68-69). */

/* Workspace for texb_segment_reduce (depends on the "rows_per_cta" knob). */
size_t texb_reduce_workspace_bytes(int64_t n, int channel);

/* out[s, :] = reduce over the rows of segment s of feats[N, channel] (fp32,
 * row-major).  sid[n] is the segment id at each segment-sorted position;
 * perm[n] the feats row at that position, or NULL when feats is already in
 * segment order; it must list the rows of one segment in increasing order
 * (texb_plan_build does) for the lowest-row tie rule of TEXB_OP_MAX to hold.
 * balance / balance_len: the table of texb_plan_balance, or NULL / 0 for an
 * even split of the rows.  plan_flags: TEXB_PLAN_* bits.  offsets may be NULL unless
 * TEXB_PLAN_HAS_EMPTY is set; with it the rows of empty segments are filled (0 for
 * sum/mean; -FLT_MAX and -1 for max, what the reference kernel writes for an empty
 * range).  Setting the bit when no segment is empty only costs the check.
 *   TEXB_OP_SUM : fp32 sum, compensated (error-free transformation) so that
 *                 long segments stay within 1e-6 + 1e-5*|x| of the exact sum.
 *   TEXB_OP_MEAN: that sum divided (IEEE fp32 division) by the row count.
 *   TEXB_OP_MAX : maximum and, in arg[num_segments, channel] (int32), the
 *                 feats row holding it plus arg_base (0 for a stand-alone call;
 *                 the first global row of a shard when feats is one shard of a
 *                 larger batch; "no row" stays -1); ties go to the lowest row;
 *                 NaN never wins (as in the reference, scatter_kernel.cu:146-151).
 * No floating-point atomics: results are bit-reproducible run to run.
 * Limits: n < 2^31, channel >= 1.
 * Stream order: the kernels are programmatic dependent launches: their CTAs may
 * be placed while the kernel that precedes the call in the stream is still
 * finishing, and they wait (griddepcontrol.wait) until all earlier work of the
 * stream has completed and its memory is visible before they read or write
 * anything -- so the call behaves like any kernel launch.  With
 * TEXB_PLAN_SETTLED the kernels read the plan arrays (sid, perm, balance) BEFORE
 * that wait, which hides about 1.5 us of prologue per call in a sequence of
 * reductions.  Only set the bit when the plan arrays were completely written and
 * the host has since synchronised with the stream (or device) that wrote them --
 * e.g. a plan built once and reused, after any cudaStreamSynchronize /
 * cudaEventSynchronize that followed its construction.  Work merely ordered
 * earlier in the same stream is NOT enough: its writes become visible at the
 * wait, not before. */
int texb_segment_reduce(int op, const float* feats, const int32_t* sid,
                        const int32_t* perm, const int32_t* offsets,
                        int plan_flags, const int32_t* balance, int balance_len,
                        int64_t n, int channel, int64_t num_segments,
                        float* out, int32_t* arg, int32_t arg_base,
                        void* workspace, size_t workspace_bytes, void* stream);

/* texb_segment_reduce for bf16 features (feats_bf16[N, channel], row-major):
 * every value is widened exactly to fp32, accumulated as in the fp32 entry
 * point (error-free sums, exact maxima) and written as fp32, so the result
 * equals texb_segment_reduce on the widened features while reading half the
 * bytes.  The reference is fp32-only (torchex/src/scatter/scatter.cpp:30, 48).
 * Limits: channel a multiple of 8 and at least 128, pointers 16-byte aligned;
 * other shapes return TEXB_ERR_UNSUPPORTED (widen them to fp32 instead).
 * Workspace: texb_reduce_workspace_bytes, as for fp32. */
int texb_segment_reduce_bf16(int op, const void* feats_bf16, const int32_t* sid,
                             const int32_t* perm, const int32_t* offsets,
                             int plan_flags, const int32_t* balance,
                             int balance_len, int64_t n, int channel,
                             int64_t num_segments, float* out, int32_t* arg,
                             int32_t arg_base, void* workspace,
                             size_t workspace_bytes, void* stream);

/* Sum (or mean) AND maximum of the same rows in one pass over feats: dynamic
 * voxel encoders pool the same point features both ways, and two calls of
 * texb_segment_reduce would read feats twice.  No counterpart in the
 * reference, which runs ScatterMeanFunction and ScatterMaxFunction one after
 * the other (torchex/operator_py/scatter_op.py:56-103).
 *   op           : TEXB_OP_SUM or TEXB_OP_MEAN, written to out_sum[num_segments, channel];
 *   out_max, arg : as out / arg of TEXB_OP_MAX;
 *   feature_bytes: 4 (feats is fp32) or 2 (bf16; channel a multiple of 8, from
 *                  128 channels, and at most 128 -- wider bf16 rows: convert);
 *   workspace    : texb_reduce_pair_workspace_bytes(n, channel) bytes.
 * Each output is bit-identical to what the single-output call writes when both
 * use the same split of the rows (they do by default for fp32 rows). */
size_t texb_reduce_pair_workspace_bytes(int64_t n, int channel);
int texb_segment_reduce_pair(int op, const void* feats, int feature_bytes,
                             const int32_t* sid, const int32_t* perm,
                             const int32_t* offsets, int plan_flags,
                             const int32_t* balance, int balance_len, int64_t n,
                             int channel, int64_t num_segments, float* out_sum,
                             float* out_max, int32_t* arg, int32_t arg_base,
                             void* workspace, size_t workspace_bytes,
                             void* stream);

/* One-launch reduction for small inputs made of short segments: one warp per
 * segment, straight from offsets[num_segments + 1] (TorchEx's preSum) and, for
 * unsorted ids, perm[n]; no workspace, no fix-up launch, no sid / balance arrays,
 * and empty segments are written by the kernel itself (0 for sum/mean, -FLT_MAX
 * and -1 for max).  It takes the place of scatter_sum_launcher /
 * scatter_max_launcher (torchex/src/scatter/scatter.cpp:12-16) on inputs of a
 * megabyte or so, where one launch of the reference's kernel used to beat the
 * launch pair of texb_segment_reduce.  Same arithmetic as texb_segment_reduce
 * (compensated sums, IEEE division, lowest row on ties, NaN never wins); max and
 * argmax are bit-identical to it, sums may differ in the last bit.
 * The result is correct for every input, but a segment is walked by a single
 * warp: use it when texb_segment_reduce_small_ok(n, channel, max_cnt) returns 1
 * (features of at most 8 MB, largest segment at most 128 rows; max_cnt < 0 =
 * unknown gives 0). */
int texb_segment_reduce_small_ok(int64_t n, int channel, int64_t max_cnt);
int texb_segment_reduce_small(int op, const float* feats, const int32_t* offsets,
                              const int32_t* perm, int64_t n, int channel,
                              int64_t num_segments, float* out, int32_t* arg,
                              int32_t arg_base, void* stream);

/* texb_segment_reduce for callers that cannot allocate device memory.
 * No counterpart in the reference.
 *
 * Who needs it: code that is not allowed to call cudaMalloc (or any allocating
 * library routine) once it is running -- a real-time perception loop whose
 * buffers are all sized at start-up, a plugin that lives inside a host
 * application's fixed memory pool, code placed between stream-ordered work
 * where an allocation would stall the device.  Such a caller owns feats, the
 * plan arrays and the outputs, but has nowhere to get the reduce workspace.
 *
 * Here the workspace is an array inside the library image,
 * texb_static_scratch_bytes() = 4 MiB, held by every GPU that loads the
 * library until the process exits.  The call allocates nothing: no cudaMalloc,
 * no cudaFree, no allocating library call.  Arguments and results are those of
 * texb_segment_reduce without the workspace pair.
 *
 * Limits and rules:
 *   - a shape whose records do not fit in the 4 MiB (only possible with a very
 *     small "rows_per_cta" knob or thousands of channels) is rejected with
 *     TEXB_ERR_UNSUPPORTED and a message; nothing is launched;
 *   - the first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current) and loads the kernels;
 *     make that first call before any stream capture begins;
 *   - all calls on one GPU share the one array and it keeps the previous
 *     call's contents (the kernels rewrite every word they later read, so
 *     nothing needs clearing); two calls that overlap on the GPU, e.g. on
 *     different streams, race on it -- keep them on one stream or order them
 *     with events. */
size_t texb_static_scratch_bytes(void);
int texb_segment_reduce_static(int op, const float* feats, const int32_t* sid,
                               const int32_t* perm, const int32_t* offsets,
                               int plan_flags, const int32_t* balance,
                               int balance_len, int64_t n, int channel,
                               int64_t num_segments, float* out, int32_t* arg,
                               int32_t arg_base, void* stream);

/* Workspace for the two reference-shaped entry points below: room to expand
 * pre_sum back into per-row segment ids plus texb_reduce_workspace_bytes. */
size_t texb_scatter_compat_workspace_bytes(int64_t num_total, int channel);

/* Drop-in for scatter_sum_launcher(feats, preSum, out, channel, num_unq,
 * max_cnt) (torchex/src/scatter/scatter.cpp:12-13): feats in segment order.
 * max_cnt (the reference sizes its thread blocks from it,
 * scatter_kernel.cu:177-183) only selects the path here: a small input whose
 * largest segment is short (texb_segment_reduce_small_ok) takes the one-launch
 * kernel and touches no workspace; pass 0 or a negative value if it is not
 * known.  num_total = feats rows, which the reference takes from the tensor. */
int texb_scatter_sum(const float* feats, const int32_t* pre_sum, float* out,
                     int channel, int num_unq, int max_cnt, int64_t num_total,
                     void* workspace, size_t workspace_bytes, void* stream);

/* Drop-in for scatter_max_launcher(feats, preSum, out, arg, channel, num_unq,
 * max_cnt) (torchex/src/scatter/scatter.cpp:15-16). */
int texb_scatter_max(const float* feats, const int32_t* pre_sum, float* out,
                     int32_t* arg, int channel, int num_unq, int max_cnt,
                     int64_t num_total, void* workspace,
                     size_t workspace_bytes, void* stream);

/* ---- backward -------------------------------------------------------------
 * Replace the ATen expressions of the autograd Functions.  In all three,
 * entry i of ids[n] names the segment and the row of g_in that is written is
 * perm[i], or i itself when perm is NULL.  Two ways to call them:
 *   - ids = unq_inv in the caller's order, perm = NULL: the reference's
 *     g[unq_inv] gather, one row of g fetched per point;
 *   - ids = the plan's sid, perm = the plan's perm (NULL if the ids arrived
 *     sorted): the same result walked in segment order, where neighbouring
 *     entries share their segment and the rows of g / arg are fetched once.
 * Every row of g_in is written exactly once (perm is a permutation). */

/* g_in[row_i, :] = g[ids[i], :]
 * (ScatterSumFunction.backward, torchex/operator_py/scatter_op.py:47-50). */
int texb_scatter_sum_backward(const float* g, const int32_t* ids,
                              const int32_t* perm, float* g_in, int64_t n,
                              int channel, int64_t num_segments, void* stream);

/* g_in[row_i, :] = g[ids[i], :] / count(ids[i]), count taken from offsets and the
 * quotient rounded as an IEEE fp32 division
 * (ScatterMeanFunction.backward, torchex/operator_py/scatter_op.py:73-78). */
int texb_scatter_mean_backward(const float* g, const int32_t* ids,
                               const int32_t* perm, const int32_t* offsets,
                               float* g_in, int64_t n, int channel,
                               int64_t num_segments, void* stream);

/* g_in[row_i, c] = (arg[ids[i], c] == row_i) ? g[ids[i], c] : 0, one fused
 * pass instead of zeros + scatter_ (the intent of ScatterMaxFunction.backward,
 * torchex/operator_py/scatter_op.py:105-111, which raises as shipped). */
int texb_scatter_max_backward(const float* g, const int32_t* arg,
                              const int32_t* ids, const int32_t* perm,
                              float* g_in, int64_t n, int channel,
                              int64_t num_segments, void* stream);

/* Backward of texb_segment_reduce_pair with TEXB_OP_MEAN: the sum of the two
 * expressions above, g_in[row_i, c] = g_mean[ids[i], c] / count(ids[i]) +
 * ((arg[ids[i], c] == row_i) ? g_max[ids[i], c] : 0), in one pass that writes
 * g_in once. */
int texb_scatter_mean_max_backward(const float* g_mean, const float* g_max,
                                   const int32_t* arg, const int32_t* ids,
                                   const int32_t* perm, const int32_t* offsets,
                                   float* g_in, int64_t n, int channel,
                                   int64_t num_segments, void* stream);

/* ---- peer buffers for the multi-GPU driver ---------------------------------------
 * One process per GPU; a caller that wants every GPU to hold the whole result of a
 * sharded reduction lets each GPU write its shard into a buffer the other processes
 * can map, and each GPU then pulls the other shards into its own memory: with one
 * kernel that loads from all peers at once (texb_peer_pull), or with plain
 * device-to-device copies on the copy engines (texb_peer_copy).  Ordering between
 * the processes -- a shard is complete before it is pulled and pulled before it is
 * overwritten -- is the caller's job (torchex_b200/peer_ring.py uses one small NCCL
 * collective per gather).  No counterpart in the reference, which has no multi-GPU code.
 *   texb_peer_buffer_create : cudaMalloc of `bytes` on the current device (THIS call
 *     allocates; free with texb_peer_buffer_destroy) and its 64-byte CUDA IPC handle,
 *     to be sent to the other processes by any host channel;
 *   texb_peer_buffer_open   : maps a peer's buffer into this process with the current
 *     device as the accessing device (peer access is enabled lazily); the pointer is
 *     only ever used as a source of texb_peer_copy / texb_peer_pull; close it before
 *     the owner destroys the buffer;
 *   texb_peer_copy          : cudaMemcpyAsync(dst, src, bytes) on `stream`;
 *   texb_peer_pull          : copies `n` regions, srcs[k] -> dsts[k] of bytes[k] bytes
 *     (host arrays; multiples of 4 bytes at 4-byte aligned addresses, 16-byte alignment
 *     is faster), with one kernel launch per TEXB_PEER_PULL_MAX regions on `stream`.
 *     Sources may be peer mappings or local memory, destinations are local memory.
 *     The kernel only loads from the sources: plain ld.global, no TMA, no multicast,
 *     no waiting on anything.
 *   texb_peer_pull_mean     : texb_peer_pull for regions that hold whole rows of SUMS
 *     (`channel` floats per row, channel divisible by 4, everything 16-byte aligned):
 *     next to every copied row it writes the row of means into mean_dsts[k], dividing by
 *     counts[first_rows[k] + row of the region] exactly as the mean reduction divides
 *     (`counts`: int32 segment sizes on this GPU; sizes <= 1 leave the row as it is).
 *     The copy is bound by the links, so the means cost no time and no second pass.
 *   texb_mean_from_sum      : out[s, :] = sums[s, :] / counts[s] for the num_segments
 *     rows of `channel` floats, with the same correctly rounded division the mean
 *     reduction applies to its sums (rows with counts[s] <= 1 are copied).  A caller
 *     that holds the replicated sums and the segment sizes gets the replicated means
 *     from local memory instead of moving a second tensor between the GPUs. */
#define TEXB_PEER_HANDLE_BYTES 64
#define TEXB_PEER_PULL_MAX 16
int texb_peer_buffer_create(size_t bytes, void** dev_ptr, unsigned char* handle_out);
int texb_peer_buffer_destroy(void* dev_ptr);
int texb_peer_buffer_open(const unsigned char* handle, void** peer_ptr);
int texb_peer_buffer_close(void* peer_ptr);
int texb_peer_copy(void* dst, const void* src, size_t bytes, void* stream);
int texb_peer_pull(const void* const* srcs, void* const* dsts, const size_t* bytes, int n, void* stream);
int texb_peer_pull_mean(const void* const* srcs, void* const* dsts, void* const* mean_dsts, const size_t* bytes,
                        const int64_t* first_rows, int n, const int32_t* counts, int channel, void* stream);
int texb_mean_from_sum(const float* sums, const int32_t* counts, int64_t num_segments, int channel,
                       float* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TEXB_SCATTER_H_ */
