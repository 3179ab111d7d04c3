/*
 * minfer_b200 -- C ABI of the B200 (sm_100a) dynamic sparse prefill attention library.
 *
 * Conventions
 *   - Every pointer named q/k/v/o/plan/..., unless marked "host", is a DEVICE pointer
 *     owned by the caller.  The library never allocates or frees device memory.
 *   - `stream` is a cudaStream_t passed as void*; every call only enqueues work on it.
 *   - Return value: 0 on success, a negative MINF_E_* code when the arguments are
 *     rejected or a CUDA launch fails (minf_last_error() then holds a message for the
 *     calling thread).  Problems found on the device (a row block with no usable slash
 *     offset, an abandoned wait) are reported through the caller's `status` words, which
 *     the caller zeroes before the first call and may read after synchronising.
 *   - Tensors are [batch, heads, tokens, head_dim] with head_dim contiguous; the three
 *     outer strides are given in elements.  head_dim must be 128, dtype bf16.
 *   - Citations name files of microsoft/MInference v0.1.6.0.
 */
#ifndef MINFER_B200_H
#define MINFER_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MINF_OK 0
#define MINF_E_ARG (-1)      /* invalid argument combination */
#define MINF_E_CUDA (-2)     /* CUDA runtime / driver error at launch */
#define MINF_E_UNSUPPORTED (-3)

/* status[] words written by the kernels (caller provides int32_t status[MINF_STATUS_WORDS], 8-byte aligned) */
#define MINF_STATUS_WORDS 4
#define MINF_ST_ERROR 0      /* bit 0: a device wait was abandoned; bit 1: misaligned smem; bit 2: bad plan (a head in
                                plan mode without a plan, a range count beyond the slot's capacity, ranges that are
                                not ascending and disjoint, or marked columns without a vertical list; the affected
                                row blocks are computed from the part of the plan read before the fault); bit 3: a
                                range check of the debug build (-DMINF_BOUNDS) failed and the access was skipped */
#define MINF_ST_NO_SLASH 1   /* number of row blocks whose slash list has no offset < end row */
#define MINF_ST_AUX0 2        /* words 2-3, read as one uint64: 64x64 tile equivalents the attention kernel sent  */
#define MINF_ST_AUX1 3        /* to the tensor pipe (its 128-row x 64/128-key steps), summed over launches         */

/* per-head attention pattern, values of head_mode[] */
#define MINF_MODE_PLAN 0     /* vertical-slash or block-sparse: tiles and columns come from the plan */
#define MINF_MODE_ASHAPE 1   /* sink + sliding window, parameters in head_param[] */

const char* minf_version(void);
const char* minf_last_error(void);

/*
 * Self-test of the bounded device wait: launches one CTA that waits on a barrier nothing arrives on.
 * After `limit_us` microseconds (1 .. 1000000) the wait is abandoned and the kernel returns through its
 * normal exit with bit 0 of status[MINF_ST_ERROR] set; the context stays usable.  Every wait inside the
 * attention and estimator kernels takes the same path (with a limit of two seconds).  No counterpart
 * in the reference.
 */
int minf_selftest_bounded_wait(int limit_us, int32_t* status, void* stream);

/*
 * Reference-format index conversion.  Replaces
 *   minference.cuda.convert_vertical_slash_indexes (csrc/kernels.cpp:7-17,
 *   csrc/vertical_slash_index.cu:127-167, kernel :27-99).
 * vertical_indexes [batch, heads, nnz_v] ascending, slash_indexes [batch, heads, nnz_s]
 * descending, both int32.  Outputs (int32): block_count [batch, heads, rows],
 * block_offset [batch, heads, rows, nnz_s], column_count [batch, heads, rows],
 * column_index [batch, heads, rows, nnz_v] with rows = ceil(context_size / 64).  Every
 * element of the outputs is written (zero tails included), so they need no memset.
 */
int minf_convert_vertical_slash_indexes(
    const int32_t* seqlens, const int32_t* vertical_indexes, const int32_t* slash_indexes,
    int batch, int heads, int context_size, int nnz_v, int nnz_s,
    int32_t* block_count, int32_t* block_offset, int32_t* column_count, int32_t* column_index,
    int32_t* status, void* stream);

/*
 * Compact plan consumed by minf_sparse_attention_fwd: the same index set as above, kept
 * as merged [start, end) token ranges plus a bit mask over the head's vertical list
 * instead of dense per-row-block tables.  `nnz_v_per_head` / `nnz_s_per_head` (int32
 * [batch*heads], device) give the live length of each head's list inside its
 * cap_v / cap_s wide row; pass NULL when every head uses the full width.
 * No counterpart in the reference (it materialises the dense tables per head,
 * ops/pit_sparse_flash_attention_v2.py:218-224).
 */
size_t minf_plan_bytes(int batch, int heads, int context_size, int cap_v, int cap_s);
int minf_vs_build_plan(
    const int32_t* seqlens, const int32_t* vertical_indexes, const int32_t* slash_indexes,
    const int32_t* nnz_v_per_head, const int32_t* nnz_s_per_head,
    int batch, int heads, int context_size, int cap_v, int cap_s,
    void* plan, int32_t* status, void* stream);

/*
 * The same for a window of the sequence: the plan covers the n_q query rows that start at
 * position q_pos0 (a multiple of 64; 256 when the plan feeds minf_sparse_attention_fwd_window).
 * Used by sequence-sharded callers, which build one plan per local query chunk from the
 * global index lists.  seqlens still holds the length of the whole sequence.
 */
size_t minf_plan_bytes_window(int batch, int heads, int q_pos0, int n_q, int cap_v, int cap_s);
int minf_vs_build_plan_window(
    const int32_t* seqlens, const int32_t* vertical_indexes, const int32_t* slash_indexes,
    const int32_t* nnz_v_per_head, const int32_t* nnz_s_per_head,
    int batch, int heads, int q_pos0, int n_q, int cap_v, int cap_s,
    void* plan, int32_t* status, void* stream);

/*
 * Block-sparse plan: top-k key blocks per query block from mean-pooled Q and K.  Replaces
 * _build_block_index (ops/block_sparse_flash_attention.py:151-166) including the padding
 * rule of its caller (:178).  Only heads whose head_mode entry is MINF_MODE_PLAN and whose
 * head_select entry is non-zero are written (head_select may be NULL = all heads).
 * `block_index_out` (optional, int32 [batch, hq, rows_pad, top_k_eff], rows_pad =
 * (context_size + pad)/64) receives the reference-format sorted block ids.
 * `scratch` holds minf_block_sparse_scratch_bytes() bytes.
 */
size_t minf_block_sparse_scratch_bytes(int batch, int hq, int hkv, int context_size);
int minf_block_sparse_build_plan(
    const void* q, const void* k,
    const int64_t q_strides[3], const int64_t k_strides[3],
    int batch, int hq, int hkv, int context_size, int head_dim, int top_k,
    const int32_t* head_select,
    int cap_v, int cap_s, void* plan, int32_t* block_index_out,
    void* scratch, int32_t* status, void* stream);

/*
 * The same planner in two steps for a sequence-sharded caller (no counterpart in the reference,
 * which has no sequence parallelism).  minf_block_sparse_pool: mean of each block of 64 rows of
 * `x` [batch, heads, n_rows, 128] -> `pooled` bf16 [batch, heads, ceil(n_rows/64), 128] (a ragged
 * last block is divided by 64 like the reference's zero padding).  The caller gathers the pooled
 * keys of the whole sequence in order.  minf_block_sparse_select_window: top-k key blocks for the
 * query blocks of rows [q_pos0, q_pos0 + n_q) (q_pos0 a multiple of 64) from `q_pooled`
 * [batch, hq, ceil(n_q/64), 128] and `k_pooled` [batch, hkv, ceil(context_size/64), 128], written
 * into a window plan (minf_plan_bytes_window) for the heads `head_select` marks.
 */
int minf_block_sparse_pool(
    const void* x, const int64_t strides[3], int batch, int heads, int n_rows, void* pooled, void* stream);
int minf_block_sparse_select_window(
    const void* q_pooled, const void* k_pooled, int batch, int hq, int hkv, int context_size,
    int q_pos0, int n_q, int top_k, const int32_t* head_select, int cap_v, int cap_s, void* plan, void* stream);

/*
 * Online vertical/slash index estimation for all heads in one call.  Replaces the torch
 * ops of vertical_and_slash_kernel (modules/minference_forward.py:599-614) and
 * sum_all_diagonal_matrix (:110-116): last-64-query x K^T logits, causal mask of the last
 * block, fp32 softmax, column sums and anti-diagonal sums, +inf forcing of the first 30
 * columns and the 100 nearest diagonals, per-head top-k.  Outputs are already in the order
 * the index conversion wants (:218-219 of ops/pit_sparse_flash_attention_v2.py):
 * v_idx_out [batch, hq, cap_v] ascending, s_idx_out [batch, hq, cap_s] descending offsets.
 * vertical_size / slash_size: int32 [batch*hq] on the device, per-head budgets before the
 * reference's clamping (:600); a negative budget skips the head (nnz = -1 is written, and
 * minf_vs_build_plan leaves heads with a negative slash count untouched).  The clamped
 * live counts are written to nnz_v_out / nnz_s_out.  vertical_scores_out /
 * slash_scores_out (optional, fp32 [batch, hq, context_size]; slash indexed by diagonal
 * offset) receive the raw scores.
 * `scratch` holds minf_vs_estimate_scratch_bytes() bytes.
 */
size_t minf_vs_estimate_scratch_bytes(int batch, int hq, int context_size);
int minf_vs_estimate(
    const void* q, const void* k,
    const int64_t q_strides[3], const int64_t k_strides[3],
    int batch, int hq, int hkv, int context_size, int head_dim,
    const int32_t* vertical_size, const int32_t* slash_size,
    int cap_v, int cap_s,
    int32_t* v_idx_out, int32_t* s_idx_out, int32_t* nnz_v_out, int32_t* nnz_s_out,
    float* vertical_scores_out, float* slash_scores_out,
    void* scratch, int32_t* status, void* stream);

/*
 * Attention plan from a block mask (the index set of the reference's FlexPrefill path: flattened block ids built at
 * modules/flexprefill.py:903-927 and walked per query block by its kernel at :353-495).  `mask` is
 * [batch*heads, nb, nb] bytes, nb = ceil(context_size / block_tokens), entry (i, j) non-zero <=> query block i
 * attends key block j; entries with j > i are ignored and every block is causal inside.  block_tokens is a multiple
 * of 64.  Runs of neighbouring key blocks become one token range of the plan; `cap_s` is the largest number of runs a
 * row of the mask may have (more sets bit 2 of status[MINF_ST_ERROR]).  The plan holds minf_plan_bytes(batch, heads,
 * context_size, 0, cap_s) bytes and is consumed by minf_sparse_attention_fwd with cap_v = 0.
 */
int minf_block_mask_build_plan(
    const uint8_t* mask, int batch, int heads, int context_size, int block_tokens, int cap_s,
    void* plan, int32_t* status, void* stream);

/*
 * The stages of minf_vs_estimate as separate calls, for callers that hold only part of the keys
 * (sequence sharding): statistics pass over the local keys, exchange of the per-block statistics,
 * combination, score pass, reduction of the score arrays over the ranks, selection.
 *   q_last   the last min(64, context_size) queries of every head, [batch, hq, last_q, 128]
 *   k        the n_k local keys at positions [col_base, col_base + n_k) (col_base % 128 == 0)
 *   stats    float2 [batch*hq][64][blocks_total]: (row max, row sum) of the softmax per block of
 *            2048 keys, blocks counted from col_base.  Pass 1 writes the
 *            minf_vs_scores_blocks(n_k) entries that start at block_offset.  The caller lays the
 *            blocks of the whole sequence out in ascending key order (all-gather, then reorder).
 *   row_stats float2 [batch*hq][64]: written by minf_vs_scores_combine from all blocks_total
 *            entries of a row, read by pass 2.
 *   vertical_scores / slash_scores   fp32 [batch, hq, context_size], zeroed by the caller before
 *            pass 2 (slash is indexed by diagonal offset; entries whose keys span two calls are
 *            accumulated with atomics, every other entry is stored).
 * When every chunk starts at a multiple of 2048 keys the scores, and with them the selected
 * index lists, are bit-identical however the sequence is split over calls or ranks.
 * No counterpart in the reference beyond minference_forward.py:599-614.
 */
int minf_vs_scores_blocks(int n_k);
int minf_vs_scores_pass(
    int pass, const void* q_last, const void* k,
    const int64_t q_strides[3], const int64_t k_strides[3],
    int batch, int hq, int hkv, int context_size, int n_k, int col_base, int head_dim,
    void* stats, int block_offset, int blocks_total, const void* row_stats,
    float* vertical_scores, float* slash_scores,
    int32_t* status, void* stream);
int minf_vs_scores_combine(const void* stats, int batch, int hq, int blocks_total, void* row_stats, void* stream);
/*
 * minf_vs_scores_pass with the divisor of the logits given by the caller instead of sqrt(head_dim): the bf16 product
 * q_last . k is divided by `logit_divisor` and rounded to bf16 again.  With 1.0 the product is used as it is, which
 * is what the FlexPrefill estimator needs: it scales the queries first and rounds once
 * (modules/flexprefill.py:968-975 of the reference).
 */
int minf_vs_scores_pass_divisor(
    int pass, const void* q_last, const void* k,
    const int64_t q_strides[3], const int64_t k_strides[3],
    int batch, int hq, int hkv, int context_size, int n_k, int col_base, int head_dim, float logit_divisor,
    void* stats, int block_offset, int blocks_total, const void* row_stats,
    float* vertical_scores, float* slash_scores,
    int32_t* status, void* stream);
/*
 * Per-head top-k over the score arrays.  The first `force_columns` keys and the `force_diagonals` nearest
 * diagonals are always taken and budgets are raised to `min_vertical` / `min_slash`: 30, 100, 30, 50 for the
 * online path (minference_forward.py:600, :608, :612), 30, 30, 30, 50 for its static variant (:421, :433) and
 * 30, 30, 0, 0 for the offline search (:140-146).  `scratch` holds minf_vs_select_scratch_bytes() bytes
 * (histograms and per-segment counts).
 */
size_t minf_vs_select_scratch_bytes(int batch, int hq, int context_size);
int minf_vs_select(
    const float* vertical_scores, const float* slash_scores, int batch, int hq, int context_size,
    const int32_t* vertical_size, const int32_t* slash_size, int cap_v, int cap_s,
    int32_t* v_idx_out, int32_t* s_idx_out, int32_t* nnz_v_out, int32_t* nnz_s_out,
    int force_columns, int force_diagonals, int min_vertical, int min_slash, void* scratch, void* stream);

/*
 * minf_vs_estimate for callers that cannot provide scratch memory and must not trigger an
 * allocation (a plugin inside a process whose device memory is a pre-carved arena it has no
 * handle to, or a caller on a path where allocators are off limits).  No counterpart in the
 * reference.  Same inputs and outputs as minf_vs_estimate minus `scratch` and the optional score
 * outputs; the scratch is a fixed 16 MiB array in the library's device image (one per GPU that
 * loads the library, held until the process exits), which limits the problem to about
 * batch*hq*context_size <= 1M (minf_vs_estimate_scratch_bytes() must not exceed
 * minf_vs_estimate_static_scratch_limit()); larger problems return MINF_E_UNSUPPORTED.
 * Nothing is allocated or freed.  All calls on a GPU share the array: calls that may overlap on
 * the device race with each other and must be serialised by the caller.  The first call on a
 * device looks up the array's device address once; make that call outside any stream capture.
 */
size_t minf_vs_estimate_static_scratch_limit(void);
int minf_vs_estimate_static(
    const void* q, const void* k,
    const int64_t q_strides[3], const int64_t k_strides[3],
    int batch, int hq, int hkv, int context_size, int head_dim,
    const int32_t* vertical_size, const int32_t* slash_size,
    int cap_v, int cap_s,
    int32_t* v_idx_out, int32_t* s_idx_out, int32_t* nnz_v_out, int32_t* nnz_s_out,
    int32_t* status, void* stream);

/*
 * Sparse flash-attention forward for all heads in one launch.  Replaces
 * _triton_mixed_sparse_attention (ops/pit_sparse_flash_attention_v2.py:48-192),
 * _triton_block_sparse_attention (ops/block_sparse_flash_attention.py:29-148) and the
 * two-stage streaming kernel (ops/streaming_kernel.py:116-239, 611-646).
 * K and V may have fewer heads than Q (hq % hkv == 0); query head h reads KV head
 * h / (hq / hkv).  head_mode [hq] (device, int32, NULL = all MINF_MODE_PLAN) selects the
 * pattern per head; head_param [hq][2] (device) holds {n_init, n_local} for A-shape heads.
 * vertical_indexes is the same array given to minf_vs_build_plan (may be NULL when the
 * plan has no columns).  Output rows >= context_size are never written.
 */
int minf_sparse_attention_fwd(
    const void* q, const void* k, const void* v, void* o,
    const int64_t q_strides[3], const int64_t k_strides[3],
    const int64_t v_strides[3], const int64_t o_strides[3],
    int batch, int hq, int hkv, int context_size, int head_dim, float sm_scale,
    const int32_t* head_mode, const int32_t* head_param,
    const void* plan, const int32_t* vertical_indexes, int cap_v, int cap_s,
    int32_t* status, void* stream);

/*
 * One (query chunk, key chunk) pair of a sequence-sharded attention.  q/o hold the n_q query
 * rows at positions [q_pos0, q_pos0 + n_q) (q_pos0 a multiple of 256), k/v hold the n_kv keys
 * at positions [kv_pos0, kv_pos0 + n_kv) (kv_pos0 a multiple of 64); `plan` was built with
 * minf_vs_build_plan_window for the same query window; context_size is the length of the whole
 * sequence.  Keys outside the key window are left to other calls.  `lse` (optional, fp32
 * [batch, hq, n_q]) receives per row the base-2 logarithm of the sum of 2^(logit * sm_scale *
 * log2(e)) over the keys this call saw (-inf when it saw none); the output rows are normalised
 * with that sum, so partial results of several key chunks combine as
 *   o = sum_i 2^(lse_i - lse) * o_i,   lse = log2(sum_i 2^lse_i).
 * The kernel does that combination itself when the carry pair is given: `o_acc` (fp32
 * [batch, hq, n_q, 128], contiguous, 16-byte aligned) and `lse_acc` (fp32 [batch, hq, n_q]) hold the
 * merged, normalised result of the key chunks seen so far and its log-sum-exp.  The caller fills
 * lse_acc with -inf before the first call (o_acc need not be initialised: a row whose lse_acc is
 * -inf is not read); every call folds its keys in, in fp32, and rewrites both.  With a carry `o` may
 * be NULL; when given it receives the merged result rounded to bf16 (pass it with the last key
 * chunk of a query chunk, so the output is rounded once).  Calls that share a carry must be ordered
 * on one stream.  No counterpart in the reference (it has no sequence parallelism).
 */
int minf_sparse_attention_fwd_window(
    const void* q, const void* k, const void* v, void* o, float* lse, float* o_acc, float* lse_acc,
    const int64_t q_strides[3], const int64_t k_strides[3],
    const int64_t v_strides[3], const int64_t o_strides[3],
    int batch, int hq, int hkv, int context_size, int n_q, int q_pos0, int n_kv, int kv_pos0,
    int head_dim, float sm_scale,
    const int32_t* head_mode, const int32_t* head_param,
    const void* plan, const int32_t* vertical_indexes, int cap_v, int cap_s,
    int32_t* status, void* stream);

/*
 * Number of 64x64 tiles the reference kernels would compute for the index set held in a
 * plan (block_count + ceil(column_count/64) summed over row blocks and heads) -- the
 * algorithmic-work figure used for throughput reporting.  tiles_out: uint64 [1], device.
 */
int minf_plan_count_tiles(const void* plan, int batch, int heads, int context_size,
                          int cap_v, int cap_s, unsigned long long* tiles_out, void* stream);
/* The same for a plan built with minf_vs_build_plan_window. */
int minf_plan_count_tiles_window(const void* plan, int batch, int heads, int q_pos0, int n_q,
                                 int cap_v, int cap_s, unsigned long long* tiles_out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MINFER_B200_H */
