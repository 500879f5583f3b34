/*
 * libftk_sm100 -- C ABI of the B200 (sm_100a) flash_topk_attn_v2 hot path.
 *
 * One entry point per native launch of the reference project; each comment
 * names the reference interface it replaces (paths inside that project).
 *
 * Conventions
 *   - All pointers are DEVICE pointers unless a name ends in `_host`.
 *   - The caller owns every buffer (inputs, outputs, workspace); the library
 *     allocates nothing and keeps no state between calls.  The one exception
 *     is ftk_build_reverse_noalloc (see there): its scratch is an array inside
 *     the library that every call shares, and it caches that array's device
 *     address per device ordinal.
 *   - Work is enqueued on `stream` (a cudaStream_t passed as void*; NULL is
 *     the legacy default stream) and the call returns without synchronising.
 *   - Return value: FTK_OK or a negative FTK_ERR_* code; nothing is launched
 *     when an argument check fails.  Device-side problems (a bounded wait
 *     that ran out, an out-of-range block id) are reported asynchronously in
 *     `*status` (device int32, see FTK_DEV_*).  The word is sticky: the
 *     library only ever writes it on a failure and the first failure wins, so
 *     the caller zeroes it once and may read it after any number of calls.
 *     `status` may be NULL.
 *   - q/k/v/o/do/dq/dk/dv are 16-bit tensors (`dtype`: FTK_F16 or FTK_BF16)
 *     addressed as element [b][n][h][d] with element strides (s*_b, s*_n,
 *     s*_h) and unit stride along d, so both the [B,N,H*D] and the [B,H,N,D]
 *     layouts of the reference API are accepted in place.  Base pointers must
 *     be 16-byte aligned and strides multiples of 8 elements.
 *   - Index tensors are int32, scores fp32, contiguous, in the reference's
 *     shapes.
 */
#ifndef FTK_API_H_
#define FTK_API_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FTK_OK 0
#define FTK_ERR_BAD_ARG (-1)      /* shape / alignment / range check failed   */
#define FTK_ERR_UNSUPPORTED (-2)  /* legal in the reference, not built here   */
#define FTK_ERR_WORKSPACE (-3)    /* workspace pointer NULL or too small      */
#define FTK_ERR_CUDA (-4)         /* a CUDA runtime call or launch failed     */
#define FTK_ERR_DRIVER (-5)       /* tensor-map encoding unavailable / failed */
#define FTK_ERR_CAPACITY (-6)     /* problem larger than a fixed built-in buffer */

#define FTK_DEV_TIMEOUT_TMA 101
#define FTK_DEV_TIMEOUT_MMA 102
#define FTK_DEV_TIMEOUT_CONSUMER 103
#define FTK_DEV_TIMEOUT_EPILOGUE 104
#define FTK_DEV_BAD_INDEX 105

#define FTK_F16 0
#define FTK_BF16 1

/* Library version (major*10000 + minor*100 + patch). */
int ftk_version(void);
/* Static, human-readable text for a return code or a device status code. */
const char* ftk_error_string(int code);

/* ---------------------------------------------------------------- scoring
 * Replaces block_score_launch (flash_topk_attn_v2/csrc/block_score.cpp:3-11,
 * csrc/block_score_kernel.cu:414) together with the permute/pad/alloc done in
 * flash_block_score_cuda (flash_topk_attn_v2/block_score_cuda.py:45-164).
 *
 * For (batch*head) slices [bh_begin, bh_begin + bh_count) writes the softmax
 * mass of every query over every score block, block_scores[slice][n][m],
 * m < M = (pad_head + N + pad_tail) / score_block_size, rows summing to 1.
 * Logits are `scale` * q.k (the reference always uses 1/sqrt(D) of the
 * unpadded head dim, block_score_cuda.py:148).  D is 64, 128 or 256 (the host
 * layer zero-pads other head dims up); score_block_size a multiple of 16.
 * `block_scores` points at slice bh_begin.  Workspace: ftk_block_score_workspace.
 */
size_t ftk_block_score_workspace(int64_t bh_count, int64_t N);
int ftk_block_score(const void* q, const void* k, int dtype, int64_t B, int64_t H, int64_t N,
                    int64_t D, int64_t sq_b, int64_t sq_n, int64_t sq_h, int64_t sk_b,
                    int64_t sk_n, int64_t sk_h, int64_t bh_begin, int64_t bh_count,
                    int score_block_size, int pad_head, int pad_tail, float scale,
                    float* block_scores, void* workspace, size_t workspace_bytes,
                    int32_t* status, void* stream);

/* Replaces topk_select_launch (csrc/topk_select.cpp:3-11,
 * csrc/topk_select_kernel.cu:142) and the Triton select kernel
 * (flash_topk_attn_v2/topk_select.py:28-125).
 *
 * rows x M fp32 block scores -> rows x M_out (idx, raw, avg), M_out =
 * min(max_topk, M) (max_topk == 0: M).  `row_scale` (optional, may be NULL)
 * holds one divisor per row applied to the scores first (used by the fused
 * scoring path whose scratch holds unnormalised sums).  Equal averages keep
 * the lower block id first.  M <= 4096.
 */
int ftk_topk_select(const float* block_scores, const float* row_scale, int64_t rows, int M,
                    int max_topk, int score_block_size, int pad_head, int pad_tail,
                    float threshold, int32_t* topk_idx, float* topk_raw, float* topk_avg,
                    int32_t* status, void* stream);

/* flash_topk_score in one call (flash_topk_attn_v2/__init__.py:16-54): scoring
 * followed by select for slices [bh_begin, bh_begin+bh_count); the [N, M]
 * score matrix only ever lives in `workspace` (ftk_score_topk_workspace).
 * Outputs point at slice bh_begin and are [slice][n][M_out].
 */
size_t ftk_score_topk_workspace(int64_t bh_count, int64_t N, int64_t M);
int ftk_score_topk(const void* q, const void* k, int dtype, int64_t B, int64_t H, int64_t N,
                   int64_t D, int64_t sq_b, int64_t sq_n, int64_t sq_h, int64_t sk_b, int64_t sk_n,
                   int64_t sk_h, int64_t bh_begin, int64_t bh_count, int score_block_size,
                   int pad_head, int pad_tail, float scale, int topk, float threshold,
                   int32_t* topk_idx, float* topk_raw, float* topk_avg, void* workspace,
                   size_t workspace_bytes, int32_t* status, void* stream);

/* ------------------------------------------------------------------ merge
 * Replaces qblock_merge_launch (csrc/qblock_merge.cpp:3-10,
 * csrc/qblock_merge_kernel.cu:100) plus the padding / unit-score / counts glue
 * of build_qblock_topk_indices (flash_topk_attn_v2/__init__.py:57-133).
 *
 * topk_idx [BH][N][K] (and topk_scores, or NULL for weight 1 per valid entry)
 * are aggregated per q-block of `q_block_size` virtual rows starting at
 * -q_pad_head; QM = (q_pad_head + N + q_pad_tail) / q_block_size.  Output
 * rows [BH][QM][qblock_topk]: blocks with positive aggregate, by aggregate
 * descending (ties: lower id), padded with (-1, 0.0); counts [BH][QM].
 * Aggregation is an fp32 sum in (row, rank) order, so results are
 * reproducible bit for bit.  num_score_blocks <= 4096.
 */
int ftk_qblock_merge(const int32_t* topk_idx, const float* topk_scores, int64_t BH, int64_t N,
                     int K, int q_block_size, int q_pad_head, int q_pad_tail,
                     int num_score_blocks, int qblock_topk, int32_t* merged_idx,
                     float* merged_scores, int32_t* counts, int32_t* status, void* stream);

/* Exact union, ascending by block id: replaces the first-generation
 * build_qblock_topk_indices (flash_topk_attn/attention.py:70-138 and its
 * kernel :23-67).  topk_idx [BH][N][K] (-1 = empty slot); output rows
 * [BH][QM][width]: the distinct ids picked by the q-block's real rows in
 * ascending order, then -1; counts [BH][QM].  width >= min(q_block_size * K,
 * num_score_blocks) always holds the whole union (the reference uses
 * next_pow2(q_block_size * K)); a longer union is cut at `width` and reported
 * through `status`.  num_score_blocks <= 65536. */
int ftk_qblock_union(const int32_t* topk_idx, int64_t BH, int64_t N, int K, int q_block_size,
                     int q_pad_head, int q_pad_tail, int num_score_blocks, int width,
                     int32_t* merged_idx, int32_t* counts, int32_t* status, void* stream);

/* Largest valid id + 1 over an int32 array (device result, int32, >= 1):
 * the `indices.max().item() + 1` of flash_topk_attn_v2/__init__.py:101-105
 * without the host round trip. */
int ftk_max_index_plus1(const int32_t* idx, int64_t count, int32_t* result, void* stream);

/* Replaces build_reverse_indices_launch (csrc/build_reverse_indices.cpp:3-10,
 * csrc/build_reverse_indices_kernel.cu:71): reverse_idx [BH][M][QM] (-1
 * padded; q-blocks in ascending order), reverse_counts [BH][M],
 * sorted_kv [BH][M] = kv blocks by count descending (ties: lower id), the
 * order in which ftk_sparse_bwd_dkv issues its tiles when it is given it.
 * `counts` may be NULL (rows are then read to their full width W; -1 entries
 * are skipped either way).  sorted_kv may be NULL; with it M <= 8192 (the
 * reference stops at 1024).  Workspace: ftk_build_reverse_workspace. */
size_t ftk_build_reverse_workspace(int64_t BH, int QM, int M);
int ftk_build_reverse(const int32_t* merged_idx, const int32_t* counts, int64_t BH, int QM,
                      int W, int M, int32_t* reverse_idx, int32_t* reverse_counts,
                      int32_t* sorted_kv, void* workspace, size_t workspace_bytes,
                      int32_t* status, void* stream);

/* No counterpart in the reference.  ftk_build_reverse for callers that cannot
 * allocate device memory where they call it (inside an allocator callback, in
 * a plugin that is only handed input and output buffers, in a loop that must
 * never enter the allocator): same inputs, outputs and results, but the
 * membership bitmap lives in a fixed 4 MiB array inside the library image
 * (present on every GPU that loads the library until the process exits), so
 * there is no workspace argument and nothing is allocated or freed.
 * Limit: BH * M * ceil(QM / 32) * 4 bytes <= ftk_build_reverse_noalloc_capacity();
 * beyond it the call returns FTK_ERR_CAPACITY and launches nothing -- use
 * ftk_build_reverse.  The first call on each device looks up the array's
 * device address (cudaGetSymbolAddress, with that device current); make that
 * call before any stream capture begins.  All calls share the one array, which
 * is cleared on `stream` at the start of each call: calls whose GPU work can
 * overlap (other streams, other threads) race and must be serialised by the
 * caller.  The cached address is kept per device ordinal and belongs to the
 * device's primary context (the one the runtime API and PyTorch use): it is
 * not refreshed after cudaDeviceReset and does not follow a caller that
 * switches between driver-API contexts on one device. */
size_t ftk_build_reverse_noalloc_capacity(void);
int ftk_build_reverse_noalloc(const int32_t* merged_idx, const int32_t* counts, int64_t BH,
                              int QM, int W, int M, int32_t* reverse_idx,
                              int32_t* reverse_counts, int32_t* sorted_kv, int32_t* status,
                              void* stream);

/* Replaces sort_by_count_launch (csrc/sort_by_count.cpp:3-9,
 * csrc/sort_by_count_kernel.cu:12): global stable descending sort of `total`
 * counts with their flat ids.  `max_count` bounds every count from above (the
 * reference derives its radix width from the maximum the same way,
 * flash_topk_attn_v2/sort_by_count_cuda.py:55-56).
 * Workspace: ftk_sort_by_count_workspace. */
size_t ftk_sort_by_count_workspace(int64_t total, int max_count);
int ftk_sort_by_count(const int32_t* counts, int64_t total, int max_count,
                      int32_t* sorted_counts, int32_t* sorted_ids, void* workspace,
                      size_t workspace_bytes, void* stream);

/* -------------------------------------------------------- sparse attention
 * Replaces sparse_attn_fwd_launch (csrc/sparse_attn.cpp:3-12,
 * csrc/sparse_attn_kernel.cu:368).  merged_idx [B*H][QM][W]; for every real
 * query row of q-block m attends to the tokens of the blocks listed in the
 * valid prefix of its row.  o in `dtype` with strides (so_*), lse fp32
 * [B*H][N] (natural log; -inf and o = 0 for an empty list).  k and v carry Hkv
 * heads (Hkv <= 0 means H; H must be a multiple): query head h reads kv head
 * h / (H / Hkv).  The reference rejects Hkv != H (__init__.py:153-156).
 * `workspace` (ftk_sparse_fwd_workspace bytes, may be NULL) enables the
 * pipelined kernel for 64-row kv blocks and q-blocks of 64 or 32 rows (bf16 or fp16):
 * it uses one fixed reference exponent per row, and the exact running-maximum
 * kernel, launched behind it, recomputes the tiles whose scores left the safe
 * exponent range (none on ordinary inputs).  Without a workspace only the
 * exact kernel runs.  Setting the environment variable FTK_FWD_PIPE=0 does the
 * same.  At head dim 128 the pipelined kernel runs on pairs of SMs (clusters of
 * two CTAs, tcgen05 cta_group::2); FTK_FWD_2CTA=0 selects the one-CTA form.
 * Head dim 256 (D is 64, 128 or 256) runs the exact kernel with one shared
 * output accumulator (dK / dV: one launch for dV, one for dK);
 * ftk_sparse_bwd_dq and ftk_sparse_bwd_dkv then take kv
 * blocks (dq) and q blocks (dkv) of at most 32 rows and return
 * FTK_ERR_UNSUPPORTED otherwise: the host layer restates longer blocks over
 * 32-row halves first. */
size_t ftk_sparse_fwd_workspace(int64_t B, int64_t H, int QM, int q_block_size);
int ftk_sparse_fwd(const void* q, const void* k, const void* v, int dtype, int64_t B, int64_t H, int64_t Hkv,
                   int64_t N, int64_t D, int64_t sq_b, int64_t sq_n, int64_t sq_h, int64_t sk_b,
                   int64_t sk_n, int64_t sk_h, int64_t sv_b, int64_t sv_n, int64_t sv_h,
                   const int32_t* merged_idx, int QM, int W, int q_block_size, int kv_block_size,
                   int q_pad_head, int kv_pad_head, float scale, void* o, int64_t so_b,
                   int64_t so_n, int64_t so_h, float* lse, void* workspace, size_t workspace_bytes,
                   int32_t* status, void* stream);

/* Replaces preprocess_delta (flash_topk_attn_v2/sparse_attn_bwd.py:12-33) and
 * sparse_attn_bwd_dq_launch (csrc/sparse_attn_bwd_dq.cpp:3-15,
 * csrc/sparse_attn_bwd_dq_kernel.cu:422): delta[bh][n] = sum_d o*do (fp32),
 * then dq for every q-block.  `delta` is an output the dK/dV call reuses. */
/* Head dim 128 with 64-row q and kv blocks runs on pairs of SMs (clusters of two
 * CTAs, tcgen05 cta_group::2) in both backward calls; FTK_DQ_2CTA=0 and
 * FTK_DKV_2CTA=0 select the one-CTA kernels that serve every other shape. */
int ftk_sparse_bwd_dq(const void* q, const void* k, const void* v, const void* o, const void* dout,
                      int dtype, int64_t B, int64_t H, int64_t Hkv, int64_t N, int64_t D, int64_t sq_b,
                      int64_t sq_n, int64_t sq_h, int64_t sk_b, int64_t sk_n, int64_t sk_h,
                      int64_t sv_b, int64_t sv_n, int64_t sv_h, int64_t so_b, int64_t so_n,
                      int64_t so_h, int64_t sdo_b, int64_t sdo_n, int64_t sdo_h,
                      const int32_t* merged_idx, int QM, int W, int q_block_size,
                      int kv_block_size, int q_pad_head, int kv_pad_head, float scale,
                      const float* lse, float* delta, void* dq, int64_t sdq_b, int64_t sdq_n,
                      int64_t sdq_h, int32_t* status, void* stream);

/* Replaces sparse_attn_bwd_dkv_launch (csrc/sparse_attn_bwd_dkv.cpp:3-16,
 * csrc/sparse_attn_bwd_dkv_kernel.cu:438): dk, dv per kv block from the
 * reverse index (one writer per kv row, no atomics).  With Hkv < H, dk and dv are
 * still written per QUERY head ([b][n][H][d] through the strides given): the
 * caller sums the H / Hkv heads of a group.  `fwd_list_width` is the
 * width W of the merged_idx lists the reverse index was built from (0 if
 * unknown); it only helps to choose between the kernel on pairs of SMs (lists
 * that can cover a good part of the blocks: 4 W >= M) and the one-CTA kernel.
 * `sorted_kv` (may be NULL: block order) is the kv-block order of
 * ftk_build_reverse; the one-CTA kernels issue their tiles in that order,
 * heaviest first, as the reference's kernel does
 * (csrc/sparse_attn_bwd_dkv_kernel.cu:43); FTK_DKV_ORDER=0 ignores it.  The
 * result does not depend on the order.
 * Block sizes: kv_block_size a multiple of 16 up to 64 in all three attention
 * calls (the forward takes up to 128), q_block_size a multiple of 16 up to 64
 * here (any size up to 128 in the forward, up to 64 in dq); the reference takes
 * any q block of 1..64 rows and any kv block.  Other sizes return
 * FTK_ERR_UNSUPPORTED. */
int ftk_sparse_bwd_dkv(const void* q, const void* k, const void* v, const void* dout, int dtype,
                       int64_t B, int64_t H, int64_t Hkv, int64_t N, int64_t D, int64_t sq_b, int64_t sq_n,
                       int64_t sq_h, int64_t sk_b, int64_t sk_n, int64_t sk_h, int64_t sv_b,
                       int64_t sv_n, int64_t sv_h, int64_t sdo_b, int64_t sdo_n, int64_t sdo_h,
                       const int32_t* reverse_idx, const int32_t* reverse_counts,
                       const int32_t* sorted_kv, int QM, int M, int q_block_size,
                       int kv_block_size, int q_pad_head, int kv_pad_head, float scale,
                       const float* lse, const float* delta, void* dk, int64_t sdk_b,
                       int64_t sdk_n, int64_t sdk_h, void* dv, int64_t sdv_b, int64_t sdv_n,
                       int64_t sdv_h, int fwd_list_width, int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FTK_API_H_ */
