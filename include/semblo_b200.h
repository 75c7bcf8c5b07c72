/* C ABI of the B200 (sm_100a) implementation of the semblo sparse-attention hot path.
 *
 * Plain pointers and sizes only; every pointer is a CUDA device pointer unless noted.
 * All buffers are allocated and owned by the caller; no entry point here allocates
 * device memory.  `stream` is a cudaStream_t passed as void*.  Each entry point
 * returns 0 on success or a negative code after host-side validation failed
 * (-1 invalid argument, -2 CUDA error, -3 workspace too small; text from
 * semblo_last_error()).  Device-side conditions (a bounded wait that ran out, a
 * sized buffer that would overflow) are written to the caller's int32 `status`
 * word and never trap: 0 ok, 101-104 wait timed out (load / mma / softmax /
 * epilogue role), 201 overflow.
 *
 * The reference is pure Python (torch + Triton) and has no C ABI of its own; each
 * declaration names the reference function whose device work it replaces
 * (paths relative to the reference checkout).
 */
#ifndef SEMBLO_B200_H_
#define SEMBLO_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { SEMBLO_BF16 = 0, SEMBLO_F32 = 1 };

int semblo_version(void);
const char* semblo_last_error(void);

/* ---- index build -------------------------------------------------------------- */

/* semblo/vllm_plugin/routing_map.py:35-64 (routing_normalize, whole-vector mode) and
 * semblo/inference/flat_index.py:144-166 (routing_space).  x [n_rows, dim] with the given
 * row stride (elements).  out (same dtype, may be NULL) = x / max(|x|, 1e-12) rounded to
 * the dtype; space_f32 / space_bf16 (may be NULL) = the fp32 re-normalisation of `out`.
 * query_mode = 1 gives semblo/vllm_plugin/trivial_router.py:48-75 instead: the second
 * normalisation is rounded to the dtype as well (space_* receive the rounded value).
 * query_mode = 2 takes x as already routed keys and applies the second step only. */
int semblo_routing_normalize(const void* x, int dtype, int64_t n_rows, int dim, int64_t row_stride,
                             void* out, float* space_f32, void* space_bf16, int query_mode,
                             void* stream);

/* Row gather for the k-means sample (semblo/inference/flat_index.py:254, 260-262). */
int semblo_gather_rows(const float* src, const int64_t* idx, int64_t m, int dim, float* dst_f32,
                       void* dst_bf16, void* stream);

/* semblo/inference/flat_index.py:356-382 (_argmax_sim_chunked / assign_flat_buckets):
 * arg-max over centroids of the bf16-rounded fp32-accumulated similarity, lowest id on
 * ties.  x_bf16 [n, dim], cent_bf16 [num_centroids, dim], assign_out [n] = id + id_offset. */
int semblo_assign_argmax(const void* x_bf16, int64_t n, const void* cent_bf16, int num_centroids,
                         int dim, int32_t* assign_out, int id_offset, int32_t* status, void* stream);

/* torch.bincount + the padded / unpadded prefix sums of semblo/vllm_plugin/state.py:44-84
 * and the empty-cluster test of semblo/inference/flat_index.py:270-285.
 * assign [heads, head_stride]; counts [heads, C]; ip_orig / ip_pad [heads, C+1] (ip_pad,
 * empty_rank [heads, C], n_empty [heads] may be NULL). */
int semblo_cluster_counts(const int32_t* assign, int64_t n, int64_t head_stride, int heads,
                          int num_clusters, int align, int32_t* counts, int32_t* ip_orig,
                          int32_t* ip_pad, int32_t* empty_rank, int32_t* n_empty, void* stream);

/* semblo/inference/flat_index.py:271-288: deterministic per-cluster sums (members added in
 * index order), empty clusters restarted on sample[repl[rank]] (repl may be NULL when no
 * cluster is empty), mean, re-normalisation.  ip_orig / empty_rank from
 * semblo_cluster_counts (heads = 1, align = 1). */
int semblo_kmeans_update(const float* sample, const int32_t* assign, int64_t n, int num_clusters,
                         int dim, const int32_t* ip_orig, const int32_t* empty_rank,
                         const int64_t* repl, float* cent_f32, void* cent_bf16, void* workspace,
                         int64_t workspace_bytes, void* stream);

/* The same update in two calls, for a caller that reads n_empty on the host between them: the member
 * lists do not depend on the restart draws, so they can be sorted (semblo_kmeans_sort_members, into
 * `workspace`) while that read is on its way, and semblo_kmeans_update_sorted then takes `repl` and the
 * workspace as the first call left it. */
int semblo_kmeans_sort_members(const int32_t* assign, int64_t n, int num_clusters, void* workspace,
                               int64_t workspace_bytes, void* stream);
int semblo_kmeans_update_sorted(const float* sample, int64_t n, int num_clusters, int dim,
                                const int32_t* ip_orig, const int32_t* empty_rank, const int64_t* repl,
                                float* cent_f32, void* cent_bf16, const void* workspace,
                                int64_t workspace_bytes, void* stream);

/* semblo/vllm_plugin/state.py:877-886: codebooks [2, C, dim/2] (bf16) = halves of
 * normalize(cents); cluster c takes row c - row_offset of cents, zero outside [0, num_rows). */
int semblo_split_descriptor(const float* cents, int num_rows, int row_offset, int num_clusters,
                            int dim, void* codebook_bf16, void* stream);

int64_t semblo_layout_workspace_bytes(int64_t n, int heads);

/* semblo/vllm_plugin/state.py:850-914 (_build_flat tail) with _page_align_order (44-84):
 * assign [heads, n] -> sizes [heads, C] (true), indptr [heads, C+1] (page-aligned starts),
 * posting [heads, posting_stride] (cluster-major, position-ascending; padding and tail rows
 * repeat the first entry), inverse [heads, n] (position -> packed row).
 * workspace >= semblo_layout_workspace_bytes(n, heads) + heads * (C + 1) * 4 bytes. */
int semblo_build_layout(const int32_t* assign, int64_t n, int heads, int num_clusters, int align,
                        int32_t* posting, int64_t posting_stride, int32_t* indptr, int32_t* sizes,
                        int32_t* inverse, void* workspace, int64_t workspace_bytes, void* stream);

/* semblo/vllm_plugin/state.py:950-997 (pack_prompt_kv): packed [2, packed_rows, Hkv, D] from
 * k, v [L, Hkv, D] through posting[:, :width]; rows >= width are zero.  With page_table the
 * packed row r lands in physical 16-row page page_table[r / 16] (a vLLM-style paged pool). */
int semblo_pack_kv(const void* k, const void* v, const int32_t* posting, int64_t posting_stride,
                   int64_t width, int64_t packed_rows, int num_kv_heads, int head_dim, void* packed,
                   int64_t kv_stride_elems, const int32_t* page_table, void* stream);

/* semblo/vllm_plugin/fused_prefill.py:126-135 (CausalSnapshot.advance):
 * sizes[h][c] += |{p in [lo, hi) : assign[h][p] == c}|. */
int semblo_snapshot_advance(const int32_t* assign, int64_t head_stride, int heads, int64_t lo,
                            int64_t hi, int num_clusters, int32_t* sizes, void* stream);

/* ---- prefill selection ---------------------------------------------------------- */

/* semblo/vllm_plugin/fused_select.py:1061-1357 (flat_mixture_scores_qtiled) fused with the
 * score transform of fused_select.py:609-613: score [Q, Hkv, C] fp32 =
 * log(max(sum_t softmax_c(q_t . mu_c / tau), 1e-38)) - beta log(1 + n_c), -3.4e38 where
 * n_c == 0.  vectors [Q, Hq, D] bf16 routing vectors, codebooks [Hkv, 2, C, D/2] bf16,
 * select_sizes [Hkv, C] (the sink cluster already held out by the caller). */
int semblo_score_clusters(const void* vectors_bf16, int num_queries, int num_q_heads, int head_dim,
                          const void* codebooks_bf16, int num_kv_heads, int num_clusters,
                          const int32_t* select_sizes, float temperature, float beta, float* score,
                          int32_t* status, void* stream);

/* semblo/vllm_plugin/fused_select.py:604-647 (_streaming_select_kernel) plus
 * fused_prefill.py:212-216 (_force_sink_bit): the bisected threshold and the packed
 * per-query bitmask qmask [Q, Hkv, C/32]; counts / tokens [Q, Hkv] may be NULL.
 * top1 (no reference counterpart) receives arg max_c of score + tile_key_beta log(1 + n_c), lowest
 * id on ties: with tile_key_beta = the penalty's beta the cluster of the largest mixture
 * probability, with 0 the best-scoring cluster.  The caller sorts queries by it to form tiles. */
int semblo_select_clusters(const float* score, const int32_t* select_sizes, int num_queries,
                           int num_kv_heads, int num_clusters, int target_tokens, int iters,
                           int force_sink, int32_t* qmask, int32_t* counts, int32_t* tokens,
                           int32_t* top1 /* [Hkv, Q] tile-order key, or NULL */, float tile_key_beta,
                           void* stream);

/* Stable arg-sort of small integer keys (keys [heads, n] in [0, max_key), max_key <= 65536):
 * order [heads, n].  Used to put queries with the same best-scoring cluster into the same
 * attention tile; the reference has no counterpart (its kv-outer body gathers queries per
 * cluster instead, semblo/vllm_plugin/kv_outer.py:254-329).
 * workspace >= semblo_layout_workspace_bytes(n, heads). */
int semblo_argsort_keys(const int32_t* keys, int64_t n, int heads, int max_key, int32_t* order,
                        void* workspace, int64_t workspace_bytes, void* stream);

/* ---- keys that arrive after the index was fitted: token-order streamed prefill and suffix flush ---- */

/* _nearest_cluster (semblo/vllm_plugin/suffix_flush.py:154-169, used by
 * token_outer_prefill.py:343-347): for every key of keys [n, Hkv, D] (bf16, unit-normalised
 * routing keys) the cluster whose unit descriptor has the largest fp32 cosine, lowest id on
 * ties; descriptors that are all zero (the sink cluster) are never chosen.  codebooks
 * [Hkv, 2, C, D/2] bf16; ids [Hkv, n]; dead_bits_scratch [Hkv, C/32] u32. */
int semblo_nearest_cluster(const void* keys_bf16, int64_t n, int num_kv_heads, int head_dim,
                           const void* codebooks, int num_clusters, int32_t* ids_out,
                           uint32_t* dead_bits_scratch, int32_t* status, void* stream);

/* append_rows (token_outer_prefill.py:66-87): ids [heads, n] in position order ->
 * rows[h, i] = indptr[h, id] + sizes[h, id] + (earlier keys of the slice with the same id) and
 * counts [heads, C].  workspace >= semblo_layout_workspace_bytes(n, heads) + heads * (C + 1) * 4. */
int semblo_append_rows(const int32_t* ids, int64_t n, int heads, int num_clusters, const int32_t* indptr,
                       const int32_t* sizes, int32_t* rows, int32_t* counts, void* workspace,
                       int64_t workspace_bytes, void* stream);

/* The index_copy_ calls of _append / _fit_and_pack (token_outer_prefill.py:296-309, 354-358):
 * k, v [n, Hkv, D] of consecutive tokens go to rows[h, i] of packed [2, packed_rows, Hkv, D]
 * (through page_table when given), posting[h, row] = positions[i], inverse[h, inverse_offset + i]
 * = row; posting / inverse may be NULL.  A row outside the store sets status 201 and is skipped. */
int semblo_scatter_kv(const void* k, const void* v, const int32_t* positions, int64_t n, int num_kv_heads,
                      int head_dim, const int32_t* rows, int64_t rows_stride, void* packed,
                      int64_t packed_rows, int64_t kv_stride_elems, int32_t* posting, int64_t posting_stride,
                      int32_t* inverse, int64_t inverse_stride, int64_t inverse_offset,
                      const int32_t* page_table, int32_t* status, void* stream);

/* The opposite direction (reads through the inverse map: the local window and the dense start
 * of the streamed mode, fused_prefill.py:155-189; the clone in _repack, token_outer_prefill.py:381):
 * out_k / out_v [n, Hkv, D] = packed rows rows[h, i]. */
int semblo_gather_kv(const void* packed, int64_t kv_stride_elems, const int32_t* rows, int64_t rows_stride,
                     int64_t n, int num_kv_heads, int head_dim, void* out_k, void* out_v,
                     const int32_t* page_table, void* stream);

/* Rows after the cluster runs moved (token_outer_prefill.py:282-287, 375-379):
 * new[h, i] = old[h, i] - old_indptr[h, b] + new_indptr[h, b] with b = bucket[h, i]. */
int semblo_relayout_rows(const int32_t* rows_old, const int32_t* bucket, int64_t n, int64_t stride, int heads,
                         const int32_t* old_indptr, const int32_t* new_indptr, int num_clusters,
                         int32_t* rows_new, void* stream);

/* repack_apply (suffix_flush.py:97-133) for all heads: n flushed tokens (flushed_k / flushed_v
 * [n, Hkv, D], positions, assign [Hkv, n] in position order) follow each cluster's old rows, every
 * cluster is re-padded to `align`, padding rows repeat the old row 0; packed, posting, sizes and
 * indptr are rewritten in place.  old_packed_copy [2, packed_rows, Hkv, D] and old_posting_copy
 * [Hkv, packed_rows] are scratch for the old store (posting_stride must equal packed_rows). */
int64_t semblo_flush_workspace_bytes(int64_t n, int heads, int num_clusters);
int semblo_flush_repack(void* packed, int64_t kv_stride_elems, int64_t packed_rows, int32_t* posting,
                        int64_t posting_stride, int32_t* sizes, int32_t* indptr, int num_clusters,
                        int num_kv_heads, int head_dim, int align, const void* flushed_k,
                        const void* flushed_v, const int32_t* flushed_pos, const int32_t* assign, int64_t n,
                        void* old_packed_copy, int32_t* old_posting_copy, void* workspace,
                        int64_t workspace_bytes, int32_t* status, void* stream);

/* semblo_argsort_keys without a workspace and without any allocation: the scratch is a fixed
 * array inside the library image, looked up once per device.  No counterpart in the reference.
 * For callers that must not allocate at the point of the call (inside a serving loop that has
 * frozen its memory pool, or under an allocator they do not own).  Limits: heads * n <=
 * semblo_argsort_keys_static_max_keys() (65536) and heads <= 64; larger inputs are refused
 * with an error and belong to semblo_argsort_keys.  The first call on a device, with that
 * device current, resolves the array's address (this may load the module).  All calls on a
 * device share the one array, so two calls whose kernels can overlap (different streams or
 * threads) race; order them on one stream.  Nothing in the array has to be cleared between
 * calls. */
int64_t semblo_argsort_keys_static_max_keys(void);
int semblo_argsort_keys_static(const int32_t* keys, int64_t n, int heads, int max_key,
                               int32_t* order, void* stream);

/* ---- prefill attention ---------------------------------------------------------- */

/* semblo/vllm_plugin/fused_prefill.py:155-189 (_dense_chunk_attention) and the chunk's own
 * causal window of semblo/vllm_plugin/kv_outer.py:661-676: every query attends positions
 * [local_start, q_position] of the position-ordered K/V, exactly causally.
 * q, out [Q, Hq, D] bf16 (consecutive queries); q_positions [Q]; ordered_k / ordered_v
 * [ordered_rows, Hkv, D] hold positions ordered_pos0 ...; lse [Q, Hq] (natural log) and
 * attended (sum over (query, KV head) of attended keys, accumulated) may be NULL.
 * partial_out [Q, Hq, D] fp32 (may be NULL): when given, the normalised result goes there
 * instead of `out`, for semblo_sparse_prefill_gather to merge without a bf16 rounding. */
int semblo_window_prefill(const void* q, int num_queries, int num_q_heads, int num_kv_heads,
                          int head_dim, const int32_t* q_positions, const void* ordered_k,
                          const void* ordered_v, int64_t ordered_rows, int ordered_pos0,
                          int local_start, float sm_scale, void* out, float* partial_out, float* lse,
                          unsigned long long* attended, int32_t* status, void* stream);

/* The sparse part of semblo/vllm_plugin/kv_outer.py:482-816 with row-granular reads: for every
 * query, attention over rows [indptr[c], indptr[c] + causal_sizes[c]) of the clusters set in
 * its qmask, gathered row by row from the cluster-ordered K/V (packed_k / packed_v
 * [packed_rows, Hkv, D]; page_table optional).  Tiles of 128 / G queries are formed in q_order
 * ([Hkv, Q], optional).  merge = 1: partial_in (fp32; or `out` as bf16 when partial_in is
 * NULL) and `lse` hold the window partial written by semblo_window_prefill (normalised
 * output, natural-log LSE); `out` / `lse` receive the LSE-merged
 * result (kv_outer.py:203-227); merge = 0: the sparse result alone.  attended (may be NULL)
 * points at two counters: [0] += attended keys summed over (query, KV head), [1] += K/V rows
 * gathered summed over tiles (the union each tile actually reads).  cta_order (optional,
 * [tiles * Hkv] from semblo_gather_launch_order): the (tile, head) pairs in the order their
 * CTAs should start; it changes the schedule only, not the result. */
int semblo_sparse_prefill_gather(const void* q, int num_queries, int num_q_heads, int num_kv_heads,
                                 int head_dim, const int32_t* q_order, const int32_t* cta_order,
                                 const void* packed_k, const void* packed_v, int64_t packed_rows,
                                 const int32_t* page_table,
                                 const int32_t* qmask, const int32_t* causal_sizes,
                                 const int32_t* indptr, int num_clusters, float sm_scale, int merge,
                                 const float* partial_in, void* out, float* lse,
                                 unsigned long long* attended,
                                 int32_t* status, void* stream);

/* Launch order for semblo_sparse_prefill_gather: the rows each (tile, head) will gather (the
 * union of the tile's selections; tiles of 128 / G queries in q_order) go to work
 * [tiles * Hkv], and order_out [tiles * Hkv] lists tile * Hkv + head one KV head after the
 * other, each head's pairs by descending work: CTAs that run together gather from one head's
 * rows (a working set the L2 holds) and the longest start first.  No reference counterpart (the
 * reference's kernels are scheduled by Triton's grid order). */
int semblo_gather_launch_order(const int32_t* q_order, const int32_t* qmask,
                               const int32_t* causal_sizes, int num_queries, int num_q_heads,
                               int num_kv_heads, int num_clusters, int32_t* work,
                               int32_t* order_out, void* stream);

/* ---- decode ----------------------------------------------------------------------- */

int64_t semblo_decode_workspace_bytes(int num_q_heads, int num_kv_heads, int head_dim,
                                      int num_clusters, int64_t packed_width, int num_splits);

/* Byte offsets of the workspace members, in order: tickets, logit [Hkv, G, C] f32,
 * block (max, sum) partials, split records [Hkv, splits, 4] i32 (CSR entry, offset inside it, selected
 * rows, selected clusters),
 * rstart, rlen, rcum [Hkv, C] i32 (the CSR of fused_decode.py:189-199), rcount, rtokens [Hkv] i32,
 * pacc, pml, vectors [Hq, D] bf16.  The workspace must be zeroed once before its first use. */
int semblo_decode_workspace_offsets(int num_q_heads, int num_kv_heads, int head_dim,
                                    int num_clusters, int64_t packed_width, int num_splits,
                                    int64_t* offsets /* host, [12] */);

/* semblo/vllm_plugin/fused_decode.py:393-521 (fused_decode_step): the whole decode step of
 * one layer over the decode arena (semblo/vllm_plugin/arena.py:66-253): suffix write at
 * positions[0] through the block table, query router, selection over the full sizes with
 * the sink rule, attention over the selected rows with posting <= position plus the
 * suffix positions [prompt_length, position], merged into output [Hq * D] bf16.
 * k_post / v_new / k_pre [Hkv, D] may be NULL (layers sharing another layer's K/V).
 * stage_mask: bit 0 score + suffix write, bit 1 select, bit 2 attend + merge (7 = all); bit 3
 * set: every stage is launched strictly after the one before it (without it the select and
 * attend kernels are programmatic dependent launches that start while their predecessor drains
 * and wait for it before reading its results).  1 <= iters <= 16, num_clusters a multiple of 32
 * up to 16384. */
int semblo_decode_step(const void* q_post, const void* q_pre, const void* k_post, const void* v_new,
                       const void* k_pre, const void* positions, int pos_is_int64,
                       const void* codebooks, const int32_t* sizes, const int32_t* indptr,
                       const int32_t* posting, const void* packed_kv, int64_t packed_width,
                       void* suffix_kv, void* suffix_kpre, const int32_t* suffix_table,
                       int suffix_blocks, int suffix_block, int table_len,
                       const int32_t* prompt_length, int num_q_heads, int num_kv_heads,
                       int head_dim, int num_clusters, float temperature, float beta,
                       int target_tokens, int sink_tokens, int iters, float sm_scale, int num_splits,
                       void* workspace, int64_t workspace_bytes, void* output, int32_t* status,
                       int stage_mask, float* lse_out /* [Hq] natural-log LSE of the result, or NULL */,
                       int flags /* bit 0: q_pre already holds the routing vectors */, void* stream);

/* semblo/vllm_plugin/paged_attention.py:961-1128 (paged_posting_attention) for one query:
 * attention over the positions listed by posting tiles (tile k of KV head h covers
 * posting_positions[h, tile_starts[h, k] + (0 .. tile_lengths[h, k]))), each kept only if it is at or
 * before the query's position, read from a vLLM-style paged cache [2, blocks, block_size, Hkv, D]
 * through block_table [block_table_len].  Writes output [Hq, D] bf16 and, if lse_out is given, the
 * natural-log log-sum-exp [Hq].  No logit soft cap.  The workspace (size from
 * semblo_paged_attention_workspace_bytes) must be zeroed once before its first use. */
int64_t semblo_paged_attention_workspace_bytes(int num_q_heads, int num_kv_heads, int head_dim,
                                               int num_splits);
int semblo_paged_posting_attention(const void* q, const void* q_position, int pos_is_int64,
                                   const void* kv_cache, int64_t cache_blocks, int block_size,
                                   const int32_t* block_table, int block_table_len,
                                   const int32_t* posting_positions, int64_t posting_stride,
                                   const int32_t* tile_starts, const int32_t* tile_lengths,
                                   const int32_t* tile_counts, int tile_stride, int token_tile,
                                   int num_q_heads, int num_kv_heads, int head_dim, float sm_scale,
                                   int num_splits, void* workspace, int64_t workspace_bytes,
                                   void* output, float* lse_out, int32_t* status, void* stream);

/* semblo/vllm_plugin/paged_attention.py:50-78 (merge_paged_attention_results): exact merge of two
 * attention states computed over disjoint key sets; out_* [rows, head_dim] bf16, lse_* [rows] fp32
 * (natural log, -inf for an empty state). */
int semblo_merge_attention_states(const void* out_a, const float* lse_a, const void* out_b,
                                  const float* lse_b, int64_t rows, int head_dim, void* out,
                                  float* lse, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SEMBLO_B200_H_ */
