/*
 * hils_b200 -- C ABI of the B200 (sm_100a) HiLS sparse-attention kernels.
 *
 * Every entry point takes plain device pointers, sizes and scalars; no torch types cross this
 * boundary.  All tensors are dense row-major in the reference's layouts:
 *     q (B, L, h_q, D)   k, v (B, T, h_kv, D)   chunk keys (B, N, h, D)
 *     indices (B, L, h_kv, K) int32   weights (B, L, h_q, num_weights)
 * `dtype` selects the element type of the activation tensors (HILS_BF16 or HILS_F32); all
 * arithmetic accumulates in fp32.  `stream` is a cudaStream_t passed as void*.  Calls enqueue
 * work on that stream and return without synchronising.  Every tensor must start on a 16-byte
 * boundary (the kernels read rows with 8- and 16-byte vector loads and through TMA descriptors);
 * the sparse-attention entry points verify it and return HILS_ERR_BAD_ARG, the Python host layer
 * verifies it for every call before anything is launched.
 *
 * Return value: 0 on success, a negative HILS_ERR_* code on an argument or launch error
 * (hils_last_error() gives the text).  The library never allocates device memory; kernels that
 * need scratch take a caller-provided workspace whose size the matching *_workspace_bytes()
 * function returns.
 *
 * Each declaration names the reference interface (file:line within the reference project) that
 * the entry point replaces.
 */
#ifndef HILS_B200_H
#define HILS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HILS_F32 0
#define HILS_BF16 1

#define HILS_OK 0
#define HILS_ERR_BAD_ARG (-1)
#define HILS_ERR_UNSUPPORTED (-2)
#define HILS_ERR_CUDA (-3)
#define HILS_ERR_WORKSPACE (-4)

/* Library identification and the text of the last error raised on the calling thread. */
int hils_version(void);
const char* hils_last_error(void);

/* Device-side error word: kernels whose bounded waits (mbarrier polls of the tensor-core paths)
 * expire record a non-zero code here and return instead of spinning.  This call synchronises the
 * device, returns the word (0 = no error, -1 = the synchronisation itself failed) and clears it.
 * The reference has no counterpart (its kernels have no device-side waits). */
int hils_take_device_status(void);

/* ---------------------------------------------------------------------------------------
 * Chunk pooling.  Replaces ChunkAttnPoolFunction.forward/backward and the kernels behind it
 * (ops/chunk_attn_pool_tilelang.py:540-602, kernels :329-533) and the GQA-aware contract of
 * chunk_attn_pool (models/FlashHiLS/hils_attention.py:66-135).
 *   mu_q (B,N,h_q,D); k: token rows of chunk n start at k + b*k_batch_stride + n*S*h_kv*D
 *   (so a (B,T,h_kv,D) cache can be pooled in place); h_q = G*h_kv.
 *   lmk_k (B,N,h_q,D) in `dtype`, lmk_b (B,N,h_q) fp32.  compact != 0: lmk_k is written as 0.
 * Backward recomputes the softmax; g_lmk_k / g_lmk_b may be NULL (treated as zero).
 *   d_mu_q (B,N,h_q,D), d_k (B,N,S,h_kv,D) dense, both in `dtype` (summed over the GQA group).
 * ------------------------------------------------------------------------------------- */
int hils_pool_fwd(const void* mu_q, const void* k, void* lmk_k, float* lmk_b,
                  int B, int N, int S, int h_q, int h_kv, int D, int64_t k_batch_stride,
                  float sm_scale, int compact, int dtype, void* stream);
int hils_pool_bwd(const void* mu_q, const void* k, const void* g_lmk_k, const float* g_lmk_b,
                  void* d_mu_q, void* d_k,
                  int B, int N, int S, int h_q, int h_kv, int D, int64_t k_batch_stride,
                  float sm_scale, int compact, int dtype, void* stream);

/* Mean pooling of each chunk (the `.mean(dim=2)` of models/FlashHiLS/hils_attention.py:445-446,
 * 458-462) and its gradient.  out (B,N,h_kv,D); d_k (B,N,S,h_kv,D) dense. */
int hils_meanpool_fwd(const void* k, void* out, int B, int N, int S, int h_kv, int D,
                      int64_t k_batch_stride, int dtype, void* stream);
int hils_meanpool_bwd(const void* g_out, void* d_k, int B, int N, int S, int h_kv, int D,
                      int dtype, void* stream);

/* ---------------------------------------------------------------------------------------
 * Chunk selection.  Replaces SoftmaxTopKMaxPoolingFusedFn.forward (ops/topk_head_softmax.py:
 * 977-1038: hils_lse_kernel :192, torch.logaddexp :1019, weighted_select_kernel :438,
 * sort_topk_indices_kernel :870, recompute_topk_max_pooling_scores_kernel :669) in one launch.
 *   q (B,L,h_kv,G,D); lmks (B,N,h_kv,D) or, per_qhead != 0, (B,N,h_kv*G,D); both in `dtype`.
 *   lse_swa (B,L,h_kv*G) in lse_dtype; bias (B,N,h_kv,G) fp32 or NULL; gumbel (h_kv*G, N) fp32
 *   or NULL; drop_mask (B,L,N) int32 or NULL.
 *   indices (B,L,h_kv,topk) int32 ascending, -1 padded; scores (B,L,h_kv*G,topk) in `dtype`
 *   (= fl(scale*q.k'), -inf at -1).
 *   Optional fp32 diagnostics (NULL to skip): lse_total (B,L,h_kv,G); rank_keys (B,L,h_kv,N) =
 *   the value the selector ranked, -inf for non-candidates.
 * q_offset is a host scalar (the reference builds a 1-element tensor from a Python int, :1199).
 * ------------------------------------------------------------------------------------- */
int hils_topk_fwd(const void* q, const void* lmks, const void* lse_swa, const float* bias,
                  const float* gumbel, const int32_t* drop_mask,
                  int32_t* indices, void* scores, float* lse_total, float* rank_keys,
                  int B, int L, int N, int h_kv, int G, int D, int topk,
                  int block_size, int window_size, int is_causal, int q_offset, int per_qhead,
                  float sm_scale, int dtype, int lse_dtype,
                  void* workspace, size_t workspace_bytes, void* stream);
/* Scratch of hils_topk_fwd: non-zero only for the bf16 decode shape (L <= 4 query rows, N >= 512), where
 * one kernel streams the chunk keys at memory speed into an fp32 array of raw dot products and a second
 * one selects from it.  workspace may be NULL (or too small): the selection kernel then reads the keys
 * itself. */
size_t hils_topk_fwd_workspace_bytes(int B, int L, int N, int h_kv, int G, int D, int dtype);

/* Gradient of the returned scores (SoftmaxTopKMaxPoolingFusedFn.backward, :1040-1092, which
 * scatters into a dense (B,h_kv,G,L,N) tensor and runs two bmm).  Here, bf16 with D = 64 or 128: the
 * dense matrix exists only as 64 x 128 tiles in shared memory and both products run on the tensor
 * cores; otherwise a K-sparse gather for dq and an fp32 scatter-add for the chunk keys.
 *   d_scores (B,L,h_kv*G,topk) in `dtype`; d_q (B,L,h_kv,G,D) in `dtype`;
 *   d_lmks_f32: fp32 accumulator with the shape of lmks, zeroed by this call;
 *   d_lmks: same shape in `dtype` (written from the accumulator). */
int hils_topk_bwd(const void* d_scores, const int32_t* indices, const void* q, const void* lmks,
                  void* d_q, float* d_lmks_f32, void* d_lmks,
                  int B, int L, int N, int h_kv, int G, int D, int topk, int per_qhead,
                  float sm_scale, int dtype, void* stream);

/* Selection backward for callers that cannot allocate device memory when they call (a frozen or
 * exhausted caching allocator, a server that reserved all memory at start-up, a plugin barred
 * from cudaMalloc after initialisation).  Same inputs, outputs and arithmetic as hils_topk_bwd,
 * but the fp32 accumulator is a fixed 4 MiB array inside the library image (every GPU that loads
 * the library holds it until exit), so nothing is allocated by the call or by the caller.
 *   Limit: B*N*heads*D (elements of lmks) <= hils_topk_bwd_noalloc_max_elems() = 1,048,576;
 *   larger problems are rejected with HILS_ERR_WORKSPACE.
 *   The first call on each device looks up the array's device address; make that first call
 *   outside any stream capture.
 *   All calls share the one array: it is cleared at the start of every call, and two calls whose
 *   work overlaps on the GPU (different streams) race on it - serialise them.
 * This entry point has no counterpart in the reference. */
int hils_topk_bwd_noalloc(const void* d_scores, const int32_t* indices, const void* q, const void* lmks,
                          void* d_q, void* d_lmks,
                          int B, int L, int N, int h_kv, int G, int D, int topk, int per_qhead,
                          float sm_scale, int dtype, void* stream);
size_t hils_topk_bwd_noalloc_max_elems(void);

/* ---------------------------------------------------------------------------------------
 * Sparse chunk attention.  Replaces _hils_block_M_attention_inverse.forward/backward
 * (ops/hils_fwd_bwd_head.py:771-913; kernels :198-496 and :506-766).
 *   o_i = sum_k w[i,k] * softmax_{j in chunk ids[i,k]}(scale*q_i.K_j - slope*max(0,S-2-j)) V_j
 *   q (B,L,h_q,D), k (B,T,h_kv,D), v (B,T,h_kv,Dv), weights (B,L,h_q,num_weights) (first K
 *   columns used), indices (B,L,h_kv,K); ids < 0 end a row's list.  slope (h_q) fp32 or NULL.
 * Backward: d_q, d_k, d_v, d_w in `dtype`; d_w has num_weights columns, those >= K are zero.
 * workspace: forward - hils_sparse_attn_fwd_workspace_bytes() bytes (0 for few query rows, for fp32 and for dense
 *   selections T/chunk_size <= 4*K; otherwise the inverse index [per (batch, kv head, chunk) the list of
 *   (token, slot) entries that selected it, with their weights] and an fp32 output accumulator; a missing or
 *   small workspace returns HILS_ERR_WORKSPACE); backward - hils_sparse_attn_bwd_workspace_bytes() bytes (the
 *   same index and fp32 accumulators).  d_k, d_v and d_w are bit-reproducible; o (sparse selections) and d_q
 *   are fp32 scatter-adds whose order varies, so their last bits differ from run to run.
 * ------------------------------------------------------------------------------------- */
int hils_sparse_attn_fwd(const void* q, const void* k, const void* v, const void* weights,
                         const int32_t* indices, const float* slope, void* o,
                         int B, int L, int T, int h_q, int h_kv, int D, int Dv, int K,
                         int num_weights, int chunk_size, float sm_scale, int mask_last_token,
                         int dtype, void* workspace, size_t workspace_bytes, void* stream);
size_t hils_sparse_attn_fwd_workspace_bytes(int B, int L, int T, int h_q, int h_kv, int D, int Dv,
                                            int K, int chunk_size, int dtype);
int hils_sparse_attn_bwd(const void* q, const void* k, const void* v, const void* weights,
                         const int32_t* indices, const float* slope, const void* d_o,
                         void* d_q, void* d_k, void* d_v, void* d_w,
                         int B, int L, int T, int h_q, int h_kv, int D, int Dv, int K,
                         int num_weights, int chunk_size, float sm_scale, int mask_last_token,
                         int dtype, void* workspace, size_t workspace_bytes, void* stream);
size_t hils_sparse_attn_bwd_workspace_bytes(int B, int L, int T, int h_q, int h_kv, int D, int Dv,
                                            int K, int chunk_size, int dtype);

/* The forward of a sparse selection (hils_sparse_attn_fwd_workspace_bytes > 0) leaves the chunk-major index of the id
 * lists in the first hils_sparse_attn_index_bytes() bytes of its workspace (0: this shape builds none).  A backward
 * over the same q shape, indices and weights can reuse it instead of building it again: keep those bytes (in place or
 * copied, 16-byte aligned) and pass them as `built_index`; NULL makes the call identical to hils_sparse_attn_bwd.
 * `workspace` is still the backward's own, of hils_sparse_attn_bwd_workspace_bytes().  No counterpart in the
 * reference, whose kernels re-walk the id lists in both passes (ops/hils_fwd_bwd_head.py:337-390, :560-640). */
size_t hils_sparse_attn_index_bytes(int B, int L, int T, int h_q, int h_kv, int D, int Dv,
                                    int K, int chunk_size, int dtype);
int hils_sparse_attn_bwd_with_index(const void* q, const void* k, const void* v, const void* weights,
                                    const int32_t* indices, const float* slope, const void* d_o,
                                    void* d_q, void* d_k, void* d_v, void* d_w,
                                    int B, int L, int T, int h_q, int h_kv, int D, int Dv, int K,
                                    int num_weights, int chunk_size, float sm_scale, int mask_last_token,
                                    int dtype, void* workspace, size_t workspace_bytes,
                                    const void* built_index, size_t built_index_bytes, void* stream);

/* ---------------------------------------------------------------------------------------
 * Exact per-chunk log Z.  Replaces _ExactChunkLogZ.forward/backward
 * (ops/exact_chunk_log_z_tilelang.py:394-478; kernels :25-137, :148-262, :273-391).
 *   q (B,L,h_q,D), k (B,L,h_kv,D); log_z (B,L,h_q,ceil(L/S)) fp32, -inf where chunk c is not
 *   strictly left of the snapped window of row i (i < (c+1)*S + W - 1).
 *   Backward (mask_lmk == 0 only): d_q, d_k in `dtype`.
 * ------------------------------------------------------------------------------------- */
int hils_chunk_logz_fwd(const void* q, const void* k, float* log_z,
                        int B, int L, int h_q, int h_kv, int D, int chunk_size, int window_size,
                        float sm_scale, int mask_lmk, int dtype, void* stream);
int hils_chunk_logz_bwd(const void* q, const void* k, const float* log_z, const float* d_log_z,
                        void* d_q, void* d_k,
                        int B, int L, int h_q, int h_kv, int D, int chunk_size, int window_size,
                        float sm_scale, int dtype, void* stream);

/* ---------------------------------------------------------------------------------------
 * Sliding-window branch with chunk-snapped left edge.  Replaces _FlexAttnTL.forward/backward
 * (ops/flex_attn_tilelang.py:609-719; kernels :26-267, :279-588).
 *   q (B,Lq,h_q,D), k (B,Lk,h_kv,D), v (B,Lk,h_kv,Dv); o (B,Lq,h_q,Dv) in `dtype`;
 *   lse (B,Lq,h_q) fp32, natural log; rows with no visible key give o = 0, lse = -inf.
 *   Query i sits at absolute position kv_start + (Lk-Lq) + i.
 *   Backward takes d_o and d_lse (fp32, may be NULL) and writes d_q, d_k, d_v in `dtype`;
 *   workspace: hils_swa_bwd_workspace_bytes() bytes of scratch (per-row Delta, fp32).
 * ------------------------------------------------------------------------------------- */
int hils_swa_fwd(const void* q, const void* k, const void* v, void* o, float* lse,
                 int B, int Lq, int Lk, int h_q, int h_kv, int D, int Dv,
                 int window_size, int chunk_size, int mask_lmk, int expand_to_chunk,
                 float sm_scale, int kv_start, int dtype, void* stream);
int hils_swa_bwd(const void* q, const void* k, const void* v, const void* o, const float* lse,
                 const void* d_o, const float* d_lse, void* d_q, void* d_k, void* d_v,
                 int B, int L, int h_q, int h_kv, int D, int Dv,
                 int window_size, int chunk_size, int mask_lmk, int expand_to_chunk,
                 float sm_scale, int dtype, void* workspace, size_t workspace_bytes, void* stream);
size_t hils_swa_bwd_workspace_bytes(int B, int L, int h_q, int h_kv, int D, int Dv, int chunk_size,
                                    int dtype);

/* ---------------------------------------------------------------------------------------
 * Inter-chunk softmax.  Replaces the PyTorch ops of HiLSAttention.forward that turn the selection
 * scores into chunk weights (models/FlashHiLS/hils_attention.py:585-610): gather of the prior bias
 * at the selected ids, add, concatenation with the sliding-window log-sum-exp (and a zero column
 * when softmax1 != 0), softmax over K+1(+1) columns.
 *   scores (B,L,h_q,K) and lse_swa (B,L,h_q) in `dtype`; indices (B,L,h_idx,K) int32, h_q a multiple
 *   of h_idx, -1 = empty slot; bias (B,N,h_q) fp32 or NULL; weights (B,L,h_q,K+1+softmax1) in `dtype`.
 *   Backward: d_scores (B,L,h_q,K) and d_lse (B,L,h_q) in `dtype`; d_bias (B,N,h_q) fp32 or NULL, zeroed
 *   here and accumulated with atomics.  K <= 94.
 * ------------------------------------------------------------------------------------- */
int hils_chunk_weights_fwd(const void* scores, const int32_t* indices, const float* bias,
                           const void* lse_swa, void* weights,
                           int B, int L, int N, int h_q, int h_idx, int K, int softmax1, int dtype,
                           void* stream);
int hils_chunk_weights_bwd(const void* weights, const void* d_weights, const int32_t* indices,
                           void* d_scores, void* d_lse, float* d_bias,
                           int B, int L, int N, int h_q, int h_idx, int K, int softmax1, int dtype,
                           void* stream);

/* ---------------------------------------------------------------------------------------
 * Combination of the two branches, o = o_hils + weights[..., swa_col] * o_swa.  Replaces the
 * torch.addcmul of HiLSAttention.forward (models/FlashHiLS/hils_attention.py:620-629).
 *   o_hils, o_swa, o, d_o, d_o_swa (B,L,h_q,D) and weights, d_weights (B,L,h_q,num_weights) in `dtype`.
 *   Backward writes d_o_swa and the single column d_weights[..., swa_col]; the gradient of o_hils is d_o.
 * ------------------------------------------------------------------------------------- */
int hils_combine_fwd(const void* o_hils, const void* o_swa, const void* weights, void* o,
                     int B, int L, int h_q, int D, int num_weights, int swa_col, int dtype, void* stream);
int hils_combine_bwd(const void* d_o, const void* o_swa, const void* weights, void* d_o_swa,
                     void* d_weights,
                     int B, int L, int h_q, int D, int num_weights, int swa_col, int dtype, void* stream);

/* ---------------------------------------------------------------------------------------
 * One decode step of the whole chain as a single call (one new token per sequence).  Replaces the
 * op-by-op decode branch of HiLSAttention.forward (models/FlashHiLS/hils_attention.py:512-633):
 * cache append, sliding-window branch, chunk selection at position `len`, prior-bias gather and
 * inter-chunk softmax, sparse chunk attention, combine.  The batch is folded into the head dimension
 * (heads_* = batch * heads), which the token-major store makes free:
 *   q and lmk_q, the query of the selection, (heads_q, D); k_new, v_new (heads_kv, D); k_store, v_store (capacity, heads_kv, D) holding `len`
 *   tokens, the new token is written to row `len` (capacity > len); lmk_k (N, heads_lmk, D) pooled
 *   chunk keys with heads_lmk = heads_kv or heads_q; prior_b (N, heads_q) fp32 or NULL;
 *   o (heads_q, D); indices_out (heads_kv, K) int32 or NULL.
 * Returns HILS_ERR_UNSUPPORTED while the store holds no complete chunk (run the step op by op).
 * ------------------------------------------------------------------------------------- */
int hils_decode_step(const void* q, const void* lmk_q, const void* k_new, const void* v_new,
                     void* k_store, void* v_store,
                     int len, const void* lmk_k, const float* prior_b, int N, void* o, int32_t* indices_out,
                     int heads_q, int heads_kv, int heads_lmk, int D, int K, int chunk_size, int window_size,
                     int softmax1, float sm_scale, int dtype,
                     void* workspace, size_t workspace_bytes, void* stream);
size_t hils_decode_step_workspace_bytes(int heads_q, int heads_kv, int heads_lmk, int D, int K, int N,
                                        int softmax1, int dtype);

/* ---------------------------------------------------------------------------------------
 * The same decode step over a PAGED store, for sequences of different lengths in one batch.  The page
 * is the chunk (64 tokens; the page size the reference's serving notes ask of the serving engine,
 * README.md:255,262), so a selected chunk is one page and the step never gathers across pages.
 * Replaces the growth by torch.cat and the CPU round trip of the reference's cache layer
 * (utils/hils_cache_utils.py:19-23, :45-62): a sequence grows by taking a page from the pool.
 *   k_pages, v_pages (num_pages, h_kv, 64, D): the pool, shared by all sequences; inside a page the 64
 *   rows of one head are contiguous (one 16 KB run at D = 128), so a selected chunk of a head is read as
 *   one run and not as 64 rows h_kv*D apart;
 *   page_table (B, page_stride) int32, device: page of chunk c of sequence b (entries past the
 *   sequence's last chunk are not read); lens (B) int32, device: tokens sequence b holds BEFORE this
 *   step; max_len: a host-side upper bound of lens (it sizes the launches; (max_len+1+63)/64 <=
 *   page_stride, and the page for position lens[b] must already be in the table);
 *   q, lmk_q, o (B, h_q, D); k_new, v_new (B, h_kv, D), written to row lens[b] % 64 of every head of
 *   page page_table[b][lens[b] / 64]; lmk_k (B, N, h_lmk, D) pooled chunk keys, row stride N for every
 *   sequence, rows at or past a sequence's selectable chunks are not read; prior_b (B, N, h_q) fp32 or
 *   NULL; indices_out (B, h_kv, K) int32 or NULL.  lens is NOT advanced (a model runs this once per
 *   layer with the same table).  A page id outside [0, num_pages) is skipped and reported through
 *   hils_take_device_status (8000001..8000003).
 * ------------------------------------------------------------------------------------- */
int hils_decode_step_paged(const void* q, const void* lmk_q, const void* k_new, const void* v_new,
                           void* k_pages, void* v_pages,
                           const int32_t* page_table, int page_stride, int num_pages,
                           const int32_t* lens, int max_len,
                           const void* lmk_k, const float* prior_b, int N, void* o, int32_t* indices_out,
                           int B, int h_q, int h_kv, int h_lmk, int D, int K, int chunk_size, int window_size,
                           int softmax1, float sm_scale, int dtype,
                           void* workspace, size_t workspace_bytes, void* stream);
size_t hils_decode_step_paged_workspace_bytes(int B, int h_q, int h_kv, int h_lmk, int D, int K, int N,
                                              int softmax1, int dtype);

/* ---------------------------------------------------------------------------------------
 * Per-head RMSNorm followed by the rotary embedding in one pass (upstream of the attention path).
 * Replaces rms_norm (models/FlashHiLS/modeling_olmo_hils.py:105-111, per-head q_norm / k_norm /
 * lmk_q_norm of hils_attention.py:250-253, :296-321) chained with single_tensor_rope_autograd
 * (ops/rope_tilelang_fp32.py:96-181; fp32 x*cos + rotate_half(x)*sin, rounded once).
 *   x, out, d_out, d_x (B,L,H,D) in `dtype`; weight (D) in `dtype` or NULL (no norm);
 *   cos, sin (L,D) shared over the batch (cos_batched = 0) or (B,L,D) (cos_batched = 1), in
 *   `cs_dtype`, or both NULL (no rotation); rstd (B,L,H) fp32 written by the forward when weight is
 *   given and read by the backward; d_weight (D) fp32, zeroed here and accumulated with atomics.
 * ------------------------------------------------------------------------------------- */
int hils_norm_rope_fwd(const void* x, const void* weight, const void* cos, const void* sin, void* out,
                       float* rstd, int B, int L, int H, int D, int cos_batched, float eps,
                       int dtype, int cs_dtype, void* stream);
int hils_norm_rope_bwd(const void* x, const void* weight, const void* cos, const void* sin,
                       const float* rstd, const void* d_out, void* d_x, float* d_weight,
                       int B, int L, int H, int D, int cos_batched, int dtype, int cs_dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* HILS_B200_H */
