// One decode step of the HiLS attention chain as a single host call.
//
// The reference runs this step as a sequence of Python-level ops (models/FlashHiLS/hils_attention.py:512-633
// with one new token per sequence: cache append, sliding-window branch, chunk selection, prior-bias gather and
// inter-chunk softmax, sparse chunk attention, combine).  At decode sizes the kernels take a few hundred
// microseconds in total, comparable to the host time of issuing them one by one through an interpreter;
// this entry point issues all of them back to back on one stream.  The batch is folded into the head
// dimension (every stage is independent per (sequence, head)): `heads_*` below are batch * heads.
#include "common.cuh"

namespace hils {

template <typename T>
__global__ void cast_rows_kernel(const float* __restrict__ src, T* __restrict__ dst, int n) {
  const int i = blockIdx.x * 256 + threadIdx.x;
  if (i < n) dst[i] = from_f<T>(src[i]);
}

static size_t up256(size_t x) { return (x + 255) & ~(size_t)255; }

struct StepLayout {
  size_t swa_o, lse32, lse_act, scores, weights, indices, topk_ws, total;
};

static StepLayout step_layout(int heads_q, int heads_kv, int D, int K, int N, int softmax1, int dtype, int h_t, int g_t) {
  const size_t es = dtype == HILS_BF16 ? 2 : 4;
  StepLayout s;
  size_t o = 0;
  s.swa_o = o;   o += up256((size_t)heads_q * D * es);
  s.lse32 = o;   o += up256((size_t)heads_q * 4);
  s.lse_act = o; o += up256((size_t)heads_q * es);
  s.scores = o;  o += up256((size_t)heads_q * K * es);
  s.weights = o; o += up256((size_t)heads_q * (K + 1 + (softmax1 ? 1 : 0)) * es);
  s.indices = o; o += up256((size_t)heads_kv * K * 4);
  s.topk_ws = o; o += up256(hils_topk_fwd_workspace_bytes(1, 1, N, h_t, g_t, D, dtype));
  s.total = o;
  return s;
}

// selection runs with shared keys (one key head per kv head) or per-q-head keys
static bool topk_shape(int heads_q, int heads_kv, int heads_lmk, int* h_t, int* g_t, int* per_qhead) {
  if (heads_lmk == heads_kv) { *h_t = heads_kv; *g_t = heads_q / heads_kv; *per_qhead = 0; return true; }
  if (heads_lmk == heads_q) { *h_t = heads_kv; *g_t = heads_q / heads_kv; *per_qhead = 1; return true; }
  return false;
}

// decode_attn.cu, topk.cu
int paged_append_launch(const void* k_new, const void* v_new, void* k_pages, void* v_pages, const int32_t* pages,
                        const int32_t* lens, int page_stride, int num_pages, int S, int B, int h_kv, int D, int dtype,
                        cudaStream_t st);
int swa_decode_paged_launch(const void* q, const void* k_pages, const void* v_pages, void* o, float* lse,
                            const int32_t* pages, const int32_t* lens, int page_stride, int num_pages, int len_add, int B,
                            int h_q, int h_kv, int D, int W, int S, int mask_lmk, float scale, int dtype, cudaStream_t st,
                            void* lse_act);
int sparse_decode_paged_launch(const void* q, const void* k_pages, const void* v_pages, const void* w, const int32_t* idx,
                               void* o, const int32_t* pages, const int32_t* lens, int page_stride, int num_pages,
                               int len_add, int B, int h_q, int h_kv, int D, int K, int num_weights, int S, float scale,
                               int mask_last, int dtype, cudaStream_t st, const void* swa_o, int swa_col);
int swa_decode_lse_launch(const void* q, const void* k, const void* v, void* o, float* lse, void* lse_act, int B, int Lk,
                          int h_q, int h_kv, int D, int W, int S, int mask_lmk, int expand, float scale, int dtype,
                          cudaStream_t st);
int sparse_decode_combine_launch(const void* q, const void* k, const void* v, const void* w, const int32_t* idx, void* o,
                                 int B, int T, int h_q, int h_kv, int D, int K, int num_weights, int S, float scale,
                                 int mask_last, int dtype, cudaStream_t st, const void* swa_o, int swa_col);
int topk_decode_step_launch(const void* q, const void* lmks, const void* lse_swa, const float* bias, int32_t* indices,
                            void* scores, void* weights, int softmax1, const int32_t* q_offsets, int q_offset, int B, int N,
                            int h_kv, int G, int D, int topk, int block_size, int window_size, int per_qhead, float sm_scale,
                            int dtype, int lse_dtype, void* workspace, size_t workspace_bytes, cudaStream_t st);

// workspace of the paged step: the same pieces, per sequence
static StepLayout paged_layout(int B, int h_q, int h_kv, int D, int K, int N, int softmax1, int dtype) {
  const size_t es = dtype == HILS_BF16 ? 2 : 4;
  StepLayout s;
  size_t o = 0;
  const size_t rows = (size_t)B * h_q;
  s.swa_o = o;   o += up256(rows * D * es);
  s.lse32 = o;   o += up256(rows * 4);
  s.lse_act = o; o += up256(rows * es);
  s.scores = o;  o += up256(rows * K * es);
  s.weights = o; o += up256(rows * (K + 1 + (softmax1 ? 1 : 0)) * es);
  s.indices = o; o += up256((size_t)B * h_kv * K * 4);
  s.topk_ws = o; o += up256(hils_topk_fwd_workspace_bytes(B, 1, N, h_kv, h_q / h_kv, D, dtype));
  s.total = o;
  return s;
}

}  // namespace hils

using namespace hils;

extern "C" size_t hils_decode_step_paged_workspace_bytes(int B, int h_q, int h_kv, int h_lmk, int D, int K, int N,
                                                         int softmax1, int dtype) {
  if (B <= 0 || h_kv <= 0 || h_q % h_kv != 0 || (h_lmk != h_kv && h_lmk != h_q)) return 0;
  return paged_layout(B, h_q, h_kv, D, K, N, softmax1, dtype).total;
}

extern "C" int hils_decode_step_paged(const void* q, const void* lmk_q, const void* k_new, const void* v_new, void* k_pages,
                                      void* v_pages, const int32_t* page_table, int page_stride, int num_pages,
                                      const int32_t* lens, int max_len, const void* lmk_k, const float* prior_b, int N,
                                      void* o, int32_t* indices_out, int B, int h_q, int h_kv, int h_lmk, int D, int K,
                                      int chunk_size, int window_size, int softmax1, float sm_scale, int dtype,
                                      void* workspace, size_t workspace_bytes, void* stream) {
  HILS_REQUIRE(dtype == HILS_BF16 || dtype == HILS_F32, "decode_step_paged: dtype must be bf16 or fp32");
  HILS_REQUIRE(B > 0 && h_q > 0 && h_kv > 0 && h_q % h_kv == 0, "decode_step_paged: h_q must be a multiple of h_kv");
  HILS_REQUIRE(h_lmk == h_kv || h_lmk == h_q, "decode_step_paged: the chunk keys must have h_kv or h_q heads");
  HILS_REQUIRE(chunk_size == 64, "decode_step_paged: the page is the chunk and must hold 64 tokens (got %d)", chunk_size);
  HILS_REQUIRE(D == 64 || D == 128, "decode_step_paged: head dimension %d (64 or 128)", D);
  HILS_REQUIRE(K > 0 && K <= 32, "decode_step_paged: topk %d (1..32)", K);
  HILS_REQUIRE(h_q / h_kv <= 8, "decode_step_paged: at most 8 query heads per kv head");
  HILS_REQUIRE(N > 0 && page_stride > 0 && num_pages > 0 && max_len >= 0, "decode_step_paged: bad size");
  HILS_REQUIRE((max_len + 1 + chunk_size - 1) / chunk_size <= page_stride,
               "decode_step_paged: %d tokens do not fit a page table of %d pages", max_len + 1, page_stride);
  HILS_REQUIRE(max_len / chunk_size <= N, "decode_step_paged: %d complete chunks but room for %d chunk keys",
               max_len / chunk_size, N);
  HILS_REQUIRE(q && lmk_q && k_new && v_new && k_pages && v_pages && page_table && lens && lmk_k && o,
               "decode_step_paged: null pointer");
  HILS_REQUIRE(((((uintptr_t)q) | ((uintptr_t)k_new) | ((uintptr_t)v_new) | ((uintptr_t)k_pages) | ((uintptr_t)v_pages) |
                 ((uintptr_t)lmk_k) | ((uintptr_t)lmk_q) | ((uintptr_t)o)) & 15) == 0,
               "decode_step_paged: tensors must be 16-byte aligned");
  const StepLayout lay = paged_layout(B, h_q, h_kv, D, K, N, softmax1, dtype);
  if (!workspace || workspace_bytes < lay.total) {
    set_error("decode_step_paged: workspace of %zu bytes needed, %zu given", lay.total, workspace_bytes);
    return HILS_ERR_WORKSPACE;
  }
  cudaStream_t st = (cudaStream_t)stream;
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  void* swa_o = ws + lay.swa_o;
  float* lse32 = reinterpret_cast<float*>(ws + lay.lse32);
  void* lse_act = ws + lay.lse_act;
  void* scores = ws + lay.scores;
  void* weights = ws + lay.weights;
  int32_t* indices = indices_out ? indices_out : reinterpret_cast<int32_t*>(ws + lay.indices);
  const int G = h_q / h_kv;
  // 1. every sequence's new token goes to row lens[b] of its own pages
  if (int rc = paged_append_launch(k_new, v_new, k_pages, v_pages, page_table, lens, page_stride, num_pages, chunk_size, B,
                                   h_kv, D, dtype, st))
    return rc;
  // 2. sliding-window branch over lens[b] + 1 tokens, landmark columns masked, left edge snapped to the chunk
  if (int rc = swa_decode_paged_launch(q, k_pages, v_pages, swa_o, lse32, page_table, lens, page_stride, num_pages, 1, B, h_q,
                                       h_kv, D, window_size, chunk_size, 1, sm_scale, dtype, st, lse_act)) {
    if (rc == HILS_ERR_UNSUPPORTED) set_error("decode_step_paged: shape not covered by the decode kernels");
    return rc;
  }
  // 3. chunk selection, sequence b at position lens[b], then prior-bias gather + softmax over [chunks, window(, 0)]
  const int nw = K + 1 + (softmax1 ? 1 : 0);
  if (int rc = topk_decode_step_launch(lmk_q, lmk_k, lse_act, prior_b, indices, scores, weights, softmax1, lens, max_len, B, N,
                                       h_kv, G, D, K, chunk_size, window_size, h_lmk == h_q && h_q != h_kv, sm_scale, dtype,
                                       dtype, ws + lay.topk_ws, lay.total - lay.topk_ws, st)) {
    if (rc == HILS_ERR_UNSUPPORTED) set_error("decode_step_paged: selection shape not covered by the decode kernels");
    return rc;
  }
  // 4. sparse chunk attention over the selected pages, and o = o_hils + w_swa * o_swa
  const int rc = sparse_decode_paged_launch(q, k_pages, v_pages, weights, indices, o, page_table, lens, page_stride, num_pages,
                                            1, B, h_q, h_kv, D, K, nw, chunk_size, sm_scale, 1, dtype, st, swa_o, K);
  if (rc == HILS_ERR_UNSUPPORTED) set_error("decode_step_paged: shape not covered by the decode kernels");
  return rc;
}

extern "C" size_t hils_decode_step_workspace_bytes(int heads_q, int heads_kv, int heads_lmk, int D, int K, int N,
                                                   int softmax1, int dtype) {
  int h_t, g_t, pq;
  if (heads_kv <= 0 || heads_q % heads_kv != 0 || !topk_shape(heads_q, heads_kv, heads_lmk, &h_t, &g_t, &pq)) return 0;
  return step_layout(heads_q, heads_kv, D, K, N, softmax1, dtype, h_t, g_t).total;
}

extern "C" int hils_decode_step(const void* q, const void* lmk_q, const void* k_new, const void* v_new, void* k_store, void* v_store,
                                int len, const void* lmk_k, const float* prior_b, int N, void* o, int32_t* indices_out,
                                int heads_q, int heads_kv, int heads_lmk, int D, int K, int chunk_size, int window_size,
                                int softmax1, float sm_scale, int dtype, void* workspace, size_t workspace_bytes,
                                void* stream) {
  HILS_REQUIRE(dtype == HILS_BF16 || dtype == HILS_F32, "decode_step: dtype must be bf16 or fp32");
  HILS_REQUIRE(heads_q > 0 && heads_kv > 0 && heads_q % heads_kv == 0, "decode_step: heads_q must be a multiple of heads_kv");
  HILS_REQUIRE(len >= 0 && N >= 0 && K > 0 && D > 0 && chunk_size > 0, "decode_step: bad size");
  int h_t, g_t, per_qhead;
  HILS_REQUIRE(topk_shape(heads_q, heads_kv, heads_lmk, &h_t, &g_t, &per_qhead),
               "decode_step: the chunk keys must have heads_kv or heads_q heads");
  if (len + 1 < chunk_size || N == 0) {
    set_error("decode_step: no complete chunk yet; run the step op by op");
    return HILS_ERR_UNSUPPORTED;
  }
  HILS_REQUIRE(q && lmk_q && k_new && v_new && k_store && v_store && lmk_k && o, "decode_step: null pointer");
  const StepLayout lay = step_layout(heads_q, heads_kv, D, K, N, softmax1, dtype, h_t, g_t);
  if (!workspace || workspace_bytes < lay.total) {
    set_error("decode_step: workspace of %zu bytes needed, %zu given", lay.total, workspace_bytes);
    return HILS_ERR_WORKSPACE;
  }
  cudaStream_t st = (cudaStream_t)stream;
  const size_t es = dtype == HILS_BF16 ? 2 : 4;
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  void* swa_o = ws + lay.swa_o;
  float* lse32 = reinterpret_cast<float*>(ws + lay.lse32);
  void* lse_act = ws + lay.lse_act;
  void* scores = ws + lay.scores;
  void* weights = ws + lay.weights;
  int32_t* indices = indices_out ? indices_out : reinterpret_cast<int32_t*>(ws + lay.indices);
  // 1. append the new token to the token-major store
  const size_t row_bytes = (size_t)heads_kv * D * es;
  cudaError_t e = cudaMemcpyAsync(static_cast<unsigned char*>(k_store) + (size_t)len * row_bytes, k_new, row_bytes,
                                  cudaMemcpyDeviceToDevice, st);
  if (e == cudaSuccess)
    e = cudaMemcpyAsync(static_cast<unsigned char*>(v_store) + (size_t)len * row_bytes, v_new, row_bytes,
                        cudaMemcpyDeviceToDevice, st);
  if (e != cudaSuccess) return cuda_fail(e, "decode_step (store append)");
  const int T = len + 1;
  HILS_REQUIRE(((((uintptr_t)q) | ((uintptr_t)lmk_q) | ((uintptr_t)k_store) | ((uintptr_t)v_store) | ((uintptr_t)lmk_k) |
                 ((uintptr_t)o) | ((uintptr_t)workspace)) & 15) == 0, "decode_step: tensors must be 16-byte aligned");
  // Four kernels where the shapes allow: the decode kernels take over the small element-wise stages between them (the
  // cast of the log-sum-exp, the inter-chunk softmax, the combination of the branches); shapes they do not cover run
  // the stage's general entry point and its follow-up kernel instead.
  // 2. sliding-window branch over the store, landmark columns masked, left edge snapped to the chunk; the chain
  //    carries its log-sum-exp in the activation dtype
  int rc = swa_decode_lse_launch(q, k_store, v_store, swa_o, lse32, lse_act, 1, T, heads_q, heads_kv, D, window_size,
                                 chunk_size, 1, 1, sm_scale, dtype, st);
  if (rc == HILS_ERR_UNSUPPORTED) {
    if ((rc = hils_swa_fwd(q, k_store, v_store, swa_o, lse32, 1, 1, T, heads_q, heads_kv, D, D, window_size, chunk_size, 1, 1,
                           sm_scale, 0, dtype, stream)))
      return rc;
    if (dtype == HILS_BF16) cast_rows_kernel<bf16><<<(heads_q + 255) / 256, 256, 0, st>>>(lse32, (bf16*)lse_act, heads_q);
    else cast_rows_kernel<float><<<(heads_q + 255) / 256, 256, 0, st>>>(lse32, (float*)lse_act, heads_q);
    HILS_LAUNCH_CHECK("decode_step (lse cast)");
  } else if (rc) {
    return rc;
  }
  // 3. chunk selection at absolute position `len`, then prior-bias gather + softmax over [chunks, window(, 0)]
  const int nw = K + 1 + (softmax1 ? 1 : 0);
  rc = topk_decode_step_launch(lmk_q, lmk_k, lse_act, prior_b, indices, scores, weights, softmax1, nullptr, len, 1, N, h_t,
                               g_t, D, K, chunk_size, window_size, per_qhead, sm_scale, dtype, dtype, ws + lay.topk_ws,
                               lay.total - lay.topk_ws, st);
  if (rc == HILS_ERR_UNSUPPORTED) {
    if ((rc = hils_topk_fwd(lmk_q, lmk_k, lse_act, prior_b, nullptr, nullptr, indices, scores, nullptr, nullptr, 1, 1, N, h_t,
                            g_t, D, K, chunk_size, window_size, 1, len, per_qhead, sm_scale, dtype, dtype, ws + lay.topk_ws,
                            lay.total - lay.topk_ws, stream)))
      return rc;
    if ((rc = hils_chunk_weights_fwd(scores, indices, prior_b, lse_act, weights, 1, 1, N, heads_q, heads_kv, K, softmax1,
                                     dtype, stream)))
      return rc;
  } else if (rc) {
    return rc;
  }
  // 4. sparse chunk attention over the store, and o = o_hils + w_swa * o_swa
  rc = (chunk_size <= 64) ? sparse_decode_combine_launch(q, k_store, v_store, weights, indices, o, 1, T, heads_q, heads_kv, D,
                                                         K, nw, chunk_size, sm_scale, 1, dtype, st, swa_o, K)
                          : HILS_ERR_UNSUPPORTED;
  if (rc != HILS_ERR_UNSUPPORTED) return rc;
  if ((rc = hils_sparse_attn_fwd(q, k_store, v_store, weights, indices, nullptr, o, 1, 1, T, heads_q, heads_kv, D, D, K, nw,
                                 chunk_size, sm_scale, 1, dtype, nullptr, 0, stream)))
    return rc;
  return hils_combine_fwd(o, swa_o, weights, o, 1, 1, heads_q, D, nw, K, dtype, stream);
}
