// C entry points of the sparse chunk attention (forward and backward) and their dispatch.
#include "sparse_attn_generic.cuh"

namespace hils {

int sparse_fwd_tc_launch(const SparseParams& p, cudaStream_t st);  // sparse_attn_tc.cu
size_t sparse_fwd_cm_workspace(const SparseParams& p);             // sparse_attn_cm.cu
int sparse_fwd_cm_launch(const SparseParams& p, void* workspace, cudaStream_t st);
int sparse_decode_launch(const void* q, const void* k, const void* v, const void* w, const int32_t* idx, const float* slope,
                         void* o, int B, int L, int T, int h_q, int h_kv, int D, int Dv, int K, int num_weights, int S,
                         float scale, int mask_last, int dtype, cudaStream_t st);  // decode_attn.cu
size_t sparse_bwd_cm_workspace(const SparseParams& p);             // sparse_attn_cm.cu
int sparse_bwd_cm_launch(const SparseParams& p, void* d_k, void* d_v, void* workspace, cudaStream_t st, const void* built_index);
size_t sparse_cm_index_bytes(const SparseParams& p);

static int check_sparse(int B, int L, int T, int h_q, int h_kv, int D, int Dv, int K, int num_weights,
                        int chunk_size, int dtype) {
  HILS_REQUIRE(B > 0 && L >= 0 && T >= 0 && h_q > 0 && h_kv > 0 && D > 0 && Dv > 0, "sparse_attn: bad size");
  HILS_REQUIRE(h_q % h_kv == 0, "sparse_attn: h_q (%d) must be a multiple of h_kv (%d)", h_q, h_kv);
  HILS_REQUIRE(K > 0 && num_weights >= K, "sparse_attn: need num_weights (%d) >= K (%d) > 0", num_weights, K);
  HILS_REQUIRE(chunk_size > 0, "sparse_attn: chunk_size must be positive");
  HILS_REQUIRE(D % 4 == 0 && Dv % 4 == 0 && D <= 256 && Dv <= 256,
               "sparse_attn: head dims (%d, %d) must be multiples of 4 and <= 256", D, Dv);
  HILS_REQUIRE(dtype == HILS_F32 || dtype == HILS_BF16, "sparse_attn: unknown dtype %d", dtype);
  return HILS_OK;
}

static SparseParams make_params(const void* q, const void* k, const void* v, const void* w, const int32_t* idx,
                                const float* slope, int B, int L, int T, int h_q, int h_kv, int D, int Dv, int K,
                                int num_weights, int S, float scale, int mask_last) {
  SparseParams p;
  p.q = q; p.k = k; p.v = v; p.w = w; p.idx = idx; p.slope = slope;
  p.o = nullptr; p.d_o = nullptr; p.d_q = nullptr; p.d_w = nullptr; p.dk_acc = nullptr; p.dv_acc = nullptr;
  p.d_k_out = nullptr; p.d_v_out = nullptr;
  p.B = B; p.L = L; p.T = T; p.h_q = h_q; p.h_kv = h_kv; p.D = D; p.Dv = Dv; p.K = K;
  p.num_weights = num_weights; p.S = S; p.mask_last = mask_last; p.scale = scale;
  return p;
}

}  // namespace hils

using namespace hils;

extern "C" size_t hils_sparse_attn_fwd_workspace_bytes(int B, int L, int T, int h_q, int h_kv, int D, int Dv,
                                                       int K, int chunk_size, int dtype) {
  if (dtype == HILS_BF16 && h_q > 0 && h_kv > 0 && h_q % h_kv == 0 && L > 4) {
    SparseParams p = make_params(nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, B, L, T, h_q, h_kv, D, Dv, K, K,
                                 chunk_size, 1.f, 1);
    if ((int64_t)(T / (chunk_size > 0 ? chunk_size : 1)) <= 4 * (int64_t)K) return 0;   // dense selections: the query-block-major kernel
    return sparse_fwd_cm_workspace(p);   // inverse index + fp32 output accumulator of the chunk-major kernel
  }
  return 0;
}

extern "C" size_t hils_sparse_attn_bwd_workspace_bytes(int B, int L, int T, int h_q, int h_kv, int D, int Dv,
                                                       int K, int chunk_size, int dtype) {
  if (dtype == HILS_BF16 && h_q > 0 && h_kv > 0 && h_q % h_kv == 0) {
    SparseParams p = make_params(nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, B, L, T, h_q, h_kv, D, Dv, K, K,
                                 chunk_size, 1.f, 1);
    const size_t cm = sparse_bwd_cm_workspace(p);
    if (cm > 0) return cm;
  }
  return (size_t)B * T * h_kv * (size_t)(D + Dv) * sizeof(float);
}

extern "C" int hils_sparse_attn_fwd(const void* q, const void* k, const void* v, const void* weights,
                                    const int32_t* indices, const float* slope, void* o, int B, int L, int T,
                                    int h_q, int h_kv, int D, int Dv, int K, int num_weights, int chunk_size,
                                    float sm_scale, int mask_last_token, int dtype, void* workspace,
                                    size_t workspace_bytes, void* stream) {
  if (int rc = check_sparse(B, L, T, h_q, h_kv, D, Dv, K, num_weights, chunk_size, dtype)) return rc;
  if (L == 0) return HILS_OK;
  HILS_REQUIRE(q && weights && indices && o, "sparse_attn_fwd: null pointer");
  HILS_REQUIRE(T < chunk_size || (k && v), "sparse_attn_fwd: null k/v");
  // every kernel behind this entry point reads rows with 8- or 16-byte vector loads
  HILS_REQUIRE((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)weights | (uintptr_t)indices | (uintptr_t)o) & 15) == 0,
               "sparse_attn_fwd: tensors must be 16-byte aligned");
  SparseParams p = make_params(q, k, v, weights, indices, slope, B, L, T, h_q, h_kv, D, Dv, K, num_weights,
                               chunk_size, sm_scale, mask_last_token);
  p.o = o;
  cudaStream_t st = (cudaStream_t)stream;
  if (L <= 4) {  // a few query rows against a long store: streaming kernel, keys and values read once
    const int rc = sparse_decode_launch(q, k, v, weights, indices, slope, o, B, L, T, h_q, h_kv, D, Dv, K, num_weights,
                                        chunk_size, sm_scale, mask_last_token, dtype, st);
    if (rc != HILS_ERR_UNSUPPORTED) return rc;
  }
  if (dtype == HILS_BF16) {  // tensor-core paths for the shapes they cover
    // Two forward kernels.  Query-block-major (a block of 128 rows walks the union of its tokens' chunks, rows that did
    // not select a chunk are masked): no gather, no scatter, but its work grows with the union, so it is the choice
    // only where a token selects a large share of its candidates (few chunks per selected slot).  Chunk-major over
    // gathered owner rows: every MMA row is a real pair, whatever the overlap; it pays a gather and a scatter.
    const bool dense = (int64_t)(T / chunk_size) <= 4 * (int64_t)K;
    if (dense) {
      const int rc = sparse_fwd_tc_launch(p, st);
      if (rc != HILS_ERR_UNSUPPORTED) return rc;
    }
    // (a dense shape that the kernel above refused - misaligned tensors - has no workspace: it goes to the generic kernel)
    const size_t need = (L > 4 && !dense) ? sparse_fwd_cm_workspace(p) : 0;
    if (need > 0) {
      if (!workspace || workspace_bytes < need) {
        set_error("sparse_attn_fwd: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
        return HILS_ERR_WORKSPACE;
      }
      const int rc = sparse_fwd_cm_launch(p, workspace, st);
      if (rc != HILS_ERR_UNSUPPORTED) return rc;
    }
    const int rc = sparse_fwd_tc_launch(p, st);
    if (rc != HILS_ERR_UNSUPPORTED) return rc;
  }
  const int64_t rows = (int64_t)B * L * h_q;
  const size_t smem = 4 * (size_t)(D + chunk_size) * sizeof(float);
  HILS_REQUIRE(smem <= 200 * 1024, "sparse_attn_fwd: chunk_size %d too large", chunk_size);
  const unsigned blocks = (unsigned)((rows + 3) / 4);
  if (dtype == HILS_BF16) {
    cudaFuncSetAttribute(sparse_fwd_generic_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sparse_fwd_generic_kernel<bf16><<<blocks, 128, smem, st>>>(p, rows);
  } else {
    cudaFuncSetAttribute(sparse_fwd_generic_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sparse_fwd_generic_kernel<float><<<blocks, 128, smem, st>>>(p, rows);
  }
  HILS_LAUNCH_CHECK("sparse_attn_fwd");
  return HILS_OK;
}

// True when hils_sparse_attn_fwd of this shape builds the chunk-major index (same tests as its dispatch)
static bool fwd_builds_index(const SparseParams& p, int L, int T, int K, int chunk_size, int dtype) {
  if (dtype != HILS_BF16 || L <= 4) return false;
  if ((int64_t)(T / chunk_size) <= 4 * (int64_t)K) return false;   // dense selections: query-block-major forward
  return sparse_fwd_cm_workspace(p) > 0;
}

extern "C" size_t hils_sparse_attn_index_bytes(int B, int L, int T, int h_q, int h_kv, int D, int Dv, int K, int chunk_size,
                                               int dtype) {
  if (B <= 0 || L <= 0 || T <= 0 || h_kv <= 0 || h_q <= 0 || h_q % h_kv != 0 || chunk_size <= 0) return 0;
  SparseParams p = make_params(nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, B, L, T, h_q, h_kv, D, Dv, K, K, chunk_size,
                               1.f, 1);
  return fwd_builds_index(p, L, T, K, chunk_size, dtype) ? sparse_cm_index_bytes(p) : 0;
}

static int sparse_attn_bwd_impl(const void* q, const void* k, const void* v, const void* weights,
                                const int32_t* indices, const float* slope, const void* d_o, void* d_q,
                                void* d_k, void* d_v, void* d_w, int B, int L, int T, int h_q, int h_kv,
                                int D, int Dv, int K, int num_weights, int chunk_size, float sm_scale,
                                int mask_last_token, int dtype, void* workspace, size_t workspace_bytes,
                                void* stream, const void* built_index);

extern "C" int hils_sparse_attn_bwd(const void* q, const void* k, const void* v, const void* weights,
                                    const int32_t* indices, const float* slope, const void* d_o, void* d_q,
                                    void* d_k, void* d_v, void* d_w, int B, int L, int T, int h_q, int h_kv,
                                    int D, int Dv, int K, int num_weights, int chunk_size, float sm_scale,
                                    int mask_last_token, int dtype, void* workspace, size_t workspace_bytes,
                                    void* stream) {
  return sparse_attn_bwd_impl(q, k, v, weights, indices, slope, d_o, d_q, d_k, d_v, d_w, B, L, T, h_q, h_kv, D, Dv, K,
                              num_weights, chunk_size, sm_scale, mask_last_token, dtype, workspace, workspace_bytes, stream,
                              nullptr);
}

extern "C" int hils_sparse_attn_bwd_with_index(const void* q, const void* k, const void* v, const void* weights,
                                               const int32_t* indices, const float* slope, const void* d_o, void* d_q,
                                               void* d_k, void* d_v, void* d_w, int B, int L, int T, int h_q, int h_kv,
                                               int D, int Dv, int K, int num_weights, int chunk_size, float sm_scale,
                                               int mask_last_token, int dtype, void* workspace, size_t workspace_bytes,
                                               const void* built_index, size_t built_index_bytes, void* stream) {
  const size_t want = hils_sparse_attn_index_bytes(B, L, T, h_q, h_kv, D, Dv, K, chunk_size, dtype);
  if (built_index && (want == 0 || built_index_bytes < want)) {
    set_error("sparse_attn_bwd_with_index: an index of %zu bytes belongs to this shape, %zu given", want, built_index_bytes);
    return HILS_ERR_BAD_ARG;
  }
  return sparse_attn_bwd_impl(q, k, v, weights, indices, slope, d_o, d_q, d_k, d_v, d_w, B, L, T, h_q, h_kv, D, Dv, K,
                              num_weights, chunk_size, sm_scale, mask_last_token, dtype, workspace, workspace_bytes, stream,
                              built_index);
}

static int sparse_attn_bwd_impl(const void* q, const void* k, const void* v, const void* weights,
                                const int32_t* indices, const float* slope, const void* d_o, void* d_q,
                                void* d_k, void* d_v, void* d_w, int B, int L, int T, int h_q, int h_kv,
                                int D, int Dv, int K, int num_weights, int chunk_size, float sm_scale,
                                int mask_last_token, int dtype, void* workspace, size_t workspace_bytes,
                                void* stream, const void* built_index) {
  if (int rc = check_sparse(B, L, T, h_q, h_kv, D, Dv, K, num_weights, chunk_size, dtype)) return rc;
  const size_t need = hils_sparse_attn_bwd_workspace_bytes(B, L, T, h_q, h_kv, D, Dv, K, chunk_size, dtype);
  if (need > 0 && (!workspace || workspace_bytes < need)) {
    set_error("sparse_attn_bwd: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
    return HILS_ERR_WORKSPACE;
  }
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == HILS_BF16 && L > 0) {  // tensor-core path for the shapes it covers
    SparseParams p = make_params(q, k, v, weights, indices, slope, B, L, T, h_q, h_kv, D, Dv, K, num_weights,
                                 chunk_size, sm_scale, mask_last_token);
    if (sparse_bwd_cm_workspace(p) > 0) {
      HILS_REQUIRE(q && k && v && weights && indices && d_o && d_q && d_k && d_v && d_w, "sparse_attn_bwd: null pointer");
      p.d_o = d_o; p.d_q = d_q; p.d_w = d_w;
      const int rc = sparse_bwd_cm_launch(p, d_k, d_v, workspace, st, built_index);
      if (rc != HILS_ERR_UNSUPPORTED) return rc;
      // the tensor-core path covers this shape but the pointers are not 16-byte aligned: no other kernel is
      // sized for the tensor-core workspace, so the call is refused rather than rerouted
      set_error("sparse_attn_bwd: tensors must be 16-byte aligned for this shape");
      return HILS_ERR_BAD_ARG;
    }
  }
  const int64_t nk = (int64_t)B * T * h_kv * D, nv = (int64_t)B * T * h_kv * Dv;
  float* dk_acc = static_cast<float*>(workspace);
  float* dv_acc = dk_acc + nk;
  if (need > 0) {
    HILS_REQUIRE(d_k && d_v, "sparse_attn_bwd: null d_k/d_v");
    cudaError_t e = cudaMemsetAsync(workspace, 0, need, st);
    if (e != cudaSuccess) return cuda_fail(e, "sparse_attn_bwd memset");
  }
  if (L > 0) {
    HILS_REQUIRE(q && weights && indices && d_o && d_q && d_w, "sparse_attn_bwd: null pointer");
    SparseParams p = make_params(q, k, v, weights, indices, slope, B, L, T, h_q, h_kv, D, Dv, K, num_weights,
                                 chunk_size, sm_scale, mask_last_token);
    p.d_o = d_o; p.d_q = d_q; p.d_w = d_w; p.dk_acc = dk_acc; p.dv_acc = dv_acc;
    const int64_t rows = (int64_t)B * L * h_q;
    const size_t smem = 4 * (size_t)(D + Dv + 2 * chunk_size) * sizeof(float);
    HILS_REQUIRE(smem <= 200 * 1024, "sparse_attn_bwd: chunk_size %d too large", chunk_size);
    const unsigned blocks = (unsigned)((rows + 3) / 4);
    if (dtype == HILS_BF16) {
      cudaFuncSetAttribute(sparse_bwd_generic_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      sparse_bwd_generic_kernel<bf16><<<blocks, 128, smem, st>>>(p, rows);
    } else {
      cudaFuncSetAttribute(sparse_bwd_generic_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      sparse_bwd_generic_kernel<float><<<blocks, 128, smem, st>>>(p, rows);
    }
    HILS_LAUNCH_CHECK("sparse_attn_bwd");
  }
  if (need > 0) {
    if (dtype == HILS_BF16) {
      launch_cast_from_f32<bf16>(dk_acc, (bf16*)d_k, nk, st);
      launch_cast_from_f32<bf16>(dv_acc, (bf16*)d_v, nv, st);
    } else {
      launch_cast_from_f32<float>(dk_acc, (float*)d_k, nk, st);
      launch_cast_from_f32<float>(dv_acc, (float*)d_v, nv, st);
    }
    HILS_LAUNCH_CHECK("sparse_attn_bwd cast");
  }
  return HILS_OK;
}
