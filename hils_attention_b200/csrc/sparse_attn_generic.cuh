// Sparse chunk attention, exact-fp32 CUDA-core form: one warp per (batch, token, q-head) row.
// Used for fp32 tensors and for shapes the tensor-core path does not cover.
//
// Math (ops/hils_fwd_bwd_head.py:21-93; kernels :404-485 forward, :651-757 backward):
//   s_j = (<q, K_{cS+j}> - slope*max(0, S-2-j)) * scale, s_{S-1} = -inf when mask_last_token
//   P = softmax_j(s);  o += w_k * sum_j P_j V_{cS+j}          (own softmax per selected chunk)
//   dP_j = <dO, V_j>; dw_k = sum_j P_j dP_j; dV_j += w_k P_j dO;
//   dS_j = scale w_k P_j (dP_j - dw_k); dK_j += dS_j q; dq += sum_j dS_j K_j
// A row's list ends at its first negative id (:343-352).
#pragma once
#include "common.cuh"

namespace hils {

struct SparseParams {
  const void* q; const void* k; const void* v; const void* w; const int32_t* idx; const float* slope;
  void* o; const void* d_o; void* d_q; void* d_w; float* dk_acc; float* dv_acc; void* d_k_out; void* d_v_out;
  int B, L, T, h_q, h_kv, D, Dv, K, num_weights, S, mask_last;
  float scale;
};

// logits of one chunk for this warp's row: lane handles keys j = lane, lane+32, ...; returns the
// probabilities (normalised) in p_s[0..S) and whether the chunk had any unmasked key.
template <typename T>
__device__ __forceinline__ bool chunk_probs(const SparseParams& p, const float* q_s, float* p_s, const T* kbase,
                                            int64_t krow_stride, float slope, int lane) {
  const int S = p.S;
  float m = -CUDART_INF_F;
  for (int j = lane; j < S; j += 32) {
    float s = dot_row(q_s, kbase + (int64_t)j * krow_stride, p.D);
    if (slope != 0.f) s -= slope * (float)max(0, S - 2 - j);
    s *= p.scale;
    if (p.mask_last && j == S - 1) s = -CUDART_INF_F;
    p_s[j] = s;
    m = fmaxf(m, s);
  }
  m = warp_max(m);
  if (!(m > -CUDART_INF_F)) return false;
  float sum = 0.f;
  for (int j = lane; j < S; j += 32) {
    float e = expf(p_s[j] - m);
    p_s[j] = e;
    sum += e;
  }
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
  for (int j = lane; j < S; j += 32) p_s[j] *= inv;
  __syncwarp();
  return true;
}

template <typename T>
__global__ void __launch_bounds__(128) sparse_fwd_generic_kernel(SparseParams p, int64_t rows) {
  extern __shared__ __align__(16) float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* q_s = smem + warp * (p.D + p.S);
  float* p_s = q_s + p.D;
  const int64_t row = (int64_t)blockIdx.x * 4 + warp;  // (b, l, hq)
  if (row >= rows) return;
  const int hq = (int)(row % p.h_q);
  const int64_t bl = row / p.h_q;
  const int64_t b = bl / p.L;
  const int G = p.h_q / p.h_kv, h = hq / G;
  const T* q = static_cast<const T*>(p.q) + row * p.D;
  for (int d = lane * 4; d < p.D; d += 128) *reinterpret_cast<float4*>(q_s + d) = load4(q + d);
  __syncwarp();
  const int32_t* ids = p.idx + (bl * p.h_kv + h) * p.K;
  const T* wrow = static_cast<const T*>(p.w) + row * p.num_weights;
  const float slope = p.slope ? p.slope[hq] : 0.f;
  const int64_t krs = (int64_t)p.h_kv * p.D, vrs = (int64_t)p.h_kv * p.Dv;
  const int nchunk = p.T / p.S;
  float4 acc[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};  // Dv <= 256
  for (int kk = 0; kk < p.K; ++kk) {
    const int id = ids[kk];
    if (id < 0) break;
    if (id >= nchunk) continue;
    const float wk = to_f(wrow[kk]);
    const T* kbase = static_cast<const T*>(p.k) + ((b * p.T + (int64_t)id * p.S) * p.h_kv + h) * p.D;
    const T* vbase = static_cast<const T*>(p.v) + ((b * p.T + (int64_t)id * p.S) * p.h_kv + h) * p.Dv;
    __syncwarp();
    if (!chunk_probs<T>(p, q_s, p_s, kbase, krs, slope, lane)) continue;
    for (int j = 0; j < p.S; ++j) {
      const float pj = p_s[j] * wk;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int d = lane * 4 + u * 128;
        if (d < p.Dv) {
          float4 vv = load4(vbase + (int64_t)j * vrs + d);
          acc[u].x = fmaf(pj, vv.x, acc[u].x); acc[u].y = fmaf(pj, vv.y, acc[u].y);
          acc[u].z = fmaf(pj, vv.z, acc[u].z); acc[u].w = fmaf(pj, vv.w, acc[u].w);
        }
      }
    }
  }
  T* o = static_cast<T*>(p.o) + row * p.Dv;
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int d = lane * 4 + u * 128;
    if (d < p.Dv) store4(o + d, acc[u]);
  }
}

template <typename T>
__global__ void __launch_bounds__(128) sparse_bwd_generic_kernel(SparseParams p, int64_t rows) {
  extern __shared__ __align__(16) float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* q_s = smem + warp * (p.D + p.Dv + 2 * p.S);
  float* do_s = q_s + p.D;
  float* p_s = do_s + p.Dv;
  float* ds_s = p_s + p.S;
  const int64_t row = (int64_t)blockIdx.x * 4 + warp;
  if (row >= rows) return;
  const int hq = (int)(row % p.h_q);
  const int64_t bl = row / p.h_q;
  const int64_t b = bl / p.L;
  const int G = p.h_q / p.h_kv, h = hq / G;
  const T* q = static_cast<const T*>(p.q) + row * p.D;
  const T* dO = static_cast<const T*>(p.d_o) + row * p.Dv;
  for (int d = lane * 4; d < p.D; d += 128) *reinterpret_cast<float4*>(q_s + d) = load4(q + d);
  for (int d = lane * 4; d < p.Dv; d += 128) *reinterpret_cast<float4*>(do_s + d) = load4(dO + d);
  __syncwarp();
  const int32_t* ids = p.idx + (bl * p.h_kv + h) * p.K;
  const T* wrow = static_cast<const T*>(p.w) + row * p.num_weights;
  T* dwrow = static_cast<T*>(p.d_w) + row * p.num_weights;
  const float slope = p.slope ? p.slope[hq] : 0.f;
  const int64_t krs = (int64_t)p.h_kv * p.D, vrs = (int64_t)p.h_kv * p.Dv;
  const int nchunk = p.T / p.S;
  float4 dq[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};
  bool ended = false;
  for (int kk = 0; kk < p.num_weights; ++kk) {
    const int id = (kk < p.K && !ended) ? ids[kk] : -1;
    if (id < 0) ended = true;
    float dw = 0.f;
    if (id >= 0 && id < nchunk) {
      const float wk = to_f(wrow[kk]);
      const int64_t tok0 = b * p.T + (int64_t)id * p.S;
      const T* kbase = static_cast<const T*>(p.k) + (tok0 * p.h_kv + h) * p.D;
      const T* vbase = static_cast<const T*>(p.v) + (tok0 * p.h_kv + h) * p.Dv;
      __syncwarp();
      if (chunk_probs<T>(p, q_s, p_s, kbase, krs, slope, lane)) {
        float part = 0.f;
        for (int j = lane; j < p.S; j += 32) {
          float dp = dot_row(do_s, vbase + (int64_t)j * vrs, p.Dv);
          ds_s[j] = dp;
          part = fmaf(p_s[j], dp, part);
        }
        dw = warp_sum(part);
        for (int j = lane; j < p.S; j += 32) ds_s[j] = p.scale * wk * p_s[j] * (ds_s[j] - dw);
        __syncwarp();
        float* dkb = p.dk_acc + (tok0 * p.h_kv + h) * p.D;
        float* dvb = p.dv_acc + (tok0 * p.h_kv + h) * p.Dv;
        for (int j = 0; j < p.S; ++j) {
          const float dsj = ds_s[j], pw = p_s[j] * wk;
          if (pw == 0.f && dsj == 0.f) continue;
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int d = lane * 4 + u * 128;
            if (d < p.D) {
              float4 kv = load4(kbase + (int64_t)j * krs + d);
              dq[u].x = fmaf(dsj, kv.x, dq[u].x); dq[u].y = fmaf(dsj, kv.y, dq[u].y);
              dq[u].z = fmaf(dsj, kv.z, dq[u].z); dq[u].w = fmaf(dsj, kv.w, dq[u].w);
              float* a = dkb + (int64_t)j * krs + d;
              atomicAdd(a + 0, dsj * q_s[d + 0]); atomicAdd(a + 1, dsj * q_s[d + 1]);
              atomicAdd(a + 2, dsj * q_s[d + 2]); atomicAdd(a + 3, dsj * q_s[d + 3]);
            }
            if (d < p.Dv) {
              float* a = dvb + (int64_t)j * vrs + d;
              atomicAdd(a + 0, pw * do_s[d + 0]); atomicAdd(a + 1, pw * do_s[d + 1]);
              atomicAdd(a + 2, pw * do_s[d + 2]); atomicAdd(a + 3, pw * do_s[d + 3]);
            }
          }
        }
      }
    }
    if (lane == 0) dwrow[kk] = from_f<T>(dw);
  }
  T* dqo = static_cast<T*>(p.d_q) + row * p.D;
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int d = lane * 4 + u * 128;
    if (d < p.D) store4(dqo + d, dq[u]);
  }
}

}  // namespace hils
