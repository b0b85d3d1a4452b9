// Sliding-window branch with a chunk-snapped left edge, exact-fp32 CUDA-core form: one warp per
// query row (forward, dQ) or per key row (dK/dV); atomic-free.
//
// Contract (ops/flex_attn_tilelang.py:115-133 positions, :155-216 masks, :246-253 empty rows,
// :685-702 dlse folded into Delta, :1307-1309 natural-log lse):
//   query i sits at absolute t = kv_start + (Lk - Lq) + i; key column jr at absolute j = kv_start + jr
//   visible: start <= j <= t, start = floor((t-W+1)/S)*S (expand_to_chunk) or t-W+1,
//            and (j+1)%S != 0 when mask_lmk
//   o = softmax(scale q.K) V over visible keys, lse natural log; empty rows: o = 0, lse = -inf
//   backward: Delta_i = <o_i, dO_i> - dlse_i;  dS = P (dP - Delta) scale
#include "common.cuh"

namespace hils {

struct SwaParams {
  const void* q; const void* k; const void* v; void* o; float* lse; const void* d_o; const float* d_lse;
  void* d_q; void* d_k; void* d_v;
  int B, Lq, Lk, h_q, h_kv, D, Dv, W, S, mask_lmk, expand, kv_start;
  float scale;
};

// raw key range [lo, hi] visible from query row i (may be empty: lo > hi)
__device__ __forceinline__ void swa_range(const SwaParams& p, int i, int& lo, int& hi) {
  const int t = p.kv_start + (p.Lk - p.Lq) + i;
  int start = t - p.W + 1;
  if (p.expand) start = floor_div(start, p.S) * p.S;
  lo = max(0, start - p.kv_start);
  hi = min(p.Lk - 1, t - p.kv_start);
}

__device__ __forceinline__ bool swa_col_masked(const SwaParams& p, int jr) {
  return p.mask_lmk && ((p.kv_start + jr + 1) % p.S == 0);
}

template <typename T>
__device__ __forceinline__ float dot_rows(const T* __restrict__ a, const T* __restrict__ b, int D) {
  float acc = 0.f;
  for (int d = 0; d < D; d += 4) {
    float4 x = load4(a + d), y = load4(b + d);
    acc = fmaf(x.x, y.x, acc); acc = fmaf(x.y, y.y, acc);
    acc = fmaf(x.z, y.z, acc); acc = fmaf(x.w, y.w, acc);
  }
  return acc;
}

template <typename T>
__global__ void __launch_bounds__(128) swa_fwd_kernel(SwaParams p, int64_t rows) {
  extern __shared__ __align__(16) float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* q_s = smem + warp * (p.D + 32);
  float* p_s = q_s + p.D;
  const int64_t row = (int64_t)blockIdx.x * 4 + warp;  // (b, i, hq)
  if (row >= rows) return;
  const int hq = (int)(row % p.h_q);
  const int64_t bi = row / p.h_q;
  const int i = (int)(bi % p.Lq);
  const int64_t b = bi / p.Lq;
  const int h = hq / (p.h_q / p.h_kv);
  const T* q = static_cast<const T*>(p.q) + row * p.D;
  for (int d = lane * 4; d < p.D; d += 128) *reinterpret_cast<float4*>(q_s + d) = load4(q + d);
  __syncwarp();
  int lo, hi;
  swa_range(p, i, lo, hi);
  const int64_t krs = (int64_t)p.h_kv * p.D, vrs = (int64_t)p.h_kv * p.Dv;
  const T* kb = static_cast<const T*>(p.k) + (b * p.Lk * p.h_kv + h) * p.D;
  const T* vb = static_cast<const T*>(p.v) + (b * p.Lk * p.h_kv + h) * p.Dv;
  float m = -CUDART_INF_F, l = 0.f;
  float4 acc[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};
  for (int j0 = lo; j0 <= hi; j0 += 32) {
    const int j = j0 + lane;
    float s = -CUDART_INF_F;
    if (j <= hi && !swa_col_masked(p, j)) s = dot_row(q_s, kb + (int64_t)j * krs, p.D) * p.scale;
    const float mn = fmaxf(m, warp_max(s));
    if (!(mn > -CUDART_INF_F)) continue;
    const float corr = (m > -CUDART_INF_F) ? expf(m - mn) : 0.f;
    const float e = expf(s - mn);
    l = l * corr + warp_sum(e);
    m = mn;
    __syncwarp();
    p_s[lane] = e;
    __syncwarp();
#pragma unroll
    for (int u = 0; u < 2; ++u) { acc[u].x *= corr; acc[u].y *= corr; acc[u].z *= corr; acc[u].w *= corr; }
    const int nj = min(32, hi - j0 + 1);
    for (int t = 0; t < nj; ++t) {
      const float pj = p_s[t];
      if (pj == 0.f) continue;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int d = lane * 4 + u * 128;
        if (d < p.Dv) {
          float4 vv = load4(vb + (int64_t)(j0 + t) * vrs + d);
          acc[u].x = fmaf(pj, vv.x, acc[u].x); acc[u].y = fmaf(pj, vv.y, acc[u].y);
          acc[u].z = fmaf(pj, vv.z, acc[u].z); acc[u].w = fmaf(pj, vv.w, acc[u].w);
        }
      }
    }
  }
  const float inv = (l > 0.f) ? 1.f / l : 0.f;
  T* o = static_cast<T*>(p.o) + row * p.Dv;
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int d = lane * 4 + u * 128;
    if (d < p.Dv) store4(o + d, make_float4(acc[u].x * inv, acc[u].y * inv, acc[u].z * inv, acc[u].w * inv));
  }
  if (lane == 0) p.lse[row] = (l > 0.f) ? m + logf(l) : -CUDART_INF_F;
}

template <typename T>
__global__ void __launch_bounds__(128) swa_bwd_dq_kernel(SwaParams p, int64_t rows) {
  extern __shared__ __align__(16) float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* q_s = smem + warp * (p.D + p.Dv + 32);
  float* do_s = q_s + p.D;
  float* ds_s = do_s + p.Dv;
  const int64_t row = (int64_t)blockIdx.x * 4 + warp;
  if (row >= rows) return;
  const int hq = (int)(row % p.h_q);
  const int64_t bi = row / p.h_q;
  const int i = (int)(bi % p.Lq);
  const int64_t b = bi / p.Lq;
  const int h = hq / (p.h_q / p.h_kv);
  const T* q = static_cast<const T*>(p.q) + row * p.D;
  const T* dO = static_cast<const T*>(p.d_o) + row * p.Dv;
  const T* orow = static_cast<const T*>(p.o) + row * p.Dv;
  float part = 0.f;
  for (int d = lane * 4; d < p.D; d += 128) *reinterpret_cast<float4*>(q_s + d) = load4(q + d);
  for (int d = lane * 4; d < p.Dv; d += 128) {
    float4 g = load4(dO + d), ov = load4(orow + d);
    *reinterpret_cast<float4*>(do_s + d) = g;
    part += g.x * ov.x + g.y * ov.y + g.z * ov.z + g.w * ov.w;
  }
  const float lse = p.lse[row];
  const float delta = warp_sum(part) - (p.d_lse ? p.d_lse[row] : 0.f);
  __syncwarp();
  int lo, hi;
  swa_range(p, i, lo, hi);
  const int64_t krs = (int64_t)p.h_kv * p.D, vrs = (int64_t)p.h_kv * p.Dv;
  const T* kb = static_cast<const T*>(p.k) + (b * p.Lk * p.h_kv + h) * p.D;
  const T* vb = static_cast<const T*>(p.v) + (b * p.Lk * p.h_kv + h) * p.Dv;
  float4 acc[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};
  if (lse > -CUDART_INF_F) {
    for (int j0 = lo; j0 <= hi; j0 += 32) {
      const int j = j0 + lane;
      float ds = 0.f;
      if (j <= hi && !swa_col_masked(p, j)) {
        const float pr = expf(dot_row(q_s, kb + (int64_t)j * krs, p.D) * p.scale - lse);
        const float dp = dot_row(do_s, vb + (int64_t)j * vrs, p.Dv);
        ds = pr * (dp - delta) * p.scale;
      }
      __syncwarp();
      ds_s[lane] = ds;
      __syncwarp();
      const int nj = min(32, hi - j0 + 1);
      for (int t = 0; t < nj; ++t) {
        const float d2 = ds_s[t];
        if (d2 == 0.f) continue;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int d = lane * 4 + u * 128;
          if (d < p.D) {
            float4 kv = load4(kb + (int64_t)(j0 + t) * krs + d);
            acc[u].x = fmaf(d2, kv.x, acc[u].x); acc[u].y = fmaf(d2, kv.y, acc[u].y);
            acc[u].z = fmaf(d2, kv.z, acc[u].z); acc[u].w = fmaf(d2, kv.w, acc[u].w);
          }
        }
      }
    }
  }
  T* o = static_cast<T*>(p.d_q) + row * p.D;
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int d = lane * 4 + u * 128;
    if (d < p.D) store4(o + d, acc[u]);
  }
}

// one warp per key row (b, j, h_kv): loops over the group's q-heads and over the queries that see j
template <typename T>
__global__ void __launch_bounds__(128) swa_bwd_dkv_kernel(SwaParams p, int64_t rows) {
  extern __shared__ __align__(16) float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* k_s = smem + warp * (p.D + p.Dv + 64);
  float* v_s = k_s + p.D;
  float* ds_s = v_s + p.Dv;
  float* pr_s = ds_s + 32;
  const int64_t row = (int64_t)blockIdx.x * 4 + warp;
  if (row >= rows) return;
  const int h = (int)(row % p.h_kv);
  const int64_t bj = row / p.h_kv;
  const int j = (int)(bj % p.Lk);
  const int64_t b = bj / p.Lk;
  const int G = p.h_q / p.h_kv;
  const T* kr = static_cast<const T*>(p.k) + row * p.D;
  const T* vr = static_cast<const T*>(p.v) + row * p.Dv;
  for (int d = lane * 4; d < p.D; d += 128) *reinterpret_cast<float4*>(k_s + d) = load4(kr + d);
  for (int d = lane * 4; d < p.Dv; d += 128) *reinterpret_cast<float4*>(v_s + d) = load4(vr + d);
  __syncwarp();
  float4 dk[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};
  float4 dv[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};
  // training layout: Lq == Lk, kv_start == 0, so query i sits at position i
  int i_hi = p.expand ? (j / p.S + 1) * p.S + p.W - 2 : j + p.W - 1;
  i_hi = min(i_hi, p.Lq - 1);
  if (!swa_col_masked(p, j)) {
    const int64_t qrs = (int64_t)p.h_q * p.D, ors = (int64_t)p.h_q * p.Dv;
    for (int g = 0; g < G; ++g) {
      const int hq = h * G + g;
      const T* qb = static_cast<const T*>(p.q) + (b * p.Lq * p.h_q + hq) * p.D;
      const T* dob = static_cast<const T*>(p.d_o) + (b * p.Lq * p.h_q + hq) * p.Dv;
      const T* ob = static_cast<const T*>(p.o) + (b * p.Lq * p.h_q + hq) * p.Dv;
      for (int i0 = j; i0 <= i_hi; i0 += 32) {
        const int i = i0 + lane;
        float pr = 0.f, ds = 0.f;
        if (i <= i_hi) {
          int lo, hi;
          swa_range(p, i, lo, hi);
          const int64_t lrow = (b * p.Lq + i) * p.h_q + hq;
          const float lse = p.lse[lrow];
          if (j >= lo && j <= hi && lse > -CUDART_INF_F) {
            pr = expf(dot_row(k_s, qb + (int64_t)i * qrs, p.D) * p.scale - lse);
            const float dp = dot_row(v_s, dob + (int64_t)i * ors, p.Dv);
            const float delta = dot_rows(ob + (int64_t)i * ors, dob + (int64_t)i * ors, p.Dv) -
                                (p.d_lse ? p.d_lse[lrow] : 0.f);
            ds = pr * (dp - delta) * p.scale;
          }
        }
        __syncwarp();
        ds_s[lane] = ds;
        pr_s[lane] = pr;
        __syncwarp();
        const int ni = min(32, i_hi - i0 + 1);
        for (int t = 0; t < ni; ++t) {
          const float d2 = ds_s[t], p2 = pr_s[t];
          if (d2 == 0.f && p2 == 0.f) continue;
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int d = lane * 4 + u * 128;
            if (d < p.D) {
              float4 qv = load4(qb + (int64_t)(i0 + t) * qrs + d);
              dk[u].x = fmaf(d2, qv.x, dk[u].x); dk[u].y = fmaf(d2, qv.y, dk[u].y);
              dk[u].z = fmaf(d2, qv.z, dk[u].z); dk[u].w = fmaf(d2, qv.w, dk[u].w);
            }
            if (d < p.Dv) {
              float4 gv = load4(dob + (int64_t)(i0 + t) * ors + d);
              dv[u].x = fmaf(p2, gv.x, dv[u].x); dv[u].y = fmaf(p2, gv.y, dv[u].y);
              dv[u].z = fmaf(p2, gv.z, dv[u].z); dv[u].w = fmaf(p2, gv.w, dv[u].w);
            }
          }
        }
      }
    }
  }
  T* dko = static_cast<T*>(p.d_k) + row * p.D;
  T* dvo = static_cast<T*>(p.d_v) + row * p.Dv;
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int d = lane * 4 + u * 128;
    if (d < p.D) store4(dko + d, dk[u]);
    if (d < p.Dv) store4(dvo + d, dv[u]);
  }
}

int swa_fwd_tc_launch(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Lq, int Lk, int h_q,
                      int h_kv, int D, int Dv, int W, int S, int mask_lmk, int expand, float scale, int kv_start,
                      cudaStream_t st);  // swa_tc.cu
int swa_decode_launch(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Lq, int Lk, int h_q,
                      int h_kv, int D, int Dv, int W, int S, int mask_lmk, int expand, float scale, int kv_start, int dtype,
                      cudaStream_t st);  // decode_attn.cu
size_t swa_bwd_tc_workspace(int B, int L, int h_q, int h_kv, int D, int Dv, int S);
int swa_bwd_tc_launch(const void* q, const void* k, const void* v, const void* o, const float* lse, const void* d_o,
                      const float* d_lse, void* d_q, void* d_k, void* d_v, void* workspace, int B, int L, int h_q, int h_kv,
                      int D, int Dv, int W, int S, int mask_lmk, int expand, float scale, cudaStream_t st);

static int check_swa(int B, int Lq, int Lk, int h_q, int h_kv, int D, int Dv, int S, int dtype) {
  HILS_REQUIRE(B > 0 && Lq >= 0 && Lk >= 0 && h_q > 0 && h_kv > 0 && D > 0 && Dv > 0 && S > 0, "swa: bad size");
  HILS_REQUIRE(h_q % h_kv == 0, "swa: h_q (%d) must be a multiple of h_kv (%d)", h_q, h_kv);
  HILS_REQUIRE(D % 4 == 0 && Dv % 4 == 0 && D <= 256 && Dv <= 256,
               "swa: head dims (%d, %d) must be multiples of 4 and <= 256", D, Dv);
  HILS_REQUIRE(dtype == HILS_F32 || dtype == HILS_BF16, "swa: unknown dtype %d", dtype);
  return HILS_OK;
}

}  // namespace hils

using namespace hils;

extern "C" int hils_swa_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Lq,
                            int Lk, int h_q, int h_kv, int D, int Dv, int window_size, int chunk_size,
                            int mask_lmk, int expand_to_chunk, float sm_scale, int kv_start, int dtype,
                            void* stream) {
  if (int rc = check_swa(B, Lq, Lk, h_q, h_kv, D, Dv, chunk_size, dtype)) return rc;
  HILS_REQUIRE(Lq <= Lk, "swa_fwd: Lq (%d) must not exceed Lk (%d)", Lq, Lk);
  if (Lq == 0) return HILS_OK;
  HILS_REQUIRE(q && k && v && o && lse, "swa_fwd: null pointer");
  if (Lq < Lk) {  // a few query rows against a long store: the streaming decode kernel
    const int rc = swa_decode_launch(q, k, v, o, lse, B, Lq, Lk, h_q, h_kv, D, Dv, window_size, chunk_size, mask_lmk,
                                     expand_to_chunk, sm_scale, kv_start, dtype, (cudaStream_t)stream);
    if (rc != HILS_ERR_UNSUPPORTED) return rc;
  }
  if (dtype == HILS_BF16) {  // tensor-core path for the shapes it covers
    const int rc = swa_fwd_tc_launch(q, k, v, o, lse, B, Lq, Lk, h_q, h_kv, D, Dv, window_size, chunk_size, mask_lmk,
                                     expand_to_chunk, sm_scale, kv_start, (cudaStream_t)stream);
    if (rc != HILS_ERR_UNSUPPORTED) return rc;
  }
  SwaParams p;
  p.q = q; p.k = k; p.v = v; p.o = o; p.lse = lse; p.d_o = nullptr; p.d_lse = nullptr;
  p.d_q = nullptr; p.d_k = nullptr; p.d_v = nullptr;
  p.B = B; p.Lq = Lq; p.Lk = Lk; p.h_q = h_q; p.h_kv = h_kv; p.D = D; p.Dv = Dv; p.W = window_size;
  p.S = chunk_size; p.mask_lmk = mask_lmk; p.expand = expand_to_chunk; p.kv_start = kv_start; p.scale = sm_scale;
  const int64_t rows = (int64_t)B * Lq * h_q;
  const size_t smem = 4 * (size_t)(D + 32) * sizeof(float);
  cudaStream_t st = (cudaStream_t)stream;
  const unsigned blocks = (unsigned)((rows + 3) / 4);
  if (dtype == HILS_BF16) swa_fwd_kernel<bf16><<<blocks, 128, smem, st>>>(p, rows);
  else swa_fwd_kernel<float><<<blocks, 128, smem, st>>>(p, rows);
  HILS_LAUNCH_CHECK("swa_fwd");
  return HILS_OK;
}

extern "C" size_t hils_swa_bwd_workspace_bytes(int B, int L, int h_q, int h_kv, int D, int Dv, int chunk_size, int dtype) {
  if (dtype != HILS_BF16 || h_q <= 0 || h_kv <= 0 || h_q % h_kv != 0) return 0;
  return swa_bwd_tc_workspace(B, L, h_q, h_kv, D, Dv, chunk_size);
}

extern "C" int hils_swa_bwd(const void* q, const void* k, const void* v, const void* o, const float* lse,
                            const void* d_o, const float* d_lse, void* d_q, void* d_k, void* d_v, int B, int L,
                            int h_q, int h_kv, int D, int Dv, int window_size, int chunk_size, int mask_lmk,
                            int expand_to_chunk, float sm_scale, int dtype, void* workspace, size_t workspace_bytes,
                            void* stream) {
  if (int rc = check_swa(B, L, L, h_q, h_kv, D, Dv, chunk_size, dtype)) return rc;
  if (L == 0) return HILS_OK;
  HILS_REQUIRE(q && k && v && o && lse && d_o && d_q && d_k && d_v, "swa_bwd: null pointer");
  if (dtype == HILS_BF16) {
    const size_t need = swa_bwd_tc_workspace(B, L, h_q, h_kv, D, Dv, chunk_size);
    if (need > 0) {
      if (!workspace || workspace_bytes < need) {
        set_error("swa_bwd: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
        return HILS_ERR_WORKSPACE;
      }
      const int rc = swa_bwd_tc_launch(q, k, v, o, lse, d_o, d_lse, d_q, d_k, d_v, workspace, B, L, h_q, h_kv, D, Dv,
                                       window_size, chunk_size, mask_lmk, expand_to_chunk, sm_scale, (cudaStream_t)stream);
      if (rc != HILS_ERR_UNSUPPORTED) return rc;
    }
  }
  SwaParams p;
  p.q = q; p.k = k; p.v = v; p.o = const_cast<void*>(o); p.lse = const_cast<float*>(lse); p.d_o = d_o;
  p.d_lse = d_lse; p.d_q = d_q; p.d_k = d_k; p.d_v = d_v;
  p.B = B; p.Lq = L; p.Lk = L; p.h_q = h_q; p.h_kv = h_kv; p.D = D; p.Dv = Dv; p.W = window_size;
  p.S = chunk_size; p.mask_lmk = mask_lmk; p.expand = expand_to_chunk; p.kv_start = 0; p.scale = sm_scale;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t rows_q = (int64_t)B * L * h_q, rows_k = (int64_t)B * L * h_kv;
  const size_t smem_q = 4 * (size_t)(D + Dv + 32) * sizeof(float);
  const size_t smem_k = 4 * (size_t)(D + Dv + 64) * sizeof(float);
  if (dtype == HILS_BF16) {
    swa_bwd_dq_kernel<bf16><<<(unsigned)((rows_q + 3) / 4), 128, smem_q, st>>>(p, rows_q);
    swa_bwd_dkv_kernel<bf16><<<(unsigned)((rows_k + 3) / 4), 128, smem_k, st>>>(p, rows_k);
  } else {
    swa_bwd_dq_kernel<float><<<(unsigned)((rows_q + 3) / 4), 128, smem_q, st>>>(p, rows_q);
    swa_bwd_dkv_kernel<float><<<(unsigned)((rows_k + 3) / 4), 128, smem_k, st>>>(p, rows_k);
  }
  HILS_LAUNCH_CHECK("swa_bwd");
  return HILS_OK;
}
