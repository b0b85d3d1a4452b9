// Exact per-chunk log Z (the chunk mass the naive block-sparse baseline selects on) and its
// gradients, exact-fp32 CUDA-core form: one warp per output row.
//
// Contract (ops/exact_chunk_log_z_tilelang.py:89-112 forward, :229-254 dQ, :358-383 dK):
//   logZ[b,i,h,c] = logsumexp_{j in [cS,(c+1)S), j<=i, j<L [, (j+1)%S != 0]} scale <q_i, k_j>
//   defined only when i >= (c+1)S + W - 1, else -inf;   N_chunk = ceil(L/S)
//   dS_ij = dlogZ[i,c(j)] exp(s_ij - logZ[i,c(j)]) scale;  dQ = dS K;  dK = dS^T Q (summed over the group)
#include "common.cuh"

namespace hils {

int logz_fwd_tc_launch(const void* q, const void* k, float* log_z, int B, int L, int h_q, int h_kv, int D, int chunk_size,
                       int window_size, float sm_scale, int mask_lmk, cudaStream_t st);   // logz_tc.cu

int logz_bwd_tc_launch(const void* q, const void* k, const float* log_z, const float* d_log_z, void* d_q, void* d_k, int B, int L,
                       int h_q, int h_kv, int D, int chunk_size, int window_size, float sm_scale, cudaStream_t st);   // logz_tc.cu

struct LogzParams {
  const void* q; const void* k; float* log_z; const float* d_log_z; void* d_q; void* d_k;
  int B, L, h_q, h_kv, D, S, W, mask_lmk, n_chunk;
  float scale;
};

template <typename T>
__global__ void __launch_bounds__(128) logz_fwd_kernel(LogzParams p, int64_t rows) {
  extern __shared__ __align__(16) float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* q_s = smem + warp * p.D;
  const int64_t row = (int64_t)blockIdx.x * 4 + warp;  // (b, i, hq)
  if (row >= rows) return;
  const int hq = (int)(row % p.h_q);
  const int64_t bi = row / p.h_q;
  const int i = (int)(bi % p.L);
  const int64_t b = bi / p.L;
  const int h = hq / (p.h_q / p.h_kv);
  const T* q = static_cast<const T*>(p.q) + row * p.D;
  for (int d = lane * 4; d < p.D; d += 128) *reinterpret_cast<float4*>(q_s + d) = load4(q + d);
  __syncwarp();
  float* out = p.log_z + row * p.n_chunk;
  const int64_t krs = (int64_t)p.h_kv * p.D;
  const T* kb = static_cast<const T*>(p.k) + (b * p.L * p.h_kv + h) * p.D;
  for (int c = 0; c < p.n_chunk; ++c) {
    float res = -CUDART_INF_F;
    if (i >= (c + 1) * p.S + p.W - 1) {
      float m = -CUDART_INF_F, sum = 0.f;
      for (int j0 = 0; j0 < p.S; j0 += 32) {
        const int jj = j0 + lane, j = c * p.S + jj;
        float s = -CUDART_INF_F;
        if (jj < p.S && j <= i && j < p.L && !(p.mask_lmk && ((j + 1) % p.S == 0)))
          s = dot_row(q_s, kb + (int64_t)j * krs, p.D) * p.scale;
        const float mn = fmaxf(m, warp_max(s));
        if (mn > -CUDART_INF_F) {
          const float e = warp_sum(expf(s - mn));
          sum = sum * ((m > -CUDART_INF_F) ? expf(m - mn) : 0.f) + e;
          m = mn;
        }
      }
      if (sum > 0.f) res = m + logf(sum);
    }
    if (lane == 0) out[c] = res;
  }
}

template <typename T>
__global__ void __launch_bounds__(128) logz_bwd_dq_kernel(LogzParams p, int64_t rows) {
  extern __shared__ __align__(16) float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* q_s = smem + warp * (p.D + 32);
  float* ds_s = q_s + p.D;
  const int64_t row = (int64_t)blockIdx.x * 4 + warp;
  if (row >= rows) return;
  const int hq = (int)(row % p.h_q);
  const int64_t bi = row / p.h_q;
  const int i = (int)(bi % p.L);
  const int64_t b = bi / p.L;
  const int h = hq / (p.h_q / p.h_kv);
  const T* q = static_cast<const T*>(p.q) + row * p.D;
  for (int d = lane * 4; d < p.D; d += 128) *reinterpret_cast<float4*>(q_s + d) = load4(q + d);
  __syncwarp();
  const float* lz = p.log_z + row * p.n_chunk;
  const float* dlz = p.d_log_z + row * p.n_chunk;
  const int64_t krs = (int64_t)p.h_kv * p.D;
  const T* kb = static_cast<const T*>(p.k) + (b * p.L * p.h_kv + h) * p.D;
  float4 acc[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};
  for (int c = 0; c < p.n_chunk; ++c) {
    if (i < (c + 1) * p.S + p.W - 1) break;  // later chunks are not remote either
    const float z = lz[c], g = dlz[c];
    if (!(z > -CUDART_INF_F) || g == 0.f) continue;
    for (int j0 = 0; j0 < p.S; j0 += 32) {
      const int jj = j0 + lane, j = c * p.S + jj;
      float ds = 0.f;
      if (jj < p.S && j <= i && j < p.L)
        ds = g * expf(dot_row(q_s, kb + (int64_t)j * krs, p.D) * p.scale - z) * p.scale;
      __syncwarp();
      ds_s[lane] = ds;
      __syncwarp();
      const int nj = min(32, p.S - j0);
      for (int t = 0; t < nj; ++t) {
        const int j2 = c * p.S + j0 + t;
        if (j2 >= p.L) break;
        const float d2 = ds_s[t];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int d = lane * 4 + u * 128;
          if (d < p.D) {
            float4 kv = load4(kb + (int64_t)j2 * krs + d);
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

template <typename T>
__global__ void __launch_bounds__(128) logz_bwd_dk_kernel(LogzParams p, int64_t rows) {
  extern __shared__ __align__(16) float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* k_s = smem + warp * (p.D + 32);
  float* cf_s = k_s + p.D;
  const int64_t row = (int64_t)blockIdx.x * 4 + warp;  // (b, j, h_kv)
  if (row >= rows) return;
  const int h = (int)(row % p.h_kv);
  const int64_t bj = row / p.h_kv;
  const int j = (int)(bj % p.L);
  const int64_t b = bj / p.L;
  const int G = p.h_q / p.h_kv;
  const T* kr = static_cast<const T*>(p.k) + row * p.D;
  for (int d = lane * 4; d < p.D; d += 128) *reinterpret_cast<float4*>(k_s + d) = load4(kr + d);
  __syncwarp();
  const int c = j / p.S;
  const int i_min = (c + 1) * p.S + p.W - 1;
  const int64_t qrs = (int64_t)p.h_q * p.D;
  float4 acc[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};
  for (int g = 0; g < G; ++g) {
    const int hq = h * G + g;
    const T* qb = static_cast<const T*>(p.q) + (b * p.L * p.h_q + hq) * p.D;
    for (int i0 = i_min; i0 < p.L; i0 += 32) {
      const int i = i0 + lane;
      float cf = 0.f;
      if (i < p.L) {
        const int64_t zo = ((b * p.L + i) * p.h_q + hq) * p.n_chunk + c;
        const float z = p.log_z[zo], gz = p.d_log_z[zo];
        if (z > -CUDART_INF_F && gz != 0.f)
          cf = gz * expf(dot_row(k_s, qb + (int64_t)i * qrs, p.D) * p.scale - z) * p.scale;
      }
      __syncwarp();
      cf_s[lane] = cf;
      __syncwarp();
      const int ni = min(32, p.L - i0);
      for (int t = 0; t < ni; ++t) {
        const float c2 = cf_s[t];
        if (c2 == 0.f) continue;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int d = lane * 4 + u * 128;
          if (d < p.D) {
            float4 qv = load4(qb + (int64_t)(i0 + t) * qrs + d);
            acc[u].x = fmaf(c2, qv.x, acc[u].x); acc[u].y = fmaf(c2, qv.y, acc[u].y);
            acc[u].z = fmaf(c2, qv.z, acc[u].z); acc[u].w = fmaf(c2, qv.w, acc[u].w);
          }
        }
      }
    }
  }
  T* o = static_cast<T*>(p.d_k) + row * p.D;
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int d = lane * 4 + u * 128;
    if (d < p.D) store4(o + d, acc[u]);
  }
}

static int check_logz(int B, int L, int h_q, int h_kv, int D, int S, int dtype) {
  HILS_REQUIRE(B > 0 && L >= 0 && h_q > 0 && h_kv > 0 && D > 0 && S > 0, "chunk_logz: bad size");
  HILS_REQUIRE(h_q % h_kv == 0, "chunk_logz: h_q (%d) must be a multiple of h_kv (%d)", h_q, h_kv);
  HILS_REQUIRE(D % 4 == 0 && D <= 256, "chunk_logz: D (%d) must be a multiple of 4 and <= 256", D);
  HILS_REQUIRE(dtype == HILS_F32 || dtype == HILS_BF16, "chunk_logz: unknown dtype %d", dtype);
  return HILS_OK;
}

}  // namespace hils

using namespace hils;

extern "C" int hils_chunk_logz_fwd(const void* q, const void* k, float* log_z, int B, int L, int h_q, int h_kv,
                                   int D, int chunk_size, int window_size, float sm_scale, int mask_lmk,
                                   int dtype, void* stream) {
  if (int rc = check_logz(B, L, h_q, h_kv, D, chunk_size, dtype)) return rc;
  if (L == 0) return HILS_OK;
  HILS_REQUIRE(q && k && log_z, "chunk_logz_fwd: null pointer");
  LogzParams p;
  p.q = q; p.k = k; p.log_z = log_z; p.d_log_z = nullptr; p.d_q = nullptr; p.d_k = nullptr;
  p.B = B; p.L = L; p.h_q = h_q; p.h_kv = h_kv; p.D = D; p.S = chunk_size; p.W = window_size;
  p.mask_lmk = mask_lmk; p.n_chunk = ceil_div(L, chunk_size); p.scale = sm_scale;
  const int64_t rows = (int64_t)B * L * h_q;
  const size_t smem = 4 * (size_t)D * sizeof(float);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == HILS_BF16) {   // chunk size 64 on the tensor cores
    const int rc = logz_fwd_tc_launch(q, k, log_z, B, L, h_q, h_kv, D, chunk_size, window_size, sm_scale, mask_lmk, st);
    if (rc != HILS_ERR_UNSUPPORTED) return rc;
  }
  const unsigned blocks = (unsigned)((rows + 3) / 4);
  if (dtype == HILS_BF16) logz_fwd_kernel<bf16><<<blocks, 128, smem, st>>>(p, rows);
  else logz_fwd_kernel<float><<<blocks, 128, smem, st>>>(p, rows);
  HILS_LAUNCH_CHECK("chunk_logz_fwd");
  return HILS_OK;
}

extern "C" int hils_chunk_logz_bwd(const void* q, const void* k, const float* log_z, const float* d_log_z,
                                   void* d_q, void* d_k, int B, int L, int h_q, int h_kv, int D, int chunk_size,
                                   int window_size, float sm_scale, int dtype, void* stream) {
  if (int rc = check_logz(B, L, h_q, h_kv, D, chunk_size, dtype)) return rc;
  if (L == 0) return HILS_OK;
  HILS_REQUIRE(q && k && log_z && d_log_z && d_q && d_k, "chunk_logz_bwd: null pointer");
  LogzParams p;
  p.q = q; p.k = k; p.log_z = const_cast<float*>(log_z); p.d_log_z = d_log_z; p.d_q = d_q; p.d_k = d_k;
  p.B = B; p.L = L; p.h_q = h_q; p.h_kv = h_kv; p.D = D; p.S = chunk_size; p.W = window_size;
  p.mask_lmk = 0; p.n_chunk = ceil_div(L, chunk_size); p.scale = sm_scale;
  const size_t smem = 4 * (size_t)(D + 32) * sizeof(float);
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t rows_q = (int64_t)B * L * h_q, rows_k = (int64_t)B * L * h_kv;
  if (dtype == HILS_BF16) {   // chunk size 64 on the tensor cores
    const int rc = logz_bwd_tc_launch(q, k, log_z, d_log_z, d_q, d_k, B, L, h_q, h_kv, D, chunk_size, window_size, sm_scale, st);
    if (rc != HILS_ERR_UNSUPPORTED) return rc;
  }
  if (dtype == HILS_BF16) {
    logz_bwd_dq_kernel<bf16><<<(unsigned)((rows_q + 3) / 4), 128, smem, st>>>(p, rows_q);
    logz_bwd_dk_kernel<bf16><<<(unsigned)((rows_k + 3) / 4), 128, smem, st>>>(p, rows_k);
  } else {
    logz_bwd_dq_kernel<float><<<(unsigned)((rows_q + 3) / 4), 128, smem, st>>>(p, rows_q);
    logz_bwd_dk_kernel<float><<<(unsigned)((rows_k + 3) / 4), 128, smem, st>>>(p, rows_k);
  }
  HILS_LAUNCH_CHECK("chunk_logz_bwd");
  return HILS_OK;
}
