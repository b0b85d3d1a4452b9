// Chunk pooling kernels: attention pooling of each chunk with its landmark query (forward and
// backward) and plain mean pooling.  HBM-streaming: one CTA per (chunk, kv-head, batch) reads the
// chunk's [S x D] key tile exactly once and serves every q-head of the GQA group from it.
//
// Math (ops/chunk_attn_pool_tilelang.py:364-408 forward, :478-531 backward; torch form :693-717):
//   l_j = scale <mu, K_j> (j < S-1), l_{S-1} = -inf;  p = softmax(l);  k' = sum_j p_j K_j;
//   b' = -sum_{p_j>0} p_j ln p_j
//   dP_j = <g_k', K_j>; delta = sum p_j dP_j; dl_j = p_j[(dP_j - delta) - g_b'(ln p_j + b')]
//   dmu = scale sum_j dl_j K_j;  dK_j = scale dl_j mu + p_j g_k'
#include "common.cuh"
#include "mma_rows.cuh"

namespace hils {

template <typename T>
__global__ void __launch_bounds__(128) pool_fwd_kernel(
    const T* __restrict__ mu_q, const T* __restrict__ k, T* __restrict__ lmk_k, float* __restrict__ lmk_b,
    int N, int S, int h_q, int h_kv, int D, int64_t k_batch_stride, float scale, int compact) {
  extern __shared__ __align__(16) float smem[];
  float* Ks = smem;              // [S][D]
  float* mu_s = Ks + S * D;      // [D]
  float* l_s = mu_s + D;         // [S] logits, then probabilities
  const int n = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int G = h_q / h_kv;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const T* kbase = k + (int64_t)b * k_batch_stride + ((int64_t)n * S * h_kv + h) * D;
  for (int idx = tid * 4; idx < S * D; idx += 128 * 4) {
    int j = idx / D, d = idx - j * D;
    store4(Ks + idx, load4(kbase + (int64_t)j * h_kv * D + d));
  }
  for (int g = 0; g < G; ++g) {
    const int hq = h * G + g;
    const int64_t orow = ((int64_t)b * N + n) * h_q + hq;
    __syncthreads();
    for (int d = tid; d < D; d += 128) mu_s[d] = to_f(mu_q[orow * D + d]);
    __syncthreads();
    for (int j = warp; j < S; j += 4) {
      float acc = 0.f;
      for (int d = lane; d < D; d += 32) acc = fmaf(mu_s[d], Ks[j * D + d], acc);
      acc = warp_sum(acc);
      if (lane == 0) l_s[j] = (j == S - 1) ? -CUDART_INF_F : acc * scale;
    }
    __syncthreads();
    float m = -CUDART_INF_F;
    for (int j = lane; j < S; j += 32) m = fmaxf(m, l_s[j]);
    m = warp_max(m);
    float sum = 0.f;
    if (m > -CUDART_INF_F)
      for (int j = lane; j < S; j += 32) sum += __expf(l_s[j] - m);
    sum = warp_sum(sum);
    const float log_sum = (sum > 0.f) ? __logf(sum) : 0.f;
    float ent = 0.f;
    for (int j = lane; j < S; j += 32) {
      float lj = l_s[j];
      float p = (sum > 0.f && lj > -CUDART_INF_F) ? __expf(lj - m) / sum : 0.f;
      if (p > 0.f) ent -= p * ((lj - m) - log_sum);
    }
    ent = warp_sum(ent);
    __syncthreads();
    for (int j = tid; j < S; j += 128) {
      float lj = l_s[j];
      l_s[j] = (sum > 0.f && lj > -CUDART_INF_F) ? __expf(lj - m) / sum : 0.f;
    }
    __syncthreads();
    if (tid == 0) lmk_b[orow] = ent;
    for (int d = tid; d < D; d += 128) {
      float acc = 0.f;
      if (!compact)
        for (int j = 0; j < S; ++j) acc = fmaf(l_s[j], Ks[j * D + d], acc);
      lmk_k[orow * D + d] = from_f<T>(acc);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(128) pool_bwd_kernel(
    const T* __restrict__ mu_q, const T* __restrict__ k, const T* __restrict__ g_lmk_k,
    const float* __restrict__ g_lmk_b, T* __restrict__ d_mu_q, T* __restrict__ d_k,
    int N, int S, int h_q, int h_kv, int D, int64_t k_batch_stride, float scale, int compact) {
  extern __shared__ __align__(16) float smem[];
  float* Ks = smem;               // [S][D]
  float* dKs = Ks + S * D;        // [S][D] gradient of the tile, summed over the GQA group
  float* mu_s = dKs + S * D;      // [D]
  float* gk_s = mu_s + D;         // [D]
  float* l_s = gk_s + D;          // [S] logits -> p
  float* dl_s = l_s + S;          // [S]
  const int n = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int G = h_q / h_kv;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const T* kbase = k + (int64_t)b * k_batch_stride + ((int64_t)n * S * h_kv + h) * D;
  for (int idx = tid * 4; idx < S * D; idx += 128 * 4) {
    int j = idx / D, d = idx - j * D;
    store4(Ks + idx, load4(kbase + (int64_t)j * h_kv * D + d));
    store4(dKs + idx, make_float4(0.f, 0.f, 0.f, 0.f));
  }
  for (int g = 0; g < G; ++g) {
    const int hq = h * G + g;
    const int64_t orow = ((int64_t)b * N + n) * h_q + hq;
    const float gb = g_lmk_b ? g_lmk_b[orow] : 0.f;
    __syncthreads();
    for (int d = tid; d < D; d += 128) {
      mu_s[d] = to_f(mu_q[orow * D + d]);
      gk_s[d] = (g_lmk_k && !compact) ? to_f(g_lmk_k[orow * D + d]) : 0.f;
    }
    __syncthreads();
    for (int j = warp; j < S; j += 4) {
      float acc = 0.f, acc2 = 0.f;
      for (int d = lane; d < D; d += 32) {
        float kv = Ks[j * D + d];
        acc = fmaf(mu_s[d], kv, acc);
        acc2 = fmaf(gk_s[d], kv, acc2);
      }
      acc = warp_sum(acc);
      acc2 = warp_sum(acc2);
      if (lane == 0) {
        l_s[j] = (j == S - 1) ? -CUDART_INF_F : acc * scale;
        dl_s[j] = acc2;  // dP_j for now
      }
    }
    __syncthreads();
    float m = -CUDART_INF_F;
    for (int j = lane; j < S; j += 32) m = fmaxf(m, l_s[j]);
    m = warp_max(m);
    float sum = 0.f;
    if (m > -CUDART_INF_F)
      for (int j = lane; j < S; j += 32) sum += __expf(l_s[j] - m);
    sum = warp_sum(sum);
    const float log_sum = (sum > 0.f) ? __logf(sum) : 0.f;
    float ent = 0.f, delta = 0.f;
    for (int j = lane; j < S; j += 32) {
      float lj = l_s[j];
      float p = (sum > 0.f && lj > -CUDART_INF_F) ? __expf(lj - m) / sum : 0.f;
      if (p > 0.f) ent -= p * ((lj - m) - log_sum);
      delta = fmaf(p, dl_s[j], delta);
    }
    ent = warp_sum(ent);
    delta = warp_sum(delta);
    __syncthreads();
    for (int j = tid; j < S; j += 128) {
      float lj = l_s[j];
      float p = (sum > 0.f && lj > -CUDART_INF_F) ? __expf(lj - m) / sum : 0.f;
      float dl = 0.f;
      if (p > 0.f) dl = p * ((dl_s[j] - delta) - gb * (((lj - m) - log_sum) + ent));
      l_s[j] = p;
      dl_s[j] = dl;
    }
    __syncthreads();
    for (int d = tid; d < D; d += 128) {
      float acc = 0.f;
      for (int j = 0; j < S; ++j) acc = fmaf(dl_s[j], Ks[j * D + d], acc);
      d_mu_q[orow * D + d] = from_f<T>(acc * scale);
    }
    for (int idx = tid; idx < S * D; idx += 128) {
      int j = idx / D, d = idx - j * D;
      dKs[idx] += scale * dl_s[j] * mu_s[d] + l_s[j] * gk_s[d];
    }
  }
  __syncthreads();
  T* obase = d_k + ((((int64_t)b * N + n) * S) * h_kv + h) * D;
  for (int idx = tid * 4; idx < S * D; idx += 128 * 4) {
    int j = idx / D, d = idx - j * D;
    store4(obase + (int64_t)j * h_kv * D + d, *reinterpret_cast<float4*>(dKs + idx));
  }
}

// mean over the S tokens of each chunk; one thread per 4 output elements, coalesced over (h, d)
template <typename T>
__global__ void meanpool_fwd_kernel(const T* __restrict__ k, T* __restrict__ out, int N, int S,
                                    int HD, int64_t k_batch_stride, int64_t total4) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total4) return;
  int hd4 = HD / 4;
  int c = (int)(i % hd4);
  int64_t bn = i / hd4;
  int n = (int)(bn % N);
  int64_t b = bn / N;
  const T* p = k + b * k_batch_stride + (int64_t)n * S * HD + c * 4;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int j = 0; j < S; ++j) {
    float4 x = load4(p + (int64_t)j * HD);
    acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
  }
  float inv = 1.f / (float)S;
  store4(out + bn * HD + c * 4, make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv));
}

template <typename T>
__global__ void meanpool_bwd_kernel(const T* __restrict__ g_out, T* __restrict__ d_k, int S, int HD,
                                    int64_t total4) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total4) return;
  int hd4 = HD / 4;
  int c = (int)(i % hd4);
  int64_t bns = i / hd4;
  int64_t bn = bns / S;
  float4 g = load4(g_out + bn * HD + c * 4);
  float inv = 1.f / (float)S;
  store4(d_k + bns * HD + c * 4, make_float4(g.x * inv, g.y * inv, g.z * inv, g.w * inv));
}

// =================================================================================================
// bf16 fast path (S <= 64, D = 64 or 128, G <= 8): one WARP per (chunk, kv-head).  Scores come from
// mma.sync with the B fragments loaded straight from the chunk's key rows (mma_rows.cuh), the weighted
// key sums run on the CUDA cores with 16-byte row loads.  Nothing is staged in shared memory beyond the
// 64 logits of the chunk, no block-wide barrier is needed, and a CTA of eight warps keeps eight 8-16 KB
// tiles in flight - the generic kernel above holds one tile per CTA and synchronises ~8 times per head.
// =================================================================================================
constexpr int kPoolWarps = 8;

// logits in pw[g*64 + j] (raw dots) -> probabilities in place; returns the entropy b' (all lanes)
__device__ __forceinline__ float pool_softmax_row(float* pw, int S, float scale, int lane, float* m_out, float* logsum_out) {
  const int j0 = lane, j1 = lane + 32;
  const float l0 = (j0 < S - 1) ? pw[j0] * scale : -CUDART_INF_F;
  const float l1 = (j1 < S - 1) ? pw[j1] * scale : -CUDART_INF_F;
  const float m = warp_max(fmaxf(l0, l1));
  float e0 = 0.f, e1 = 0.f;
  if (m > -CUDART_INF_F) { e0 = __expf(l0 - m); e1 = __expf(l1 - m); }
  const float sum = warp_sum(e0 + e1);
  const float log_sum = (sum > 0.f) ? __logf(sum) : 0.f;
  const float p0 = (sum > 0.f) ? e0 / sum : 0.f, p1 = (sum > 0.f) ? e1 / sum : 0.f;
  float ent = 0.f;
  if (p0 > 0.f) ent -= p0 * ((l0 - m) - log_sum);
  if (p1 > 0.f) ent -= p1 * ((l1 - m) - log_sum);
  ent = warp_sum(ent);
  pw[j0] = p0;
  pw[j1] = p1;
  *m_out = m;
  *logsum_out = log_sum;
  return ent;
}

// The whole [S x D] key tile of a warp is requested from HBM at once (one L2 prefetch per 128-byte line, spread over the
// lanes): the products below then find their rows in L2.  Without it a warp has only the few rows of its current
// fragment loads in flight, and a kernel of one-tile warps cannot cover the latency of HBM (c3: 183 -> 168 us forward,
// 375 -> 327 us backward).  Persistent warps that prefetch their next tile while working on the current one were
// slower (230 / 441 us): an oversubscribed grid of one-tile warps keeps more tiles in flight.
template <int D>
__device__ __forceinline__ void prefetch_tile_l2(const bf16* kbase, int64_t row_stride, int S, int lane) {
  constexpr int LPRW = D * 2 / 128;                      // 128-byte lines per row
  for (int i = lane; i < S * LPRW; i += 32) {
    const bf16* a = kbase + (int64_t)(i / LPRW) * row_stride + (i % LPRW) * 64;
    asm volatile("prefetch.global.L2 [%0];" ::"l"(a));
  }
}

template <int NK, int GM>
__global__ void __launch_bounds__(32 * kPoolWarps, 3) pool_fwd_bf16_kernel(
    const bf16* __restrict__ mu_q, const bf16* __restrict__ k, bf16* __restrict__ lmk_k, float* __restrict__ lmk_b,
    int N, int S, int h_q, int h_kv, int64_t k_batch_stride, float scale, int compact) {
  constexpr int D = NK * 16, LPR = 2 * NK;
  extern __shared__ __align__(16) float smem[];
  const int G = h_q / h_kv;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* q_s = smem + warp * (G * D + G * 64);           // [G][D] landmark queries
  float* pw = q_s + G * D;                               // [G][64] logits -> probabilities
  const int n = blockIdx.x * kPoolWarps + warp, h = blockIdx.y, b = blockIdx.z;
  if (n >= N) return;
  const bf16* kbase = k + (int64_t)b * k_batch_stride + ((int64_t)n * S * h_kv + h) * D;
  const int64_t rs = (int64_t)h_kv * D;
  prefetch_tile_l2<D>(kbase, rs, S, lane);
  const int64_t orow0 = ((int64_t)b * N + n) * h_q + h * G;
  for (int i = lane; i < G * D; i += 32) q_s[i] = to_f(mu_q[orow0 * D + i]);
  __syncwarp();
  uint32_t af[NK][4];
  make_q_frags<NK>(q_s, lane, af, [G](int r) { return r < G ? r : -1; });
  score_rows_mma<NK>(af, kbase, rs, S, G, pw, 64, lane);
  __syncwarp();
  for (int g = 0; g < G; ++g) {
    float m, ls;
    const float ent = pool_softmax_row(pw + g * 64, S, scale, lane, &m, &ls);
    if (lane == 0) lmk_b[orow0 + g] = ent;
  }
  __syncwarp();
  float acc[GM][8];
#pragma unroll
  for (int g = 0; g < GM; ++g)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[g][e] = 0.f;
  if (!compact) {
    pv_rows16<NK, GM>(pw, 64, kbase, rs, S, G, acc, lane);
    pv_reduce<NK, GM>(acc);
  }
  if (lane < LPR)
#pragma unroll
    for (int g = 0; g < GM; ++g)
      if (g < G) {
        uint4 o;
        o.x = pack_bf16(acc[g][0], acc[g][1]); o.y = pack_bf16(acc[g][2], acc[g][3]);
        o.z = pack_bf16(acc[g][4], acc[g][5]); o.w = pack_bf16(acc[g][6], acc[g][7]);
        *reinterpret_cast<uint4*>(lmk_k + (orow0 + g) * D + lane * 8) = o;
      }
}

// backward: fragment rows 0..G-1 = landmark queries, rows G..2G-1 = g_k' (so one pass over the tile gives
// both the logits and dP); then dmu = scale * sum_j dl_j K_j (row loads) and the dK tile, written once.
template <int NK, int GM>
__global__ void __launch_bounds__(32 * kPoolWarps) pool_bwd_bf16_kernel(
    const bf16* __restrict__ mu_q, const bf16* __restrict__ k, const bf16* __restrict__ g_lmk_k,
    const float* __restrict__ g_lmk_b, bf16* __restrict__ d_mu_q, bf16* __restrict__ d_k, int N, int S, int h_q,
    int h_kv, int64_t k_batch_stride, float scale, int compact) {
  constexpr int D = NK * 16, LPR = 2 * NK, RPI = 32 / LPR;
  extern __shared__ __align__(16) float smem[];
  const int G = h_q / h_kv;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* q_s = smem + warp * (2 * G * D + 2 * G * 64);   // [2G][D]: mu rows, then g_k' rows
  float* pw = q_s + 2 * G * D;                           // [2G][64]: logits -> p, dP -> dl
  const int n = blockIdx.x * kPoolWarps + warp, h = blockIdx.y, b = blockIdx.z;
  if (n >= N) return;
  prefetch_tile_l2<D>(k + (int64_t)b * k_batch_stride + ((int64_t)n * S * h_kv + h) * D, (int64_t)h_kv * D, S, lane);
  const int64_t orow0 = ((int64_t)b * N + n) * h_q + h * G;
  const bool has_gk = g_lmk_k != nullptr && !compact;
  for (int i = lane; i < G * D; i += 32) {
    q_s[i] = to_f(mu_q[orow0 * D + i]);
    q_s[G * D + i] = has_gk ? to_f(g_lmk_k[orow0 * D + i]) : 0.f;
  }
  __syncwarp();
  uint32_t af[NK][4];
  make_q_frags<NK>(q_s, lane, af, [G](int r) { return r < 2 * G ? r : -1; });
  const bf16* kbase = k + (int64_t)b * k_batch_stride + ((int64_t)n * S * h_kv + h) * D;
  bf16* dkbase = d_k + (int64_t)b * k_batch_stride + ((int64_t)n * S * h_kv + h) * D;
  const int64_t rs = (int64_t)h_kv * D;
  score_rows_mma<NK>(af, kbase, rs, S, 2 * G, pw, 64, lane);
  __syncwarp();
  for (int g = 0; g < G; ++g) {
    float* pg = pw + g * 64;
    float* dg = pw + (G + g) * 64;
    const int j0 = lane, j1 = lane + 32;
    const float l0 = (j0 < S - 1) ? pg[j0] * scale : -CUDART_INF_F;
    const float l1 = (j1 < S - 1) ? pg[j1] * scale : -CUDART_INF_F;
    float m, log_sum;
    const float ent = pool_softmax_row(pg, S, scale, lane, &m, &log_sum);
    const float p0 = pg[j0], p1 = pg[j1];
    const float dp0 = (j0 < S) ? dg[j0] : 0.f, dp1 = (j1 < S) ? dg[j1] : 0.f;
    const float delta = warp_sum(p0 * dp0 + p1 * dp1);
    const float gb = g_lmk_b ? g_lmk_b[orow0 + g] : 0.f;
    // ln p_j = (l_j - m) - log_sum
    dg[j0] = (p0 > 0.f) ? p0 * ((dp0 - delta) - gb * (((l0 - m) - log_sum) + ent)) : 0.f;
    dg[j1] = (p1 > 0.f) ? p1 * ((dp1 - delta) - gb * (((l1 - m) - log_sum) + ent)) : 0.f;
  }
  __syncwarp();
  // dmu_g = scale * sum_j dl_{g,j} K_j
  {
    float acc[GM][8];
#pragma unroll
    for (int g = 0; g < GM; ++g)
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[g][e] = 0.f;
    pv_rows16<NK, GM>(pw + G * 64, 64, kbase, rs, S, G, acc, lane);
    pv_reduce<NK, GM>(acc);
    if (lane < LPR)
#pragma unroll
      for (int g = 0; g < GM; ++g)
        if (g < G) {
          uint4 o;
          o.x = pack_bf16(acc[g][0] * scale, acc[g][1] * scale); o.y = pack_bf16(acc[g][2] * scale, acc[g][3] * scale);
          o.z = pack_bf16(acc[g][4] * scale, acc[g][5] * scale); o.w = pack_bf16(acc[g][6] * scale, acc[g][7] * scale);
          *reinterpret_cast<uint4*>(d_mu_q + (orow0 + g) * D + lane * 8) = o;
        }
  }
  // dK_j = sum_g (scale * dl_{g,j} mu_g + p_{g,j} g_k'_g): D/8 lanes per key row, 32/(D/8) rows per step
  const int sub = lane % LPR, rg = lane / LPR;
  for (int j0 = 0; j0 < S; j0 += RPI) {
    const int j = j0 + rg;
    if (j < S) {
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = 0.f;
      for (int g = 0; g < G; ++g) {
        const float a = scale * pw[(G + g) * 64 + j], pj = pw[g * 64 + j];
        const float* mu = q_s + g * D + sub * 8;
        const float* gk = q_s + (G + g) * D + sub * 8;
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = fmaf(a, mu[e], fmaf(pj, gk[e], o[e]));
      }
      uint4 w4;
      w4.x = pack_bf16(o[0], o[1]); w4.y = pack_bf16(o[2], o[3]); w4.z = pack_bf16(o[4], o[5]); w4.w = pack_bf16(o[6], o[7]);
      *reinterpret_cast<uint4*>(dkbase + (int64_t)j * rs + sub * 8) = w4;
    }
  }
}

static bool pool_bf16_ok(const void* mu_q, const void* k, int S, int h_q, int h_kv, int D, int64_t k_batch_stride) {
  const int G = h_q / h_kv;
  return S >= 2 && S <= 64 && (D == 64 || D == 128) && G <= 8 && (k_batch_stride % 8) == 0 &&
         ((((uintptr_t)mu_q) | ((uintptr_t)k)) & 15) == 0;
}

static int check_pool_args(int B, int N, int S, int h_q, int h_kv, int D, int dtype) {
  HILS_REQUIRE(B > 0 && N >= 0 && S > 0 && h_q > 0 && h_kv > 0 && D > 0, "pool: non-positive size");
  HILS_REQUIRE(h_q % h_kv == 0, "pool: h_q (%d) must be a multiple of h_kv (%d)", h_q, h_kv);
  HILS_REQUIRE(D % 4 == 0, "pool: D (%d) must be a multiple of 4", D);
  HILS_REQUIRE(dtype == HILS_F32 || dtype == HILS_BF16, "pool: unknown dtype %d", dtype);
  return HILS_OK;
}

}  // namespace hils

using namespace hils;

extern "C" int hils_pool_fwd(const void* mu_q, const void* k, void* lmk_k, float* lmk_b, int B, int N,
                             int S, int h_q, int h_kv, int D, int64_t k_batch_stride, float sm_scale,
                             int compact, int dtype, void* stream) {
  if (int rc = check_pool_args(B, N, S, h_q, h_kv, D, dtype)) return rc;
  if (N == 0) return HILS_OK;
  HILS_REQUIRE(mu_q && k && lmk_k && lmk_b, "pool_fwd: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == HILS_BF16 && pool_bf16_ok(mu_q, k, S, h_q, h_kv, D, k_batch_stride) && (((uintptr_t)lmk_k) & 15) == 0) {
    const int G = h_q / h_kv;
    const size_t sm = (size_t)kPoolWarps * (G * D + G * 64) * sizeof(float);
    dim3 grid((N + kPoolWarps - 1) / kPoolWarps, h_kv, B);
#define HILS_POOL_FWD(NK, GM)                                                                                     \
    do {                                                                                                          \
      cudaFuncSetAttribute(pool_fwd_bf16_kernel<NK, GM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);   \
      pool_fwd_bf16_kernel<NK, GM><<<grid, 32 * kPoolWarps, sm, st>>>((const bf16*)mu_q, (const bf16*)k, (bf16*)lmk_k, \
                                                                      lmk_b, N, S, h_q, h_kv, k_batch_stride, sm_scale, compact); \
    } while (0)
    if (D == 64) { if (G == 1) HILS_POOL_FWD(4, 1); else if (G == 2) HILS_POOL_FWD(4, 2); else if (G <= 4) HILS_POOL_FWD(4, 4); else HILS_POOL_FWD(4, 8); }
    else { if (G == 1) HILS_POOL_FWD(8, 1); else if (G == 2) HILS_POOL_FWD(8, 2); else if (G <= 4) HILS_POOL_FWD(8, 4); else HILS_POOL_FWD(8, 8); }
#undef HILS_POOL_FWD
    HILS_LAUNCH_CHECK("pool_fwd");
    return HILS_OK;
  }
  size_t smem = (size_t)(S * D + D + S) * sizeof(float);
  HILS_REQUIRE(smem <= 200 * 1024, "pool_fwd: chunk tile S*D=%d too large for shared memory", S * D);
  dim3 grid(N, h_kv, B);
  if (dtype == HILS_BF16) {
    cudaFuncSetAttribute(pool_fwd_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    pool_fwd_kernel<bf16><<<grid, 128, smem, st>>>((const bf16*)mu_q, (const bf16*)k, (bf16*)lmk_k, lmk_b, N, S,
                                                   h_q, h_kv, D, k_batch_stride, sm_scale, compact);
  } else {
    cudaFuncSetAttribute(pool_fwd_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    pool_fwd_kernel<float><<<grid, 128, smem, st>>>((const float*)mu_q, (const float*)k, (float*)lmk_k, lmk_b, N,
                                                    S, h_q, h_kv, D, k_batch_stride, sm_scale, compact);
  }
  HILS_LAUNCH_CHECK("pool_fwd");
  return HILS_OK;
}

extern "C" int hils_pool_bwd(const void* mu_q, const void* k, const void* g_lmk_k, const float* g_lmk_b,
                             void* d_mu_q, void* d_k, int B, int N, int S, int h_q, int h_kv, int D,
                             int64_t k_batch_stride, float sm_scale, int compact, int dtype, void* stream) {
  if (int rc = check_pool_args(B, N, S, h_q, h_kv, D, dtype)) return rc;
  if (N == 0) return HILS_OK;
  HILS_REQUIRE(mu_q && k && d_mu_q && d_k, "pool_bwd: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == HILS_BF16 && pool_bf16_ok(mu_q, k, S, h_q, h_kv, D, k_batch_stride) &&
      ((((uintptr_t)d_mu_q) | ((uintptr_t)d_k) | ((uintptr_t)g_lmk_k)) & 15) == 0) {
    const int G = h_q / h_kv;
    const size_t sm = (size_t)kPoolWarps * (2 * G * D + 2 * G * 64) * sizeof(float);
    dim3 grid((N + kPoolWarps - 1) / kPoolWarps, h_kv, B);
#define HILS_POOL_BWD(NK, GM)                                                                                     \
    do {                                                                                                          \
      cudaFuncSetAttribute(pool_bwd_bf16_kernel<NK, GM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);   \
      pool_bwd_bf16_kernel<NK, GM><<<grid, 32 * kPoolWarps, sm, st>>>((const bf16*)mu_q, (const bf16*)k, (const bf16*)g_lmk_k, \
                                                                      g_lmk_b, (bf16*)d_mu_q, (bf16*)d_k, N, S, h_q, h_kv,     \
                                                                      k_batch_stride, sm_scale, compact);                      \
    } while (0)
    if (D == 64) { if (G == 1) HILS_POOL_BWD(4, 1); else if (G == 2) HILS_POOL_BWD(4, 2); else if (G <= 4) HILS_POOL_BWD(4, 4); else HILS_POOL_BWD(4, 8); }
    else { if (G == 1) HILS_POOL_BWD(8, 1); else if (G == 2) HILS_POOL_BWD(8, 2); else if (G <= 4) HILS_POOL_BWD(8, 4); else HILS_POOL_BWD(8, 8); }
#undef HILS_POOL_BWD
    HILS_LAUNCH_CHECK("pool_bwd");
    return HILS_OK;
  }
  size_t smem = (size_t)(2 * S * D + 2 * D + 2 * S) * sizeof(float);
  HILS_REQUIRE(smem <= 200 * 1024, "pool_bwd: chunk tile S*D=%d too large for shared memory", S * D);
  dim3 grid(N, h_kv, B);
  if (dtype == HILS_BF16) {
    cudaFuncSetAttribute(pool_bwd_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    pool_bwd_kernel<bf16><<<grid, 128, smem, st>>>((const bf16*)mu_q, (const bf16*)k, (const bf16*)g_lmk_k,
                                                   g_lmk_b, (bf16*)d_mu_q, (bf16*)d_k, N, S, h_q, h_kv, D,
                                                   k_batch_stride, sm_scale, compact);
  } else {
    cudaFuncSetAttribute(pool_bwd_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    pool_bwd_kernel<float><<<grid, 128, smem, st>>>((const float*)mu_q, (const float*)k, (const float*)g_lmk_k,
                                                    g_lmk_b, (float*)d_mu_q, (float*)d_k, N, S, h_q, h_kv, D,
                                                    k_batch_stride, sm_scale, compact);
  }
  HILS_LAUNCH_CHECK("pool_bwd");
  return HILS_OK;
}

extern "C" int hils_meanpool_fwd(const void* k, void* out, int B, int N, int S, int h_kv, int D,
                                 int64_t k_batch_stride, int dtype, void* stream) {
  if (int rc = check_pool_args(B, N, S, h_kv, h_kv, D, dtype)) return rc;
  if (N == 0) return HILS_OK;
  HILS_REQUIRE(k && out, "meanpool_fwd: null pointer");
  int HD = h_kv * D;
  int64_t total4 = (int64_t)B * N * (HD / 4);
  int blocks = (int)((total4 + 255) / 256);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == HILS_BF16)
    meanpool_fwd_kernel<bf16><<<blocks, 256, 0, st>>>((const bf16*)k, (bf16*)out, N, S, HD, k_batch_stride, total4);
  else
    meanpool_fwd_kernel<float><<<blocks, 256, 0, st>>>((const float*)k, (float*)out, N, S, HD, k_batch_stride, total4);
  HILS_LAUNCH_CHECK("meanpool_fwd");
  return HILS_OK;
}

extern "C" int hils_meanpool_bwd(const void* g_out, void* d_k, int B, int N, int S, int h_kv, int D, int dtype,
                                 void* stream) {
  if (int rc = check_pool_args(B, N, S, h_kv, h_kv, D, dtype)) return rc;
  if (N == 0) return HILS_OK;
  HILS_REQUIRE(g_out && d_k, "meanpool_bwd: null pointer");
  int HD = h_kv * D;
  int64_t total4 = (int64_t)B * N * S * (HD / 4);
  int blocks = (int)((total4 + 255) / 256);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == HILS_BF16)
    meanpool_bwd_kernel<bf16><<<blocks, 256, 0, st>>>((const bf16*)g_out, (bf16*)d_k, S, HD, total4);
  else
    meanpool_bwd_kernel<float><<<blocks, 256, 0, st>>>((const float*)g_out, (float*)d_k, S, HD, total4);
  HILS_LAUNCH_CHECK("meanpool_bwd");
  return HILS_OK;
}
