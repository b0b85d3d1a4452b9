// Decode-shaped attention kernels: a handful of query rows per sequence against a long KV store.
// With one query row a 128-row tensor-core tile would be 99 % padding and the step is bound by
// streaming K/V out of HBM, so these kernels are CUDA-core streamers: one CTA per (kv-head, batch,
// query row) reads each K/V row once with 16-byte loads (16 lanes per row) and serves all G query
// heads of the group from it.  Same contracts as the sparse chunk attention
// (ops/hils_fwd_bwd_head.py:404-485) and the sliding-window branch (ops/flex_attn_tilelang.py:115-253).
#include <algorithm>

#include "common.cuh"
#include "mma_rows.cuh"

namespace hils {

constexpr int kDecWarps = 8;
constexpr int kDecMaxG = 8;

struct DecodeParams {
  const void* q; const void* k; const void* v; const void* w; const int32_t* idx; const float* slope;
  void* o; float* lse;
  int B, L, T, h_q, h_kv, D, K, num_weights, S, mask_last;       // sparse
  int W, mask_lmk, expand, kv_start;                              // sliding window
  float scale;
  // Paged store (pages != null): K/V are a pool of pages of S tokens, (num_pages, h_kv, S, D) - inside a page the rows
  // of one head are contiguous, so a chunk of one head is one 16 KB run (D = 128) instead of 64 rows h_kv * D apart;
  // chunk c of sequence b lives in page pages[b * page_stride + c]; sequence b holds lens[b] + len_add tokens (T is
  // ignored).  The paged kernels walk rows with stride D.
  const int32_t* pages; const int32_t* lens;
  int page_stride, num_pages, len_add;
  // Decode step fusions.  Window kernel: lse_act (or null) receives the log-sum-exp again, rounded to the activation
  // dtype the chain carries it in.  Sparse kernel: with swa_o given, o = round(o_hils) + w[swa_col] * swa_o, the
  // combination of the two branches with the rounding of the separate kernels.
  void* lse_act; const void* swa_o; int swa_col;
};

// Set when a page table holds an id outside the pool or a chunk past the table's width; the access is skipped.
__device__ int g_paged_status = 0;

template <bool PG>
__device__ __forceinline__ int seq_tokens(const DecodeParams& p, int b) {
  if constexpr (PG) return p.lens[b] + p.len_add;
  else return p.T;
}

// Row `tok` of sequence b (holding T tokens), kv-head h.  Paged: rows that follow it in the same chunk are contiguous
// at the usual stride h_kv * D; a run of rows must not leave its chunk.  Null when the page table is inconsistent.
// Key and value rows `tok` of (sequence b, head h): k0 / v0 are row 0 of that (sequence, head) in the token-major store;
// the paged kernels look the chunk's page up once for both.  The two forms are separate instantiations (PG), so the
// kernels over the token-major store carry none of the table look-ups.  False when the page table is inconsistent.
template <typename T, bool PG>
__device__ __forceinline__ bool kv_rows_at(const DecodeParams& p, const T* k0, const T* v0, int64_t rs, int b, int tok, int h,
                                           const T*& kb, const T*& vb) {
  if constexpr (PG) {
    const int c = tok / p.S;
    const int pg = (c < p.page_stride) ? p.pages[(int64_t)b * p.page_stride + c] : -1;
    if ((unsigned)pg >= (unsigned)p.num_pages) {
      atomicExch(&g_paged_status, 8000000 + (c < p.page_stride ? 1 : 2));
      return false;
    }
    const int64_t off = (((int64_t)pg * p.h_kv + h) * p.S + (tok - c * p.S)) * p.D;
    kb = static_cast<const T*>(p.k) + off;
    vb = static_cast<const T*>(p.v) + off;
  } else {
    kb = k0 + (int64_t)tok * rs;
    vb = v0 + (int64_t)tok * rs;
  }
  return true;
}

// scores of `n` consecutive key rows (row stride rs elements) against the G query rows in q_s:
// out[g * ostride + j] = <q_g, K_j>.  Half-warp per key row, four rows in flight per half-warp.
template <typename T, int PER>
__device__ __forceinline__ void score_rows(const float* q_s, const T* kbase, int64_t rs, int n, int G, int D, float* out,
                                           int ostride, int lane) {
  const int half = lane >> 4, sub = lane & 15;
  for (int j0 = 0; j0 < n; j0 += 8) {
    float kv[4][PER];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int j = j0 + u * 2 + half;
      if (j < n) {
#pragma unroll
        for (int e = 0; e < PER; e += 4) {
          const float4 x = load4(kbase + (int64_t)j * rs + sub * PER + e);
          kv[u][e] = x.x; kv[u][e + 1] = x.y; kv[u][e + 2] = x.z; kv[u][e + 3] = x.w;
        }
      } else {
#pragma unroll
        for (int e = 0; e < PER; ++e) kv[u][e] = 0.f;
      }
    }
    for (int g = 0; g < G; ++g) {
      float qv[PER];
#pragma unroll
      for (int e = 0; e < PER; ++e) qv[e] = q_s[g * D + sub * PER + e];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        float acc = 0.f;
#pragma unroll
        for (int e = 0; e < PER; ++e) acc = fmaf(qv[e], kv[u][e], acc);
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        const int j = j0 + u * 2 + half;
        if (sub == 0 && j < n) out[g * ostride + j] = acc;
      }
    }
  }
}

// acc[g][.] += sum_j p[g * pstride + j] * V_j ; lane owns PER consecutive output columns
template <typename T, int PER>
__device__ __forceinline__ void pv_rows(const float* p_s, int pstride, const T* vbase, int64_t rs, int n, int G,
                                        float (&acc)[kDecMaxG][PER], int lane) {
  for (int j0 = 0; j0 < n; j0 += 8) {          // eight value rows in flight per lane
    float vv[8][PER];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int j = min(j0 + u, n - 1);
      if constexpr (PER >= 4) {
#pragma unroll
        for (int e = 0; e < PER; e += 4) {
          const float4 x = load4(vbase + (int64_t)j * rs + lane * PER + e);
          vv[u][e] = x.x; vv[u][e + 1] = x.y; vv[u][e + 2] = x.z; vv[u][e + 3] = x.w;
        }
      } else {
        const float2 x = load2(vbase + (int64_t)j * rs + lane * PER);
        vv[u][0] = x.x; vv[u][1] = x.y;
      }
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (j0 + u < n) {
#pragma unroll
        for (int g = 0; g < kDecMaxG; ++g) {
          if (g < G) {
            const float pj = p_s[g * pstride + j0 + u];
#pragma unroll
            for (int e = 0; e < PER; ++e) acc[g][e] = fmaf(pj, vv[u][e], acc[g][e]);
          }
        }
      }
    }
  }
}

// ---- sparse chunk attention, decode shape: D = 32 * PER columns, keys per chunk S <= 64 -------------
template <typename T, int PER, bool PG>
__global__ void __launch_bounds__(kDecWarps * 32) sparse_decode_kernel(DecodeParams p) {
  constexpr int D = 32 * PER, KPER = D / 16;
  extern __shared__ __align__(16) float smem[];
  const int G = p.h_q / p.h_kv;
  float* q_s = smem;                                  // [G][D]
  float* p_s = q_s + G * D;                           // [warps][G][64]
  float* o_s = p_s + kDecWarps * G * 64;              // [warps][G][D]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int h = blockIdx.x, b = blockIdx.y, l = blockIdx.z;
  const int64_t row0 = (((int64_t)b * p.L + l) * p.h_q + h * G);
  const T* q = static_cast<const T*>(p.q) + row0 * D;
  for (int i = tid; i < G * D; i += kDecWarps * 32) q_s[i] = to_f(q[i]);
  __syncthreads();
  const int32_t* ids = p.idx + (((int64_t)b * p.L + l) * p.h_kv + h) * p.K;
  const T* wts = static_cast<const T*>(p.w) + row0 * p.num_weights;
  const int T_b = seq_tokens<PG>(p, b);
  const int nchunk = T_b / p.S;
  int nvalid = 0;
  while (nvalid < p.K && ids[nvalid] >= 0) ++nvalid;
  float acc[kDecMaxG][PER];
#pragma unroll
  for (int g = 0; g < kDecMaxG; ++g)
#pragma unroll
    for (int e = 0; e < PER; ++e) acc[g][e] = 0.f;
  float* pw = p_s + warp * G * 64;
  const int64_t rs = PG ? (int64_t)D : (int64_t)p.h_kv * D;
  const T* kb0 = static_cast<const T*>(p.k) + ((int64_t)b * p.T * p.h_kv + h) * D;
  const T* vb0 = static_cast<const T*>(p.v) + ((int64_t)b * p.T * p.h_kv + h) * D;
  for (int kk = warp; kk < nvalid; kk += kDecWarps) {
    const int c = ids[kk];
    if (c >= nchunk) continue;
    const T* kb;
    const T* vb;
    if (!kv_rows_at<T, PG>(p, kb0, vb0, rs, b, c * p.S, h, kb, vb)) continue;
    __syncwarp();
    score_rows<T, KPER>(q_s, kb, rs, p.S, G, D, pw, 64, lane);
    __syncwarp();
    for (int g = 0; g < G; ++g) {
      const float slope = p.slope ? p.slope[h * G + g] : 0.f;
      float s0 = -CUDART_INF_F, s1 = -CUDART_INF_F;
      const int j0 = lane, j1 = lane + 32;
      if (j0 < p.S && !(p.mask_last && j0 == p.S - 1)) s0 = (pw[g * 64 + j0] - slope * (float)max(0, p.S - 2 - j0)) * p.scale;
      if (j1 < p.S && !(p.mask_last && j1 == p.S - 1)) s1 = (pw[g * 64 + j1] - slope * (float)max(0, p.S - 2 - j1)) * p.scale;
      const float m = warp_max(fmaxf(s0, s1));
      float e0 = 0.f, e1 = 0.f;
      if (m > -CUDART_INF_F) { e0 = expf(s0 - m); e1 = expf(s1 - m); }
      const float sum = warp_sum(e0 + e1);
      const float f = (sum > 0.f) ? to_f(wts[g * p.num_weights + kk]) / sum : 0.f;
      if (j0 < 64) pw[g * 64 + j0] = e0 * f;
      if (j1 < 64) pw[g * 64 + j1] = e1 * f;
    }
    __syncwarp();
    pv_rows<T, PER>(pw, 64, vb, rs, p.S, G, acc, lane);
  }
  float* ow = o_s + warp * G * D;
#pragma unroll
  for (int g = 0; g < kDecMaxG; ++g)
    if (g < G)
#pragma unroll
      for (int e = 0; e < PER; ++e) ow[g * D + lane * PER + e] = acc[g][e];
  __syncthreads();
  T* o = static_cast<T*>(p.o) + row0 * D;
  for (int i = tid; i < G * D; i += kDecWarps * 32) {
    float s = 0.f;
    for (int w = 0; w < kDecWarps; ++w) s += o_s[w * G * D + i];
    if (p.swa_o)
      s = fmaf(to_f(static_cast<const T*>(p.swa_o)[row0 * D + i]), to_f(wts[(i / D) * p.num_weights + p.swa_col]),
               to_f(from_f<T>(s)));
    o[i] = from_f<T>(s);
  }
}

// ---- sliding-window branch, decode shape ------------------------------------------------------------
template <typename T, int PER, bool PG>
__global__ void __launch_bounds__(kDecWarps * 32) swa_decode_kernel(DecodeParams p) {
  constexpr int D = 32 * PER, KPER = D / 16;
  extern __shared__ __align__(16) float smem[];
  const int G = p.h_q / p.h_kv;
  float* q_s = smem;                                  // [G][D]
  float* p_s = q_s + G * D;                           // [warps][G][64]
  float* o_s = p_s + kDecWarps * G * 64;              // [warps][G][D]
  float* ml_s = o_s + kDecWarps * G * D;              // [warps][G][2]  running max, sum
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int h = blockIdx.x, b = blockIdx.y, i = blockIdx.z;
  const int64_t row0 = (((int64_t)b * p.L + i) * p.h_q + h * G);
  const T* q = static_cast<const T*>(p.q) + row0 * D;
  for (int x = tid; x < G * D; x += kDecWarps * 32) q_s[x] = to_f(q[x]);
  __syncthreads();
  const int T_b = seq_tokens<PG>(p, b);
  const int t = p.kv_start + (T_b - p.L) + i;
  int start = t - p.W + 1;
  if (p.expand) start = floor_div(start, p.S) * p.S;
  const int lo = max(0, start - p.kv_start), hi = min(T_b - 1, t - p.kv_start);
  float acc[kDecMaxG][PER], m[kDecMaxG], lsum[kDecMaxG];
#pragma unroll
  for (int g = 0; g < kDecMaxG; ++g) {
    m[g] = -CUDART_INF_F; lsum[g] = 0.f;
#pragma unroll
    for (int e = 0; e < PER; ++e) acc[g][e] = 0.f;
  }
  float* pw = p_s + warp * G * 64;
  const int64_t rs = PG ? (int64_t)D : (int64_t)p.h_kv * D;
  const T* kb0 = static_cast<const T*>(p.k) + ((int64_t)b * p.T * p.h_kv + h) * D;
  const T* vb0 = static_cast<const T*>(p.v) + ((int64_t)b * p.T * p.h_kv + h) * D;
  // paged: lo is a multiple of S = 64 (the window's left edge is snapped to its chunk), so a step stays in one page
  for (int j0 = lo + warp * 64; j0 <= hi; j0 += kDecWarps * 64) {   // 64 keys per warp step
    const int n = min(64, hi - j0 + 1);
    const T* kb;
    const T* vb;
    if (!kv_rows_at<T, PG>(p, kb0, vb0, rs, b, j0, h, kb, vb)) continue;
    __syncwarp();
    score_rows<T, KPER>(q_s, kb, rs, n, G, D, pw, 64, lane);
    __syncwarp();
#pragma unroll
    for (int g = 0; g < kDecMaxG; ++g) {
      if (g < G) {
        const int ja = lane, jb = lane + 32;
        float s0 = -CUDART_INF_F, s1 = -CUDART_INF_F;
        if (ja < n && !(p.mask_lmk && ((p.kv_start + j0 + ja + 1) % p.S == 0))) s0 = pw[g * 64 + ja] * p.scale;
        if (jb < n && !(p.mask_lmk && ((p.kv_start + j0 + jb + 1) % p.S == 0))) s1 = pw[g * 64 + jb] * p.scale;
        const float mn = fmaxf(m[g], warp_max(fmaxf(s0, s1)));
        float e0 = 0.f, e1 = 0.f, corr = 1.f;
        if (mn > -CUDART_INF_F) {
          corr = (m[g] > -CUDART_INF_F) ? expf(m[g] - mn) : 0.f;
          e0 = expf(s0 - mn); e1 = expf(s1 - mn);
        }
        lsum[g] = lsum[g] * corr + warp_sum(e0 + e1);
        m[g] = mn;
#pragma unroll
        for (int e = 0; e < PER; ++e) acc[g][e] *= corr;
        pw[g * 64 + ja] = e0;
        pw[g * 64 + jb] = e1;
      }
    }
    __syncwarp();
    pv_rows<T, PER>(pw, 64, vb, rs, n, G, acc, lane);
  }
  float* ow = o_s + warp * G * D;
#pragma unroll
  for (int g = 0; g < kDecMaxG; ++g)
    if (g < G) {
#pragma unroll
      for (int e = 0; e < PER; ++e) ow[g * D + lane * PER + e] = acc[g][e];
      if (lane == 0) { ml_s[(warp * G + g) * 2] = m[g]; ml_s[(warp * G + g) * 2 + 1] = lsum[g]; }
    }
  __syncthreads();
  T* o = static_cast<T*>(p.o) + row0 * D;
  for (int x = tid; x < G * D; x += kDecWarps * 32) {
    const int g = x / D;
    float mm = -CUDART_INF_F;
    for (int w = 0; w < kDecWarps; ++w) mm = fmaxf(mm, ml_s[(w * G + g) * 2]);
    float tot = 0.f, s = 0.f;
    if (mm > -CUDART_INF_F)
      for (int w = 0; w < kDecWarps; ++w) {
        const float mw = ml_s[(w * G + g) * 2];
        const float c = (mw > -CUDART_INF_F) ? expf(mw - mm) : 0.f;
        tot += ml_s[(w * G + g) * 2 + 1] * c;
        s += o_s[w * G * D + x] * c;
      }
    o[x] = from_f<T>(tot > 0.f ? s / tot : 0.f);
    if (x % D == 0) {
      const float lse = (tot > 0.f) ? mm + logf(tot) : -CUDART_INF_F;
      p.lse[row0 + g] = lse;
      if (p.lse_act) static_cast<T*>(p.lse_act)[row0 + g] = from_f<T>(lse);
    }
  }
}

// =================================================================================================
// bf16 fast path.  Scores come from mma.sync with B fragments loaded straight from the key rows in
// global memory (mma_rows.cuh): no shared-memory staging, no barrier.  P.V runs on the CUDA cores with
// 16-byte loads: D/8 lanes cover one value row, 32/(D/8) rows per instruction, eight loads in flight.
// =================================================================================================
template <int NK, int GM, bool PG>
__global__ void __launch_bounds__(kDecWarps * 32, 2) sparse_decode_bf16_kernel(DecodeParams p) {
  constexpr int D = NK * 16, LPR = 2 * NK;
  extern __shared__ __align__(16) float smem[];
  const int G = p.h_q / p.h_kv;
  float* q_s = smem;                                  // [G][D]
  float* p_s = q_s + G * D;                           // [warps][G][64]
  float* o_s = p_s + kDecWarps * G * 64;              // [warps][G][D]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int h = blockIdx.x, b = blockIdx.y, l = blockIdx.z;
  const int64_t row0 = (((int64_t)b * p.L + l) * p.h_q + h * G);
  const bf16* q = static_cast<const bf16*>(p.q) + row0 * D;
  for (int i = tid; i < G * D; i += kDecWarps * 32) q_s[i] = to_f(q[i]);
  __syncthreads();
  uint32_t af[NK][4];
  make_q_frags<NK>(q_s, lane, af, [G](int r) { return r < G ? r : -1; });
  const int32_t* ids = p.idx + (((int64_t)b * p.L + l) * p.h_kv + h) * p.K;
  const bf16* wts = static_cast<const bf16*>(p.w) + row0 * p.num_weights;
  const int T_b = seq_tokens<PG>(p, b);
  const int nchunk = T_b / p.S;
  int nvalid = p.K;                                   // ids are valid up to the first negative one
  for (int k0 = 0; k0 < p.K; k0 += 32) {
    const int id = (k0 + lane < p.K) ? ids[k0 + lane] : -1;
    const uint32_t neg = __ballot_sync(0xffffffffu, id < 0);
    if (neg) { nvalid = min(p.K, k0 + __ffs(neg) - 1); break; }
  }
  float acc[GM][8];
#pragma unroll
  for (int g = 0; g < GM; ++g)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[g][e] = 0.f;
  float* pw = p_s + warp * G * 64;
  const int64_t rs = PG ? (int64_t)D : (int64_t)p.h_kv * D;
  const bf16* kb0 = static_cast<const bf16*>(p.k) + ((int64_t)b * p.T * p.h_kv + h) * D;
  const bf16* vb0 = static_cast<const bf16*>(p.v) + ((int64_t)b * p.T * p.h_kv + h) * D;
  for (int kk = warp; kk < nvalid; kk += kDecWarps) {
    const int c = ids[kk];
    if (c >= nchunk) continue;
    const bf16* kb;
    const bf16* vb;
    if (!kv_rows_at<bf16, PG>(p, kb0, vb0, rs, b, c * p.S, h, kb, vb)) continue;
    __syncwarp();
    score_rows_mma<NK>(af, kb, rs, p.S, G, pw, 64, lane);
    __syncwarp();
    for (int g = 0; g < G; ++g) {
      const float slope = p.slope ? p.slope[h * G + g] : 0.f;
      float s0 = -CUDART_INF_F, s1 = -CUDART_INF_F;
      const int j0 = lane, j1 = lane + 32;
      if (j0 < p.S && !(p.mask_last && j0 == p.S - 1)) s0 = (pw[g * 64 + j0] - slope * (float)max(0, p.S - 2 - j0)) * p.scale;
      if (j1 < p.S && !(p.mask_last && j1 == p.S - 1)) s1 = (pw[g * 64 + j1] - slope * (float)max(0, p.S - 2 - j1)) * p.scale;
      const float m = warp_max(fmaxf(s0, s1));
      float e0 = 0.f, e1 = 0.f;
      if (m > -CUDART_INF_F) { e0 = expf(s0 - m); e1 = expf(s1 - m); }
      const float sum = warp_sum(e0 + e1);
      const float f = (sum > 0.f) ? to_f(wts[g * p.num_weights + kk]) / sum : 0.f;
      pw[g * 64 + j0] = e0 * f;
      pw[g * 64 + j1] = e1 * f;
    }
    __syncwarp();
    pv_rows16<NK, GM>(pw, 64, vb, rs, p.S, G, acc, lane);
  }
  pv_reduce<NK, GM>(acc);
  float* ow = o_s + warp * G * D;
  if (lane < LPR)
#pragma unroll
    for (int g = 0; g < GM; ++g)
      if (g < G)
#pragma unroll
        for (int e = 0; e < 8; ++e) ow[g * D + lane * 8 + e] = acc[g][e];
  __syncthreads();
  bf16* o = static_cast<bf16*>(p.o) + row0 * D;
  for (int i = tid; i < G * D; i += kDecWarps * 32) {
    float sacc = 0.f;
    for (int w = 0; w < kDecWarps; ++w) sacc += o_s[w * G * D + i];
    if (p.swa_o)
      sacc = fmaf(to_f(static_cast<const bf16*>(p.swa_o)[row0 * D + i]), to_f(wts[(i / D) * p.num_weights + p.swa_col]),
                  to_f(__float2bfloat16_rn(sacc)));
    o[i] = __float2bfloat16_rn(sacc);
  }
}

constexpr int kSwaDecTile = 32;      // keys per warp step

// NW warps per CTA: the window is at most (W + S) / 32 steps of 32 keys, and 18 steps (W = 512) split evenly over 6 warps
// but 3 + 2 over 8.
template <int NK, int GM, bool PG, int NW>
__global__ void __launch_bounds__(NW * 32, NW == 6 ? 3 : 2) swa_decode_bf16_kernel(DecodeParams p) {
  constexpr int D = NK * 16, LPR = 2 * NK;
  extern __shared__ __align__(16) float smem[];
  const int G = p.h_q / p.h_kv;
  float* q_s = smem;                                  // [G][D]
  float* p_s = q_s + G * D;                           // [warps][G][64]
  float* o_s = p_s + NW * G * 64;              // [warps][G][D]
  float* ml_s = o_s + NW * G * D;              // [warps][G][2]  running max, sum
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int h = blockIdx.x, b = blockIdx.y, i = blockIdx.z;
  const int64_t row0 = (((int64_t)b * p.L + i) * p.h_q + h * G);
  const bf16* q = static_cast<const bf16*>(p.q) + row0 * D;
  for (int x = tid; x < G * D; x += NW * 32) q_s[x] = to_f(q[x]);
  __syncthreads();
  uint32_t af[NK][4];
  make_q_frags<NK>(q_s, lane, af, [G](int r) { return r < G ? r : -1; });
  const int T_b = seq_tokens<PG>(p, b);
  const int t = p.kv_start + (T_b - p.L) + i;
  int start = t - p.W + 1;
  if (p.expand) start = floor_div(start, p.S) * p.S;
  const int lo = max(0, start - p.kv_start), hi = min(T_b - 1, t - p.kv_start);
  float acc[GM][8], m[GM], lsum[GM];
#pragma unroll
  for (int g = 0; g < GM; ++g) {
    m[g] = -CUDART_INF_F; lsum[g] = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[g][e] = 0.f;
  }
  float* pw = p_s + warp * G * 64;
  const int64_t rs = PG ? (int64_t)D : (int64_t)p.h_kv * D;
  const bf16* kb0 = static_cast<const bf16*>(p.k) + ((int64_t)b * p.T * p.h_kv + h) * D;
  const bf16* vb0 = static_cast<const bf16*>(p.v) + ((int64_t)b * p.T * p.h_kv + h) * D;
  // paged: lo is a multiple of S = 64 and the step is 32 keys, so a step stays in one page
  for (int j0 = lo + warp * kSwaDecTile; j0 <= hi; j0 += NW * kSwaDecTile) {
    const int n = min(kSwaDecTile, hi - j0 + 1);
    const bf16* kb;
    const bf16* vb;
    if (!kv_rows_at<bf16, PG>(p, kb0, vb0, rs, b, j0, h, kb, vb)) continue;
    __syncwarp();
    score_rows_mma<NK>(af, kb, rs, n, G, pw, 64, lane);
    __syncwarp();
#pragma unroll
    for (int g = 0; g < GM; ++g) {
      if (g < G) {
        float s0 = -CUDART_INF_F;
        if (lane < n && !(p.mask_lmk && ((p.kv_start + j0 + lane + 1) % p.S == 0))) s0 = pw[g * 64 + lane] * p.scale;
        const float mn = fmaxf(m[g], warp_max(s0));
        float e0 = 0.f, corr = 1.f;
        if (mn > -CUDART_INF_F) {
          corr = (m[g] > -CUDART_INF_F) ? expf(m[g] - mn) : 0.f;
          e0 = expf(s0 - mn);
        }
        lsum[g] = lsum[g] * corr + warp_sum(e0);
        m[g] = mn;
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[g][e] *= corr;
        pw[g * 64 + lane] = e0;
      }
    }
    __syncwarp();
    pv_rows16<NK, GM>(pw, 64, vb, rs, n, G, acc, lane);
  }
  pv_reduce<NK, GM>(acc);
  float* ow = o_s + warp * G * D;
#pragma unroll
  for (int g = 0; g < GM; ++g)
    if (g < G) {
      if (lane < LPR)
#pragma unroll
        for (int e = 0; e < 8; ++e) ow[g * D + lane * 8 + e] = acc[g][e];
      if (lane == 0) { ml_s[(warp * G + g) * 2] = m[g]; ml_s[(warp * G + g) * 2 + 1] = lsum[g]; }
    }
  __syncthreads();
  bf16* o = static_cast<bf16*>(p.o) + row0 * D;
  for (int x = tid; x < G * D; x += NW * 32) {
    const int g = x / D;
    float mm = -CUDART_INF_F;
    for (int w = 0; w < NW; ++w) mm = fmaxf(mm, ml_s[(w * G + g) * 2]);
    float tot = 0.f, sacc = 0.f;
    if (mm > -CUDART_INF_F)
      for (int w = 0; w < NW; ++w) {
        const float mw = ml_s[(w * G + g) * 2];
        const float c = (mw > -CUDART_INF_F) ? expf(mw - mm) : 0.f;
        tot += ml_s[(w * G + g) * 2 + 1] * c;
        sacc += o_s[w * G * D + x] * c;
      }
    o[x] = __float2bfloat16_rn(tot > 0.f ? sacc / tot : 0.f);
    if (x % D == 0) {
      const float lse = (tot > 0.f) ? mm + logf(tot) : -CUDART_INF_F;
      p.lse[row0 + g] = lse;
      if (p.lse_act) static_cast<bf16*>(p.lse_act)[row0 + g] = __float2bfloat16_rn(lse);
    }
  }
}

template <int NK, int GM, bool PG>
static void launch_decode_bf16_pg(const DecodeParams& p, bool swa, dim3 grid, size_t smem, cudaStream_t st) {
  if (swa) {
    // warps per CTA that leave the fewest idle warp steps
    const int nstep = (p.W + p.S + kSwaDecTile - 1) / kSwaDecTile;
    if ((nstep + 5) / 6 * 6 < (nstep + 7) / 8 * 8) {
      cudaFuncSetAttribute(swa_decode_bf16_kernel<NK, GM, PG, 6>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      swa_decode_bf16_kernel<NK, GM, PG, 6><<<grid, 6 * 32, smem, st>>>(p);
    } else {
      cudaFuncSetAttribute(swa_decode_bf16_kernel<NK, GM, PG, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      swa_decode_bf16_kernel<NK, GM, PG, 8><<<grid, 8 * 32, smem, st>>>(p);
    }
  } else {
    cudaFuncSetAttribute(sparse_decode_bf16_kernel<NK, GM, PG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sparse_decode_bf16_kernel<NK, GM, PG><<<grid, kDecWarps * 32, smem, st>>>(p);
  }
}

template <int NK, int GM>
static void launch_decode_bf16_g(const DecodeParams& p, bool swa, dim3 grid, size_t smem, cudaStream_t st) {
  if (p.pages) launch_decode_bf16_pg<NK, GM, true>(p, swa, grid, smem, st);
  else launch_decode_bf16_pg<NK, GM, false>(p, swa, grid, smem, st);
}

template <int NK>
static void launch_decode_bf16(const DecodeParams& p, bool swa, dim3 grid, size_t smem, cudaStream_t st) {
  const int G = p.h_q / p.h_kv;
  if (G == 1) launch_decode_bf16_g<NK, 1>(p, swa, grid, smem, st);
  else if (G == 2) launch_decode_bf16_g<NK, 2>(p, swa, grid, smem, st);
  else if (G <= 4) launch_decode_bf16_g<NK, 4>(p, swa, grid, smem, st);
  else launch_decode_bf16_g<NK, 8>(p, swa, grid, smem, st);
}

template <typename T>
static int launch_decode(const DecodeParams& p, bool swa, cudaStream_t st) {
  const int G = p.h_q / p.h_kv;
  const size_t smem = ((size_t)G * p.D + (size_t)kDecWarps * G * 64 + (size_t)kDecWarps * G * p.D +
                       (size_t)kDecWarps * G * 2) * sizeof(float);
  dim3 grid(p.h_kv, p.B, p.L);
  if (sizeof(T) == 2) {
    if (p.D == 128) launch_decode_bf16<8>(p, swa, grid, smem, st); else launch_decode_bf16<4>(p, swa, grid, smem, st);
    HILS_LAUNCH_CHECK(swa ? "swa_fwd (decode)" : "sparse_attn_fwd (decode)");
    return HILS_OK;
  }
#define HILS_DEC_LAUNCH(KERNEL, PER)                                                                       \
  do {                                                                                                     \
    if (p.pages) {                                                                                         \
      cudaFuncSetAttribute(KERNEL<T, PER, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
      KERNEL<T, PER, true><<<grid, kDecWarps * 32, smem, st>>>(p);                                         \
    } else {                                                                                               \
      cudaFuncSetAttribute(KERNEL<T, PER, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      KERNEL<T, PER, false><<<grid, kDecWarps * 32, smem, st>>>(p);                                        \
    }                                                                                                      \
  } while (0)
  if (swa) {
    if (p.D == 128) HILS_DEC_LAUNCH(swa_decode_kernel, 4); else HILS_DEC_LAUNCH(swa_decode_kernel, 2);
  } else {
    if (p.D == 128) HILS_DEC_LAUNCH(sparse_decode_kernel, 4); else HILS_DEC_LAUNCH(sparse_decode_kernel, 2);
  }
#undef HILS_DEC_LAUNCH
  HILS_LAUNCH_CHECK(swa ? "swa_fwd (decode)" : "sparse_attn_fwd (decode)");
  return HILS_OK;
}

static bool decode_shape_ok(int B, int L, int h_q, int h_kv, int D, int Dv) {
  const int G = h_q / h_kv;
  return L >= 1 && L <= 4 && D == Dv && (D == 64 || D == 128) && G <= kDecMaxG && B <= 65535 && h_kv <= (1 << 30);
}

// HILS_ERR_UNSUPPORTED when the shape is not a decode shape
struct PagedArgs { const int32_t* pages; const int32_t* lens; int page_stride, num_pages, len_add; };

static void set_paged(DecodeParams& p, const PagedArgs* pa) {
  if (!pa) return;
  p.pages = pa->pages; p.lens = pa->lens; p.page_stride = pa->page_stride; p.num_pages = pa->num_pages; p.len_add = pa->len_add;
}

static int sparse_decode_impl(const void* q, const void* k, const void* v, const void* w, const int32_t* idx, const float* slope,
                              void* o, int B, int L, int T, int h_q, int h_kv, int D, int Dv, int K, int num_weights, int S,
                              float scale, int mask_last, int dtype, cudaStream_t st, const PagedArgs* pa,
                              const void* swa_o = nullptr, int swa_col = 0) {
  if (!decode_shape_ok(B, L, h_q, h_kv, D, Dv) || S > 64) return HILS_ERR_UNSUPPORTED;
  if (dtype == HILS_BF16 && (((uintptr_t)k | (uintptr_t)v) & 15)) return HILS_ERR_UNSUPPORTED;   // 16-byte row loads
  DecodeParams p = {};
  p.q = q; p.k = k; p.v = v; p.w = w; p.idx = idx; p.slope = slope; p.o = o;
  p.B = B; p.L = L; p.T = T; p.h_q = h_q; p.h_kv = h_kv; p.D = D; p.K = K; p.num_weights = num_weights; p.S = S;
  p.mask_last = mask_last; p.scale = scale; p.swa_o = swa_o; p.swa_col = swa_col;
  set_paged(p, pa);
  return dtype == HILS_BF16 ? launch_decode<bf16>(p, false, st) : launch_decode<float>(p, false, st);
}

static int swa_decode_impl(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Lq, int Lk, int h_q,
                           int h_kv, int D, int Dv, int W, int S, int mask_lmk, int expand, float scale, int kv_start, int dtype,
                           cudaStream_t st, const PagedArgs* pa, void* lse_act = nullptr) {
  if (!decode_shape_ok(B, Lq, h_q, h_kv, D, Dv)) return HILS_ERR_UNSUPPORTED;
  if (dtype == HILS_BF16 && (((uintptr_t)k | (uintptr_t)v) & 15)) return HILS_ERR_UNSUPPORTED;   // 16-byte row loads
  DecodeParams p = {};
  p.q = q; p.k = k; p.v = v; p.o = o; p.lse = lse;
  p.B = B; p.L = Lq; p.T = Lk; p.h_q = h_q; p.h_kv = h_kv; p.D = D; p.S = S; p.W = W; p.mask_lmk = mask_lmk;
  p.expand = expand; p.kv_start = kv_start; p.scale = scale; p.lse_act = lse_act;
  set_paged(p, pa);
  return dtype == HILS_BF16 ? launch_decode<bf16>(p, true, st) : launch_decode<float>(p, true, st);
}

int sparse_decode_launch(const void* q, const void* k, const void* v, const void* w, const int32_t* idx, const float* slope,
                         void* o, int B, int L, int T, int h_q, int h_kv, int D, int Dv, int K, int num_weights, int S,
                         float scale, int mask_last, int dtype, cudaStream_t st) {
  return sparse_decode_impl(q, k, v, w, idx, slope, o, B, L, T, h_q, h_kv, D, Dv, K, num_weights, S, scale, mask_last, dtype,
                            st, nullptr);
}

int swa_decode_launch(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Lq, int Lk, int h_q,
                      int h_kv, int D, int Dv, int W, int S, int mask_lmk, int expand, float scale, int kv_start, int dtype,
                      cudaStream_t st) {
  return swa_decode_impl(q, k, v, o, lse, B, Lq, Lk, h_q, h_kv, D, Dv, W, S, mask_lmk, expand, scale, kv_start, dtype, st,
                         nullptr);
}

// One new query row per sequence against a paged store: sequence b holds lens[b] + len_add tokens, chunk c of it lives in
// page pages[b * page_stride + c] of the pools k_pages / v_pages (num_pages, h_kv, 64, D).  The page is the chunk (S = 64)
// and the window's left edge is snapped to its chunk, so no run of rows a warp reads crosses a page.
int sparse_decode_paged_launch(const void* q, const void* k_pages, const void* v_pages, const void* w, const int32_t* idx,
                               void* o, const int32_t* pages, const int32_t* lens, int page_stride, int num_pages,
                               int len_add, int B, int h_q, int h_kv, int D, int K, int num_weights, int S, float scale,
                               int mask_last, int dtype, cudaStream_t st, const void* swa_o, int swa_col) {
  if (S != 64) return HILS_ERR_UNSUPPORTED;
  const PagedArgs pa = {pages, lens, page_stride, num_pages, len_add};
  return sparse_decode_impl(q, k_pages, v_pages, w, idx, nullptr, o, B, 1, 0, h_q, h_kv, D, D, K, num_weights, S, scale,
                            mask_last, dtype, st, &pa, swa_o, swa_col);
}

// The two decode kernels as the one-call decode step uses them over the token-major store: the window kernel also
// writes the log-sum-exp in the activation dtype, the sparse kernel also combines the two branches.
int sparse_decode_combine_launch(const void* q, const void* k, const void* v, const void* w, const int32_t* idx, void* o,
                                 int B, int T, int h_q, int h_kv, int D, int K, int num_weights, int S, float scale,
                                 int mask_last, int dtype, cudaStream_t st, const void* swa_o, int swa_col) {
  return sparse_decode_impl(q, k, v, w, idx, nullptr, o, B, 1, T, h_q, h_kv, D, D, K, num_weights, S, scale, mask_last, dtype,
                            st, nullptr, swa_o, swa_col);
}

int swa_decode_lse_launch(const void* q, const void* k, const void* v, void* o, float* lse, void* lse_act, int B, int Lk,
                          int h_q, int h_kv, int D, int W, int S, int mask_lmk, int expand, float scale, int dtype,
                          cudaStream_t st) {
  return swa_decode_impl(q, k, v, o, lse, B, 1, Lk, h_q, h_kv, D, D, W, S, mask_lmk, expand, scale, 0, dtype, st, nullptr,
                         lse_act);
}

int swa_decode_paged_launch(const void* q, const void* k_pages, const void* v_pages, void* o, float* lse,
                            const int32_t* pages, const int32_t* lens, int page_stride, int num_pages, int len_add, int B,
                            int h_q, int h_kv, int D, int W, int S, int mask_lmk, float scale, int dtype, cudaStream_t st,
                            void* lse_act) {
  if (S != 64) return HILS_ERR_UNSUPPORTED;
  const PagedArgs pa = {pages, lens, page_stride, num_pages, len_add};
  return swa_decode_impl(q, k_pages, v_pages, o, lse, B, 1, 0, h_q, h_kv, D, D, W, S, mask_lmk, /*expand=*/1, scale, 0, dtype,
                         st, &pa, lse_act);
}

// The new token of every sequence goes to row lens[b] % S (of every head) of page pages[b * page_stride + lens[b] / S].
template <typename T>
__global__ void paged_append_kernel(const T* __restrict__ k_new, const T* __restrict__ v_new, T* __restrict__ k_pages,
                                    T* __restrict__ v_pages, const int32_t* __restrict__ pages,
                                    const int32_t* __restrict__ lens, int page_stride, int num_pages, int S, int row_elems,
                                    int D) {
  const int b = blockIdx.x;
  const int len = lens[b], c = len / S;
  const int pg = (len >= 0 && c < page_stride) ? pages[(int64_t)b * page_stride + c] : -1;
  if ((unsigned)pg >= (unsigned)num_pages) {
    if (threadIdx.x == 0) atomicExch(&g_paged_status, 8000003);
    return;
  }
  const int64_t page0 = (int64_t)pg * S * row_elems + (int64_t)(len - c * S) * D, src = (int64_t)b * row_elems;
  for (int i = threadIdx.x * 4; i < row_elems; i += blockDim.x * 4) {     // row_elems = h_kv * D; D is a multiple of 4
    const int h = i / D;
    const int64_t dst = page0 + (int64_t)h * S * D + (i - h * D);
    if constexpr (sizeof(T) == 2) {
      *reinterpret_cast<uint2*>(k_pages + dst) = *reinterpret_cast<const uint2*>(k_new + src + i);
      *reinterpret_cast<uint2*>(v_pages + dst) = *reinterpret_cast<const uint2*>(v_new + src + i);
    } else {
      *reinterpret_cast<float4*>(k_pages + dst) = *reinterpret_cast<const float4*>(k_new + src + i);
      *reinterpret_cast<float4*>(v_pages + dst) = *reinterpret_cast<const float4*>(v_new + src + i);
    }
  }
}

int paged_append_launch(const void* k_new, const void* v_new, void* k_pages, void* v_pages, const int32_t* pages,
                        const int32_t* lens, int page_stride, int num_pages, int S, int B, int h_kv, int D, int dtype,
                        cudaStream_t st) {
  const int row = h_kv * D;
  if (row % 4 != 0) return HILS_ERR_UNSUPPORTED;
  const int threads = std::min(256, std::max(32, (row / 4 + 31) / 32 * 32));
  if (dtype == HILS_BF16)
    paged_append_kernel<bf16><<<B, threads, 0, st>>>((const bf16*)k_new, (const bf16*)v_new, (bf16*)k_pages, (bf16*)v_pages,
                                                     pages, lens, page_stride, num_pages, S, row, D);
  else
    paged_append_kernel<float><<<B, threads, 0, st>>>((const float*)k_new, (const float*)v_new, (float*)k_pages,
                                                      (float*)v_pages, pages, lens, page_stride, num_pages, S, row, D);
  HILS_LAUNCH_CHECK("decode_step_paged (append)");
  return HILS_OK;
}

int take_status_paged() {
  int v = 0, zero = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  if (cudaMemcpyFromSymbol(&v, g_paged_status, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(g_paged_status, &zero, sizeof(int));
  return v;
}

}  // namespace hils
