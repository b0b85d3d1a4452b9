// Chunk selection: chunk-score GEMM, HiLS log-sum-exp, lse_total, top-k select, ascending id sort
// and the scores of the selected chunks, in ONE launch (the reference uses four kernels plus a
// torch op, ops/topk_head_softmax.py:977-1038).
//
// Contract (ops/topk_head_softmax.py:15-154 and the kernels :192-971), for query row i at absolute
// position t = q_offset + i, kv-head h, group member g:
//   limit = floor((t - W + 1)/S) (W > 0) or floor(t/S); candidates c in [0, min(limit, N))
//   v[g,c]   = fl32(fl32(<q_g, k'_c>) * scale) + bias[c,g] + gumbel[g,c]
//   lse_hils = logsumexp_c v[g,c];  lse_total[g] = logaddexp(lse_swa[g], lse_hils[g])
//   key[c]   = max_g (v[g,c] - lse_total[g]);  drop_mask removes candidates
//   pick the K largest keys; ties go to the smaller chunk id; -inf is never picked
//   ids ascending, -1 padded;  scores[g,k] = fl(<q_g,k'_id> * scale), -inf at -1
//
// Layout of one CTA: 4 warps, RB = 4*RW consecutive query rows of one (batch, kv-head).  Chunk keys
// stream through shared memory in tiles of 64; scores of a tile are formed by a register-tiled
// CUDA-core product (fp32 exact for both element types).  Each warp owns RW rows and keeps each
// row's running top-K as a sorted list spread over its lanes (packed 64-bit items: order-preserving
// key bits above, inverted id below, so one unsigned compare implements "greater key, then smaller
// id").  New candidates are filtered by a warp ballot against the current K-th item.
#include "common.cuh"
#include "mma_rows.cuh"
#include "topk_params.cuh"

namespace hils {

constexpr int TN = 128;  // candidates per tile
constexpr int CPT = TN / 16;  // candidates per thread in the score product

__device__ __forceinline__ uint32_t order_bits(float f) {
  uint32_t u = __float_as_uint(f + 0.0f);  // -0 -> +0
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ float log_add_exp(float a, float b) {
  if (isinf(a) && a == b) return a;
  float mx = fmaxf(a, b), mn = fminf(a, b);
  return mx + log1pf(expf(mn - mx));
}

__host__ __device__ __forceinline__ int row_limit(const TopkParams& p, int l) {
  if (l >= p.L) return 0;
  if (!p.is_causal) return p.N;
  int t = p.q_offset + l;
  int lim = (p.window_size > 0) ? floor_div(t - p.window_size + 1, p.block_size) : floor_div(t, p.block_size);
  return max(0, min(lim, p.N));
}

// decode kernels: sequences of one batch may stand at different positions
__device__ __forceinline__ int row_limit_b(const TopkParams& p, int b, int l) {
  if (!p.q_offsets) return row_limit(p, l);
  if (l >= p.L) return 0;
  if (!p.is_causal) return p.N;
  const int t = p.q_offsets[b] + l;
  const int lim = (p.window_size > 0) ? floor_div(t - p.window_size + 1, p.block_size) : floor_div(t, p.block_size);
  return max(0, min(lim, p.N));
}

typedef unsigned long long u64;

__device__ __forceinline__ u64 shfl_xor64(u64 v, int m) { return __shfl_xor_sync(0xffffffffu, v, m); }
__device__ __forceinline__ u64 max64(u64 a, u64 b) { return a > b ? a : b; }
__device__ __forceinline__ u64 min64(u64 a, u64 b) { return a > b ? b : a; }

// Descending bitonic sort of 128 packed items held 4 per lane; item index = lane*4 + i.
__device__ __forceinline__ void sort128_desc(u64 (&x)[4], int lane) {
#pragma unroll
  for (int k = 2; k <= 128; k <<= 1) {
#pragma unroll
    for (int j = k >> 1; j > 0; j >>= 1) {
      if (j >= 4) {
        const int lj = j >> 2;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int idx = lane * 4 + i;
          const u64 o = shfl_xor64(x[i], lj);
          const bool keep_max = ((idx & k) == 0) == ((idx & j) == 0);
          x[i] = keep_max ? max64(x[i], o) : min64(x[i], o);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if ((i & j) == 0) {
            const int idx = lane * 4 + i;
            const u64 a = x[i], c = x[i ^ j];
            const bool first_max = ((idx & k) == 0);
            x[i] = first_max ? max64(a, c) : min64(a, c);
            x[i ^ j] = first_max ? min64(a, c) : max64(a, c);
          }
        }
      }
    }
  }
}

// one item per lane, bitonic input (first descending then ascending or the reverse) -> descending
__device__ __forceinline__ u64 merge32_desc(u64 v, int lane) {
#pragma unroll
  for (int j = 16; j > 0; j >>= 1) {
    const u64 o = shfl_xor64(v, j);
    v = ((lane & j) == 0) ? max64(v, o) : min64(v, o);
  }
  return v;
}

// ascending bitonic sort of one int per lane
__device__ __forceinline__ int sort32_asc(int v, int lane) {
#pragma unroll
  for (int k = 2; k <= 32; k <<= 1) {
#pragma unroll
    for (int j = k >> 1; j > 0; j >>= 1) {
      const int o = __shfl_xor_sync(0xffffffffu, v, j);
      const bool keep_min = ((lane & k) == 0) == ((lane & j) == 0);
      v = keep_min ? min(v, o) : max(v, o);
    }
  }
  return v;
}

template <typename T, int KPL>
__global__ void __launch_bounds__(128) topk_fwd_kernel(TopkParams p) {
  extern __shared__ __align__(16) float smem[];
  const int G = p.G, D = p.D, RW = p.RW, RB = 4 * RW, M = RB * G, RS = D + 4;
  float* q_s = smem;                       // [M][D]
  float* kt_s = q_s + (size_t)M * D;       // [TN][RS]
  float* sc_s = kt_s + TN * RS;            // [M][TN]
  float* lse_s = sc_s + (size_t)M * TN;    // [M] running max, later lse_total
  float* sum_s = lse_s + M;                // [M] running sum
  float* bias_s = sum_s + M;               // [G][TN] bias + gumbel of the current tile
  int* ids_s = reinterpret_cast<int*>(bias_s + G * TN);  // [4][32*KPL]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int l0 = blockIdx.x * RB, h = blockIdx.y, b = blockIdx.z;
  const T* q = static_cast<const T*>(p.q);
  const T* lmks = static_cast<const T*>(p.lmks);
  const int HL = p.per_qhead ? p.h_kv * G : p.h_kv;  // heads in lmks

  for (int idx = tid * 4; idx < M * D; idx += 128 * 4) {
    int m = idx / D, d = idx - m * D;
    int l = l0 + m / G;
    float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
    if (l < p.L) x = load4(q + (((int64_t)b * p.L + l) * p.h_kv + h) * (int64_t)G * D + (int64_t)(m % G) * D + d);
    *reinterpret_cast<float4*>(q_s + idx) = x;
  }
  for (int m = tid; m < M; m += 128) { lse_s[m] = -CUDART_INF_F; sum_s[m] = 0.f; }

  const int last_row = min(l0 + RB, p.L) - 1;
  const int cta_limit = row_limit(p, last_row);  // limits are non-decreasing in l
  const int tx = tid & 15, ty = tid >> 4;

  // selection logits v of one 128-candidate tile into sc_s (-inf where not a candidate)
  auto score_tile = [&](int c0) {
    const int ng = p.per_qhead ? G : 1;
    __syncthreads();
    if (p.bias || p.gumbel) {
      for (int e = tid; e < G * TN; e += 128) {
        const int gg = e / TN, c = c0 + (e - gg * TN);
        float x = 0.f;
        if (c < p.N) {
          if (p.bias) x += p.bias[(((int64_t)b * p.N + c) * p.h_kv + h) * G + gg];
          if (p.gumbel) x += p.gumbel[(int64_t)(h * G + gg) * p.N + c];
        }
        bias_s[e] = x;
      }
    }
    for (int g = 0; g < ng; ++g) {
      __syncthreads();
      for (int idx = tid * 4; idx < TN * D; idx += 128 * 4) {
        int j = idx / D, d = idx - j * D;
        int c = c0 + j;
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < p.N) x = load4(lmks + (((int64_t)b * p.N + c) * HL + (p.per_qhead ? h * G + g : h)) * D + d);
        *reinterpret_cast<float4*>(kt_s + j * RS + d) = x;
      }
      __syncthreads();
      const int nrow = p.per_qhead ? RB : M;
      for (int i0 = ty; i0 < nrow; i0 += 16) {
        const int i1 = i0 + 8;
        const int m0 = p.per_qhead ? i0 * G + g : i0;
        const int m1 = (i1 < nrow) ? (p.per_qhead ? i1 * G + g : i1) : m0;
        float a0[CPT], a1[CPT];
#pragma unroll
        for (int jj = 0; jj < CPT; ++jj) { a0[jj] = 0.f; a1[jj] = 0.f; }
        const float* q0 = q_s + (size_t)m0 * D;
        const float* q1 = q_s + (size_t)m1 * D;
        for (int d = 0; d < D; d += 4) {
          float4 x0 = *reinterpret_cast<const float4*>(q0 + d);
          float4 x1 = *reinterpret_cast<const float4*>(q1 + d);
#pragma unroll
          for (int jj = 0; jj < CPT; ++jj) {
            float4 kv = *reinterpret_cast<const float4*>(kt_s + (tx + 16 * jj) * RS + d);
            a0[jj] = fmaf(x0.x, kv.x, a0[jj]); a0[jj] = fmaf(x0.y, kv.y, a0[jj]);
            a0[jj] = fmaf(x0.z, kv.z, a0[jj]); a0[jj] = fmaf(x0.w, kv.w, a0[jj]);
            a1[jj] = fmaf(x1.x, kv.x, a1[jj]); a1[jj] = fmaf(x1.y, kv.y, a1[jj]);
            a1[jj] = fmaf(x1.z, kv.z, a1[jj]); a1[jj] = fmaf(x1.w, kv.w, a1[jj]);
          }
        }
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
          if (rr == 1 && i1 >= nrow) break;
          const int m = rr ? m1 : m0;
          const int l = l0 + m / G, gg = m % G;
          const int lim = row_limit(p, l);
#pragma unroll
          for (int jj = 0; jj < CPT; ++jj) {
            const int c = c0 + tx + 16 * jj;
            float v = -CUDART_INF_F;
            if (c < lim) {
              v = (rr ? a1[jj] : a0[jj]) * p.scale;
              if (p.bias || p.gumbel) v += bias_s[gg * TN + tx + 16 * jj];
            }
            sc_s[(size_t)m * TN + tx + 16 * jj] = v;
          }
        }
      }
    }
    __syncthreads();
  };

  // ---------------- pass 1: online log-sum-exp of the selection logits ----------------------
  for (int c0 = 0; c0 < cta_limit; c0 += TN) {
    score_tile(c0);
    for (int r = 0; r < RW; ++r) {
      for (int g = 0; g < G; ++g) {
        const int m = (warp * RW + r) * G + g;
        const float4 v = *reinterpret_cast<const float4*>(sc_s + (size_t)m * TN + lane * 4);
        float tmax = warp_max(fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)));
        float mo = lse_s[m];
        float mn = fmaxf(mo, tmax);
        if (mn > -CUDART_INF_F) {
          float s = expf(v.x - mn) + expf(v.y - mn) + expf(v.z - mn) + expf(v.w - mn);
          s = warp_sum(s);
          if (lane == 0) {
            sum_s[m] = sum_s[m] * ((mo > -CUDART_INF_F) ? expf(mo - mn) : 0.f) + s;
            lse_s[m] = mn;
          }
        }
        __syncwarp();
      }
    }
  }
  __syncthreads();
  for (int m = tid; m < M; m += 128) {
    const int l = l0 + m / G, g = m % G;
    if (l < p.L) {
      float lh = (sum_s[m] > 0.f) ? lse_s[m] + logf(sum_s[m]) : -CUDART_INF_F;
      const int64_t o = (((int64_t)b * p.L + l) * p.h_kv + h) * G + g;
      float ls = (p.lse_dtype == HILS_BF16) ? to_f(static_cast<const bf16*>(p.lse_swa)[o])
                                            : static_cast<const float*>(p.lse_swa)[o];
      float lt = log_add_exp(ls, lh);
      lse_s[m] = lt;
      if (p.lse_total) p.lse_total[o] = lt;
    } else {
      lse_s[m] = 0.f;
    }
  }
  __syncthreads();

  // ---------------- pass 2: ranking keys and the running top-K -------------------------------
  // Items pack the order-preserving key bits above the inverted chunk id, so one unsigned compare
  // means "greater key, then smaller id"; 0 marks "no candidate".  Item index inside a tile is
  // lane*4 + i (a float4 of logits per lane).
  u64 best[4][KPL];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int i = 0; i < KPL; ++i) best[r][i] = 0ull;
  const int K = p.topk;
  const int thr_lane = (K - 1) / KPL, thr_i = (K - 1) % KPL;
  const int sel_limit = p.rank_keys ? p.N : cta_limit;
  for (int c0 = 0; c0 < sel_limit; c0 += TN) {
    score_tile(c0);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      if (r >= RW) break;
      const int row = warp * RW + r;
      const int l = l0 + row;
      if (l >= p.L) continue;
      float key[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
      for (int g = 0; g < G; ++g) {
        const float4 v = *reinterpret_cast<const float4*>(sc_s + (size_t)(row * G + g) * TN + lane * 4);
        const float lt = lse_s[row * G + g];
        if (v.x > -CUDART_INF_F) key[0] = fmaxf(key[0], v.x - lt);
        if (v.y > -CUDART_INF_F) key[1] = fmaxf(key[1], v.y - lt);
        if (v.z > -CUDART_INF_F) key[2] = fmaxf(key[2], v.z - lt);
        if (v.w > -CUDART_INF_F) key[3] = fmaxf(key[3], v.w - lt);
      }
      u64 item[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int c = c0 + lane * 4 + i;
        if (p.drop_mask && c < p.N && p.drop_mask[((int64_t)b * p.L + l) * p.N + c] != 0) key[i] = -CUDART_INF_F;
        if (p.rank_keys && c < p.N) p.rank_keys[(((int64_t)b * p.L + l) * p.h_kv + h) * p.N + c] = key[i];
        const bool cand = key[i] > -CUDART_INF_F;  // false for NaN too
        item[i] = cand ? (((u64)order_bits(key[i]) << 32) | (0xFFFFFFFFu - (uint32_t)c)) : 0ull;
      }
      if (KPL == 1) {
        // sort the tile, keep its best 32, merge with the running (descending, one per lane) list
        const u64 thr = __shfl_sync(0xffffffffu, best[r][0], thr_lane);
        const bool any = item[0] > thr || item[1] > thr || item[2] > thr || item[3] > thr;
        if (__any_sync(0xffffffffu, any)) {
          sort128_desc(item, lane);
          u64 top = 0ull;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const u64 t = __shfl_sync(0xffffffffu, item[i], lane >> 2);
            if ((lane & 3) == i) top = t;
          }
          const u64 rev = __shfl_sync(0xffffffffu, top, 31 - lane);
          best[r][0] = merge32_desc(max64(best[r][0], rev), lane);
        }
      } else {
        // K > 32: insertion into a sorted list spread over the lanes, candidates filtered by a ballot
#pragma unroll
        for (int i4 = 0; i4 < 4; ++i4) {
          u64 thr = 0ull;
#pragma unroll
          for (int i = 0; i < KPL; ++i) {
            u64 t = __shfl_sync(0xffffffffu, best[r][i], thr_lane);
            if (i == thr_i) thr = t;
          }
          unsigned mask = __ballot_sync(0xffffffffu, item[i4] > thr);
          while (mask) {
            const int src = __ffs(mask) - 1;
            mask &= mask - 1;
            const u64 x = __shfl_sync(0xffffffffu, item[i4], src);
            if (x > thr) {
              u64 prev_last = __shfl_up_sync(0xffffffffu, best[r][KPL - 1], 1);
              if (lane == 0) prev_last = ~0ull;
#pragma unroll
              for (int i = KPL - 1; i >= 0; --i) {
                const u64 prev = (i > 0) ? best[r][i - 1] : prev_last;
                const u64 cur = best[r][i];
                best[r][i] = (cur > x) ? cur : ((prev > x) ? x : prev);
              }
#pragma unroll
              for (int i = 0; i < KPL; ++i) {
                u64 t = __shfl_sync(0xffffffffu, best[r][i], thr_lane);
                if (i == thr_i) thr = t;
              }
            }
          }
        }
      }
    }
  }

  // ---------------- epilogue: ascending ids, -1 padding, scores of the picked chunks ----------
  T* scores = static_cast<T*>(p.scores);
  int* my_ids = ids_s + warp * 32 * KPL;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    if (r >= RW) break;
    const int row = warp * RW + r;
    const int l = l0 + row;
    if (l >= p.L) continue;  // warp-uniform
    int32_t* out = p.indices + (((int64_t)b * p.L + l) * p.h_kv + h) * K;
    __syncwarp();
    if (KPL == 1) {
      const u64 it = best[r][0];
      int id = (lane < K && it != 0ull) ? (int)(0xFFFFFFFFu - (uint32_t)(it & 0xFFFFFFFFull)) : 0x7fffffff;
      id = sort32_asc(id, lane);
      if (id == 0x7fffffff) id = -1;
      if (lane < K) out[lane] = id;
      my_ids[lane] = id;
    } else {
#pragma unroll
      for (int i = 0; i < KPL; ++i) {
        const int pos = lane * KPL + i;
        const u64 it = best[r][i];
        my_ids[pos] = (pos < K && it != 0ull) ? (int)(0xFFFFFFFFu - (uint32_t)(it & 0xFFFFFFFFull)) : 0x7fffffff;
      }
      __syncwarp();
      int sorted[KPL], mine[KPL];
#pragma unroll
      for (int i = 0; i < KPL; ++i) {
        const int pos = lane * KPL + i;
        mine[i] = my_ids[pos];
        int rank = 0;
        for (int j = 0; j < K; ++j) {
          const int o = my_ids[j];
          rank += (o < mine[i] || (o == mine[i] && j < pos)) ? 1 : 0;
        }
        sorted[i] = rank;
      }
      __syncwarp();
#pragma unroll
      for (int i = 0; i < KPL; ++i) {
        const int pos = lane * KPL + i;
        if (pos < K) {
          const int v = (mine[i] == 0x7fffffff) ? -1 : mine[i];
          out[sorted[i]] = v;
          my_ids[sorted[i]] = v;
        }
      }
    }
    __syncwarp();
    // scores of the picked chunks: each lane forms the full dot product of its own chunk key
    for (int kp = lane; kp < K; kp += 32) {
      const int id = my_ids[kp];
      for (int g = 0; g < G; ++g) {
        float acc = 0.f;
        if (id >= 0) {
          const T* krow = lmks + (((int64_t)b * p.N + id) * HL + (p.per_qhead ? h * G + g : h)) * D;
          acc = dot_row(q_s + (size_t)(row * G + g) * D, krow, D);
        }
        scores[((((int64_t)b * p.L + l) * p.h_kv + h) * G + g) * K + kp] =
            from_f<T>(id >= 0 ? acc * p.scale : -CUDART_INF_F);
      }
    }
  }
}

// ---- selection for training / prefill shapes, bf16: scores on the warp-level tensor cores -------------
// One CTA = RB consecutive tokens x G group members of one (batch, kv-head): M = RB*G score rows, held
// member-major (row = g*RB + token).  The scaled scores of every candidate chunk of the CTA stay in
// shared memory (fp32), so the keys are read once and nothing is recomputed: log-sum-exp per row, then
// per token a warp builds the ranking keys, finds the K-th largest by bisection over the key bits
// (warp-wide population counts), and compacts the selected ids in ascending order.
constexpr int kSelTile = 128;     // candidates per key tile
constexpr int kSelWarps = 8;      // warp w owns candidates 16w..16w+15 of a tile, and every 8th row / token

struct SelLayout {
  int RB, M, Npad, RSV, NS, SW;   // SW: warps that run the per-token selection (each needs a key-bit row)
  size_t q_off, k_off, v_off, add_off, lt_off, lim_off, bits_off, total;
};

static SelLayout sel_layout_for(int G, int D, int N, int RB, int NS) {
  SelLayout s;
  s.RB = RB;
  s.M = RB * G;
  s.Npad = (N + kSelTile - 1) / kSelTile * kSelTile;
  s.RSV = s.Npad + 8;                                      // row stride of the score rows (floats)
  s.NS = NS;
  size_t o = 0;
  s.q_off = o;    o += (size_t)s.M * (D + 8) * 2;
  // the key tiles are dead once the scores are formed: the per-warp key-bit rows of the selection reuse them
  s.k_off = o;    s.bits_off = o;
  const size_t k_bytes = (size_t)NS * kSelTile * (D + 8) * 2;
  s.SW = ((size_t)kSelWarps * s.Npad * (4 + 2) <= k_bytes) ? kSelWarps : 4;   // bits (u32) + ids (u16) per selecting warp
  o += std::max(k_bytes, (size_t)s.SW * s.Npad * (4 + 2));
  s.v_off = o;    o += (size_t)s.M * s.RSV * 4;
  s.add_off = o;  o += (size_t)G * s.Npad * 4;
  s.lt_off = o;   o += (size_t)s.M * 4;
  s.lim_off = o;  o += (size_t)RB * 4;
  s.total = o;
  return s;
}

// Rows per CTA: as many tokens as keep three (else two, else one) CTAs resident per SM with the scores of
// all candidates in shared memory.  total == 0: no layout fits.
static SelLayout sel_layout(int G, int D, int N, int cta_tiles_max, int per_qhead) {
  const int rb_max = (G == 1) ? 64 : (G == 2) ? 32 : 16;
  const size_t classes[3] = {75 * 1024, 113 * 1024, 200 * 1024};
  for (int c = 0; c < 3; ++c)
    for (int RB = rb_max; RB >= 1; RB >>= 1) {
      if ((RB * G) % 16 != 0 || RB * G > 256 || (per_qhead && RB % 16 != 0)) continue;
      for (int NS = (cta_tiles_max > 1 ? 2 : 1); NS >= 1; --NS) {
        const SelLayout s = sel_layout_for(G, D, N, RB, NS);
        if (s.total <= classes[c]) return s;
      }
    }
  SelLayout none = {};
  return none;
}

template <int NK>   // NK = D / 16
__global__ void __launch_bounds__(kSelWarps * 32) topk_fwd_mma_kernel(TopkParams p, SelLayout sl) {
  constexpr int NT = kSelWarps * 32;             // threads
  constexpr int CW = kSelTile / kSelWarps;       // candidates of a key tile per warp
  constexpr int NBW = CW / 8;                    // 8-candidate blocks per warp
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int D = NK * 16, RS = D + 8, CPR = D / 8;
  const int G = p.G, RB = sl.RB, M = sl.M, Npad = sl.Npad, RSV = sl.RSV, K = p.topk;
  bf16* q_s = reinterpret_cast<bf16*>(smem_raw + sl.q_off);        // [M][RS]
  bf16* k_s = reinterpret_cast<bf16*>(smem_raw + sl.k_off);        // [NS][128][RS]
  float* v_s = reinterpret_cast<float*>(smem_raw + sl.v_off);      // [M][RSV] scaled scores, -inf = no candidate
  float* add_s = reinterpret_cast<float*>(smem_raw + sl.add_off);  // [G][Npad] bias + gumbel
  float* lt_s = reinterpret_cast<float*>(smem_raw + sl.lt_off);    // [M] lse of the window branch, then lse_total
  int* lim_s = reinterpret_cast<int*>(smem_raw + sl.lim_off);      // [RB] candidates of each token
  uint32_t* bits_s = reinterpret_cast<uint32_t*>(smem_raw + sl.bits_off);  // [warps][Npad]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int l0 = blockIdx.x * RB, h = blockIdx.y, b = blockIdx.z;
  const bf16* q = static_cast<const bf16*>(p.q);
  const bf16* lmks = static_cast<const bf16*>(p.lmks);
  const int HL = p.per_qhead ? p.h_kv * G : p.h_kv;
  const bool has_add = p.bias || p.gumbel;
  const int cta_limit = row_limit(p, min(l0 + RB, p.L) - 1);       // limits are non-decreasing in l
  const int ntile = (cta_limit + kSelTile - 1) / kSelTile;
  const int n_pass = p.per_qhead ? G : 1;
  const int total = n_pass * ntile;

  auto load_keys = [&](int it, int stage) {
    const int pass = it / ntile, c0 = (it - pass * ntile) * kSelTile;
    const bf16* src = lmks + ((int64_t)b * p.N * HL + (p.per_qhead ? h * G + pass : h)) * D;
    bf16* dst = k_s + (size_t)stage * kSelTile * RS;
    for (int i = tid; i < kSelTile * CPR; i += NT) {
      const int row = i / CPR, col = (i - row * CPR) * 8;
      if (c0 + row < p.N)                                  // rows past the last key stay stale: never candidates
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst + row * RS + col)),
                     "l"(src + (int64_t)(c0 + row) * HL * D + col) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  if (total > 0) load_keys(0, 0);
  // queries (member-major rows), per-token limits, lse of the window branch, additive terms
  for (int i = tid; i < M * CPR; i += NT) {
    const int row = i / CPR, col = (i - row * CPR) * 8;
    const int g = row / RB, l = l0 + (row - g * RB);
    uint4 x = make_uint4(0u, 0u, 0u, 0u);
    if (l < p.L) x = *reinterpret_cast<const uint4*>(q + ((((int64_t)b * p.L + l) * p.h_kv + h) * G + g) * D + col);
    *reinterpret_cast<uint4*>(q_s + row * RS + col) = x;
  }
  for (int t = tid; t < RB; t += NT) lim_s[t] = row_limit(p, l0 + t);
  for (int row = tid; row < M; row += NT) {
    const int g = row / RB, l = l0 + (row - g * RB);
    float ls = 0.f;
    if (l < p.L) {
      const int64_t o = (((int64_t)b * p.L + l) * p.h_kv + h) * G + g;
      ls = (p.lse_dtype == HILS_BF16) ? to_f(static_cast<const bf16*>(p.lse_swa)[o])
                                      : static_cast<const float*>(p.lse_swa)[o];
    }
    lt_s[row] = ls;
  }
  if (has_add)
    for (int g = 0; g < G; ++g)
      for (int c = tid; c < ntile * kSelTile; c += NT) {
        float x = 0.f;
        if (c < p.N) {
          if (p.bias) x += p.bias[(((int64_t)b * p.N + c) * p.h_kv + h) * G + g];
          if (p.gumbel) x += p.gumbel[(int64_t)(h * G + g) * p.N + c];
        }
        add_s[g * Npad + c] = x;
      }

  // ---------------- scores: A = query rows, B = key tile, fp32 accumulators -> v_s --------------------------
  const int mb_pass = p.per_qhead ? RB / 16 : M / 16;      // 16-row blocks multiplied with one key tile
  const uint32_t q32 = (uint32_t)__cvta_generic_to_shared(q_s);
  const uint32_t k32 = (uint32_t)__cvta_generic_to_shared(k_s);
  const uint32_t a_off = (uint32_t)(((lane & 7) + ((lane >> 3) & 1) * 8) * RS + (lane >> 4) * 8) * 2u;
  const uint32_t b_off = (uint32_t)((warp * CW + (lane & 7) + ((lane >> 4) & 1) * 8) * RS + ((lane >> 3) & 1) * 8) * 2u;
  for (int it = 0; it < total; ++it) {
    const int stage = (sl.NS == 2) ? (it & 1) : 0;
    if (sl.NS == 2 && it + 1 < total) {
      load_keys(it + 1, stage ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const int pass = it / ntile, c0 = (it - pass * ntile) * kSelTile;
    const int cw = c0 + warp * CW;
    if (cw < cta_limit) {
      const uint32_t kb = k32 + (uint32_t)stage * (kSelTile * RS * 2) + b_off;
      for (int mb0 = 0; mb0 < mb_pass; mb0 += 4) {
        const int row_base = (p.per_qhead ? pass * RB : 0) + mb0 * 16;
        const int nmb = min(4, mb_pass - mb0);
        float acc[4][NBW][4];
#pragma unroll
        for (int mi = 0; mi < 4; ++mi)
#pragma unroll
          for (int ni = 0; ni < NBW; ++ni)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[mi][ni][e] = 0.f;
#pragma unroll
        for (int kk = 0; kk < NK; ++kk) {
          uint32_t bfr[NBW][2];
#pragma unroll
          for (int np = 0; np < NBW / 2; ++np)             // two 8-candidate blocks per ldmatrix.x4
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                         : "=r"(bfr[2 * np][0]), "=r"(bfr[2 * np][1]), "=r"(bfr[2 * np + 1][0]), "=r"(bfr[2 * np + 1][1])
                         : "r"(kb + (uint32_t)(np * 16 * RS * 2 + kk * 32)));
#pragma unroll
          for (int mi = 0; mi < 4; ++mi) {
            if (mi < nmb) {
              uint32_t a[4];
              asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                           : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3])
                           : "r"(q32 + (uint32_t)((row_base + mi * 16) * RS * 2 + kk * 32) + a_off));
#pragma unroll
              for (int ni = 0; ni < NBW; ++ni)
                asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                             : "+f"(acc[mi][ni][0]), "+f"(acc[mi][ni][1]), "+f"(acc[mi][ni][2]), "+f"(acc[mi][ni][3])
                             : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(bfr[ni][0]), "r"(bfr[ni][1]));
            }
          }
        }
        // accumulator rows lane/4 and lane/4+8 of each block, columns 2*(lane%4)+{0,1} of each 8-candidate block
#pragma unroll
        for (int mi = 0; mi < 4; ++mi) {
          if (mi < nmb) {
#pragma unroll
            for (int hr = 0; hr < 2; ++hr) {
              const int row = row_base + mi * 16 + (lane >> 2) + hr * 8;
              const int lim = lim_s[row & (RB - 1)];
              float* vrow = v_s + (size_t)row * RSV + cw + (lane & 3) * 2;
#pragma unroll
              for (int ni = 0; ni < NBW; ++ni) {
                const int c = cw + ni * 8 + (lane & 3) * 2;
                float2 o;
                o.x = (c < lim) ? __fmul_rn(acc[mi][ni][2 * hr], p.scale) : -CUDART_INF_F;
                o.y = (c + 1 < lim) ? __fmul_rn(acc[mi][ni][2 * hr + 1], p.scale) : -CUDART_INF_F;
                *reinterpret_cast<float2*>(vrow + ni * 8) = o;
              }
            }
          }
        }
      }
    }
    __syncthreads();
    if (sl.NS == 1 && it + 1 < total) load_keys(it + 1, 0);
  }
  if (total == 0) __syncthreads();

  // ---------------- log-sum-exp of the selection logits per row, lse_total ---------------------------------
  for (int row = warp; row < M; row += kSelWarps) {
    const int g = row / RB, tok = row - g * RB, l = l0 + tok;
    if (l >= p.L) continue;                                 // warp-uniform
    const int lim = lim_s[tok];
    const float* vrow = v_s + (size_t)row * RSV;
    const float* arow = add_s + g * Npad;
    float m = -CUDART_INF_F;
    for (int c = lane; c < lim; c += 32) m = fmaxf(m, has_add ? vrow[c] + arow[c] : vrow[c]);
    m = warp_max(m);
    float sum = 0.f;
    if (m > -CUDART_INF_F)
      for (int c = lane; c < lim; c += 32) sum += expf((has_add ? vrow[c] + arow[c] : vrow[c]) - m);
    sum = warp_sum(sum);
    if (lane == 0) {
      const float lh = (sum > 0.f) ? m + logf(sum) : -CUDART_INF_F;
      const float lt = log_add_exp(lt_s[row], lh);
      lt_s[row] = lt;
      if (p.lse_total) p.lse_total[(((int64_t)b * p.L + l) * p.h_kv + h) * G + g] = lt;
    }
  }
  __syncthreads();

  // ---------------- per token: ranking keys, K-th largest by bisection, ordered compaction ------------------
  uint32_t* bits = bits_s + warp * Npad;
  uint16_t* cand_id = reinterpret_cast<uint16_t*>(bits_s + sl.SW * Npad) + warp * Npad;   // long rows: ids of the survivors
  bf16* scores = static_cast<bf16*>(p.scores);
  const uint32_t lt_mask = (1u << lane) - 1u;
  for (int tok = warp; tok < RB; tok += sl.SW) {
    if (warp >= sl.SW) break;
    const int l = l0 + tok;
    if (l >= p.L) continue;                                 // warp-uniform
    const int lim = lim_s[tok];
    const int lim32 = (lim + 31) & ~31;
    const int key_end = p.rank_keys ? ((p.N + 31) & ~31) : lim32;
    int n_cand = 0;
    uint32_t lane_max = 0u;
    __syncwarp();
    for (int c = lane; c < key_end; c += 32) {
      float key = -CUDART_INF_F;
      if (c < lim) {
        for (int g = 0; g < G; ++g) {
          float v = v_s[(size_t)(g * RB + tok) * RSV + c];
          if (has_add) v += add_s[g * Npad + c];
          if (v > -CUDART_INF_F) key = fmaxf(key, v - lt_s[g * RB + tok]);
        }
        if (p.drop_mask && p.drop_mask[((int64_t)b * p.L + l) * p.N + c] != 0) key = -CUDART_INF_F;
      }
      if (p.rank_keys && c < p.N) p.rank_keys[(((int64_t)b * p.L + l) * p.h_kv + h) * p.N + c] = key;
      const uint32_t u = (key > -CUDART_INF_F) ? order_bits(key) : 0u;   // false for NaN too
      if (c < lim32) bits[c] = u;
      n_cand += (u != 0u) ? 1 : 0;
      lane_max = max(lane_max, u);
    }
    n_cand = __reduce_add_sync(0xffffffffu, n_cand);
    __syncwarp();
    // thr / take: chunks with bits > thr are selected, plus the `take` lowest-id chunks with bits == thr
    uint32_t thr = 0u;
    int take = 0, scan_end = lim32;
    bool compacted = false;
    if (n_cand > K) {
      // The K-th largest lies between the smallest per-lane maximum (32 distinct elements are at least that
      // large; used for K <= 32) and the row maximum: the bits above their highest differing bit are known.
      const uint32_t row_max = __reduce_max_sync(0xffffffffu, lane_max);
      const uint32_t floor_u = (K <= 32) ? __reduce_min_sync(0xffffffffu, lane_max) : 0u;
      const uint32_t diff = row_max ^ floor_u;
      const int top = diff ? 31 - __clz(diff) : -1;
      thr = (top >= 0) ? (top == 31 ? 0u : (row_max & ~((2u << top) - 1u))) : row_max;
      if (lim32 <= 128) {                                   // the whole row in registers
        uint32_t u[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) u[i] = (lane + 32 * i < lim32) ? bits[lane + 32 * i] : 0u;
        bool exact = false;
        for (int bit = top; bit >= 0; --bit) {
          const uint32_t trial = thr | (1u << bit);
          int cnt = (u[0] >= trial) + (u[1] >= trial) + (u[2] >= trial) + (u[3] >= trial);
          cnt = __reduce_add_sync(0xffffffffu, cnt);
          if (cnt >= K) {
            thr = trial;
            if (cnt == K) { exact = true; break; }
          }
        }
        if (exact) {
          thr -= 1u;                                        // bits > thr  <=>  bits >= trial: exactly K chunks
        } else {
          int gt = (u[0] > thr) + (u[1] > thr) + (u[2] > thr) + (u[3] > thr);
          take = K - __reduce_add_sync(0xffffffffu, gt);
        }
      } else {
        // long row: keep only the survivors (bits >= floor_u), compacted in id order together with their
        // ids, then bisect and select over the short survivor list
        if (floor_u > 0u && Npad <= 65536) {
          int n_s = 0;
          for (int c0 = 0; c0 < lim32; c0 += 32) {
            const uint32_t u = bits[c0 + lane];
            const bool keep = u >= floor_u;
            const uint32_t m = __ballot_sync(0xffffffffu, keep);
            if (keep) {
              const int pos = n_s + __popc(m & lt_mask);     // pos <= c0 + lane: in place is safe
              bits[pos] = u;
              cand_id[pos] = (uint16_t)(c0 + lane);
            }
            n_s += __popc(m);
          }
          const int n_s32 = (n_s + 31) & ~31;
          if (n_s + lane < n_s32) bits[n_s + lane] = 0u;      // pad the last group
          __syncwarp();
          compacted = true;
          scan_end = n_s32;
        }
        bool exact = false;
        for (int bit = top; bit >= 0; --bit) {
          const uint32_t trial = thr | (1u << bit);
          int cnt = 0;
          for (int c = lane; c < scan_end; c += 32) cnt += (bits[c] >= trial) ? 1 : 0;
          cnt = __reduce_add_sync(0xffffffffu, cnt);
          if (cnt >= K) {
            thr = trial;
            if (cnt == K) { exact = true; break; }
          }
        }
        if (exact) {
          thr -= 1u;
        } else {
          int gt = 0;
          for (int c = lane; c < scan_end; c += 32) gt += (bits[c] > thr) ? 1 : 0;
          take = K - __reduce_add_sync(0xffffffffu, gt);
        }
      }
    }
    // compaction in chunk-id order
    int32_t* out_ids = p.indices + (((int64_t)b * p.L + l) * p.h_kv + h) * K;
    bf16* out_sc = scores + ((((int64_t)b * p.L + l) * p.h_kv + h) * G) * K;
    int n_out = 0, eq_seen = 0;
    for (int c0 = 0; c0 < scan_end; c0 += 32) {
      const uint32_t u = bits[c0 + lane];
      const int c = compacted ? (int)cand_id[c0 + lane] : c0 + lane;
      const bool is_eq = take > 0 && u == thr;
      const uint32_t m_eq = __ballot_sync(0xffffffffu, is_eq);
      const bool sel = (u > thr) || (is_eq && eq_seen + __popc(m_eq & lt_mask) < take);
      const uint32_t m_sel = __ballot_sync(0xffffffffu, sel);
      if (sel) {
        const int pos = n_out + __popc(m_sel & lt_mask);
        if (pos < K) {
          out_ids[pos] = c;
          for (int g = 0; g < G; ++g)
            out_sc[g * K + pos] = __float2bfloat16_rn(v_s[(size_t)(g * RB + tok) * RSV + c]);
        }
      }
      n_out += __popc(m_sel);
      eq_seen += __popc(m_eq);
    }
    for (int pos = n_out + lane; pos < K; pos += 32) {
      out_ids[pos] = -1;
      for (int g = 0; g < G; ++g) out_sc[g * K + pos] = __float2bfloat16_rn(-CUDART_INF_F);
    }
  }
}

template <int NK>
static int launch_topk_mma(const TopkParams& p, cudaStream_t st) {
  // largest number of key tiles any CTA walks (the last tokens see the most chunks)
  TopkParams hp = p;
  const int max_lim = p.is_causal ? std::max(0, std::min(p.N, (p.window_size > 0)
                          ? (p.q_offset + p.L - 1 - p.window_size + 1) / p.block_size
                          : (p.q_offset + p.L - 1) / p.block_size)) : p.N;
  const SelLayout sl = sel_layout(p.G, p.D, p.N, (max_lim + kSelTile - 1) / kSelTile, p.per_qhead);
  if (sl.total == 0) return HILS_ERR_UNSUPPORTED;
  cudaFuncSetAttribute(topk_fwd_mma_kernel<NK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sl.total);
  dim3 grid((p.L + sl.RB - 1) / sl.RB, p.h_kv, p.B);
  topk_fwd_mma_kernel<NK><<<grid, kSelWarps * 32, sl.total, st>>>(hp, sl);
  HILS_LAUNCH_CHECK("topk_fwd (tensor-core scores)");
  return HILS_OK;
}

// Raw dot products q.k' of the decode selection, bf16: a pure streaming kernel.  One persistent CTA per SM
// walks work items = (batch, query row, kv-head[, group member], range of kDotKeys keys); the 64-key tiles of
// consecutive items flow through ONE cp.async ring that fills almost all of the SM's shared memory, so about
// 190 KB of loads are in flight per SM at any time - what it takes to cover HBM latency at full bandwidth (a
// register-resident or two-CTA design holds a third of that and stalls at ~3.7 TB/s).  Warp w computes keys
// 16w..16w+15 of a tile with mma.sync m16n8k16; the item's query rows travel in the stage of its first tile.
constexpr int kDotKeys = 1024, kDotTile = 128;   // warp w computes keys 16w..16w+15 of a tile

struct DotCursor {
  int item, tile, ntile, key_lo, key_hi;
  const bf16* keys;      // key row key_lo of the item's key head, advanced tile by tile
  const bf16* q;         // the item's query rows
  float* out;            // dots of the item's first fragment row, advanced tile by tile
};

template <int NK, int STAGES>
__global__ void __launch_bounds__(256, 1) topk_decode_dots_kernel(TopkParams p, int Npad, int n_items, int ranges) {
  constexpr int stages = STAGES;
  constexpr int D = NK * 16, RS = D + 8, CPR = D / 8;
  constexpr int kStageRows = kDotTile + 16;              // key rows + query rows
  constexpr uint32_t kStageBytes = kStageRows * RS * 2;
  extern __shared__ __align__(16) unsigned char ring[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = p.G, ng = p.per_qhead ? G : 1;
  const int HL = p.per_qhead ? p.h_kv * G : p.h_kv;
  const int64_t rs = (int64_t)HL * D;
  const uint32_t ring32 = (uint32_t)__cvta_generic_to_shared(ring);

  auto load_item = [&](DotCursor& c) {                   // skips items without candidates
    for (; c.item < n_items; c.item += gridDim.x) {
      const int r = c.item % ranges, x = c.item / ranges;
      const int g0 = x % ng, row = x / ng;                 // row = (b*L + l)*h_kv + h
      const int h = row % p.h_kv, bl = row / p.h_kv, l = bl % p.L;
      const int64_t b = bl / p.L;
      const int lim = row_limit_b(p, (int)b, l);
      c.key_lo = r * kDotKeys;
      c.key_hi = min(lim, c.key_lo + kDotKeys);
      c.tile = 0;
      c.ntile = (c.key_hi - c.key_lo + kDotTile - 1) / kDotTile;
      if (c.ntile > 0) {
        c.keys = static_cast<const bf16*>(p.lmks) + ((b * p.N + c.key_lo) * HL + (p.per_qhead ? h * G + g0 : h)) * D;
        c.q = static_cast<const bf16*>(p.q) + ((int64_t)row * G + (p.per_qhead ? g0 : 0)) * D;
        c.out = p.dots + ((int64_t)row * G + (p.per_qhead ? g0 : 0)) * Npad + c.key_lo;
        return;
      }
    }
  };
  auto advance = [&](DotCursor& c) {
    if (++c.tile == c.ntile) {
      c.item += gridDim.x;
      load_item(c);
    } else {
      c.keys += (int64_t)kDotTile * rs;
      c.out += kDotTile;
      c.key_lo += kDotTile;                                // key_lo is now the first key of the current tile
    }
  };
  const int cp_row = tid / CPR, cp_col = (tid % CPR) * 8;   // this thread's 16-byte pieces: rows cp_row + i*(256/CPR)
  constexpr int RSTEP = 256 / CPR, NCP = kDotTile / RSTEP;
  const uint32_t cp_dst = (uint32_t)(cp_row * RS + cp_col) * 2u;
  const int64_t cp_src = (int64_t)cp_row * rs + cp_col, cp_step = (int64_t)RSTEP * rs;
  auto issue = [&](DotCursor& c, int stage) {
    if (c.item < n_items) {
      const uint32_t dst = ring32 + (uint32_t)stage * kStageBytes + cp_dst;
      const bf16* src = c.keys + cp_src;
      const int key0 = c.key_lo + cp_row;
#pragma unroll
      for (int i = 0; i < NCP; ++i)
        if (key0 + i * RSTEP < c.key_hi)                  // rows past the range stay stale: never stored
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + (uint32_t)(i * RSTEP * RS * 2)),
                       "l"(src + i * cp_step) : "memory");
      if (c.tile == 0) {                                  // the item's query rows ride in this stage
        const int nq = p.per_qhead ? 1 : G;
        if (tid < nq * CPR)                               // thread's piece: query row cp_row, columns cp_col..
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ring32 + (uint32_t)stage * kStageBytes +
                       (uint32_t)(kDotTile * RS * 2) + cp_dst), "l"(c.q + cp_row * D + cp_col) : "memory");
      }
      advance(c);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // query rows beyond the group are zero in every stage
  for (int i = tid; i < stages * 16 * RS; i += 256) {
    const int st = i / (16 * RS), o = i - st * 16 * RS;
    reinterpret_cast<bf16*>(ring + (size_t)st * kStageBytes)[kDotTile * RS + o] = __float2bfloat16_rn(0.f);
  }
  __syncthreads();
  DotCursor prod, cons;
  prod.item = cons.item = blockIdx.x;
  load_item(prod);
  cons = prod;
  int st_issue = 0, st_use = 0;
  for (int i = 0; i < stages - 1; ++i) {
    issue(prod, st_issue);
    if (++st_issue == stages) st_issue = 0;
  }
  uint32_t af[NK][4];
  const uint32_t a_off = (uint32_t)((kDotTile + (lane & 7) + ((lane >> 3) & 1) * 8) * RS + (lane >> 4) * 8) * 2u;
  const uint32_t b_off = (uint32_t)((warp * 16 + (lane & 7) + ((lane >> 4) & 1) * 8) * RS + ((lane >> 3) & 1) * 8) * 2u;
  const int kr = lane >> 2, j = lane & 3;
  while (cons.item < n_items) {
    asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
    __syncthreads();
    issue(prod, st_issue);
    if (++st_issue == stages) st_issue = 0;
    const uint32_t sbase = ring32 + (uint32_t)st_use * kStageBytes;
    if (cons.tile == 0) {
#pragma unroll
      for (int kk = 0; kk < NK; ++kk)
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(af[kk][0]), "=r"(af[kk][1]), "=r"(af[kk][2]), "=r"(af[kk][3]) : "r"(sbase + a_off + kk * 32));
    }
    float ca[4] = {0.f, 0.f, 0.f, 0.f}, cb[4] = {0.f, 0.f, 0.f, 0.f};   // keys 16w..16w+7 and 16w+8..16w+15
#pragma unroll
    for (int kk = 0; kk < NK; ++kk) {
      uint32_t b0, b1, b2, b3;
      asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                   : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(sbase + b_off + kk * 32));
      asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                   : "+f"(ca[0]), "+f"(ca[1]), "+f"(ca[2]), "+f"(ca[3])
                   : "r"(af[kk][0]), "r"(af[kk][1]), "r"(af[kk][2]), "r"(af[kk][3]), "r"(b0), "r"(b1));
      asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                   : "+f"(cb[0]), "+f"(cb[1]), "+f"(cb[2]), "+f"(cb[3])
                   : "r"(af[kk][0]), "r"(af[kk][1]), "r"(af[kk][2]), "r"(af[kk][3]), "r"(b2), "r"(b3));
    }
    {
      const int koff = warp * 16 + 2 * j;                 // even: 8-byte aligned pair
#pragma unroll
      for (int hr = 0; hr < 2; ++hr) {
        const int row = kr + 8 * hr;
        const bool ok = p.per_qhead ? (row == 0) : (row < G);
        if (ok) {
          float* o = cons.out + (int64_t)row * Npad + koff;
          if (cons.key_lo + koff < cons.key_hi) *reinterpret_cast<float2*>(o) = make_float2(ca[2 * hr], ca[2 * hr + 1]);
          if (cons.key_lo + koff + 8 < cons.key_hi)
            *reinterpret_cast<float2*>(o + 8) = make_float2(cb[2 * hr], cb[2 * hr + 1]);
        }
      }
    }
    advance(cons);
    if (++st_use == stages) st_use = 0;
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// Logits of all chunk keys of one (batch, kv-head) for up to 16 query rows, bf16: mma.sync with the B
// fragments loaded straight from the key rows (mma_rows.cuh), warp w taking every 8th group of 32 keys.
// Nothing is staged in shared memory, so the CTA is small and many are resident per SM.
template <int NK>   // NK = D / 16
__device__ __forceinline__ void decode_logits_bf16(const TopkParams& p, const bf16* q, const bf16* lmks, int b, int h,
                                                   int lim, int G, int Npad, int HL, float* q_s, float* v_s, int tid) {
  constexpr int D = NK * 16;
  const int lane = tid & 31, warp = tid >> 5;
  // query rows as fp32 (also used for the returned scores) and the additive terms of the logits
  for (int i = tid; i < G * D; i += 256) q_s[i] = __bfloat162float(q[i]);
  for (int g = 0; g < G; ++g)
    for (int c = tid; c < Npad; c += 256) {
      float add = -CUDART_INF_F;
      if (c < lim) {
        add = 0.f;
        if (p.bias) add = p.bias[(((int64_t)b * p.N + c) * p.h_kv + h) * G + g];
        if (p.gumbel) add += p.gumbel[(int64_t)(h * G + g) * p.N + c];
      }
      v_s[(size_t)g * Npad + c] = add;
    }
  __syncthreads();
  const int ng = p.per_qhead ? G : 1;
  const int64_t rs = (int64_t)HL * D;
  const int kr = lane >> 2, j = lane & 3;
  for (int g0 = 0; g0 < ng; ++g0) {
    uint32_t af[NK][4];
    if (p.per_qhead) make_q_frags<NK>(q_s, lane, af, [g0](int r) { return r == 0 ? g0 : -1; });
    else make_q_frags<NK>(q_s, lane, af, [G](int r) { return r < G ? r : -1; });
    const bf16* base = lmks + ((int64_t)b * p.N * HL + (p.per_qhead ? h * G + g0 : h)) * D;
    for (int k0 = warp * 32; k0 < lim; k0 += 8 * 32) {
      float c[4][4];
      dot32_mma<NK>(af, base + (int64_t)k0 * rs, rs, lim - k0, lane, c);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int key = k0 + u * 8 + 2 * j;
#pragma unroll
        for (int hr = 0; hr < 2; ++hr) {
          const int row = kr + 8 * hr;
          const bool ok = p.per_qhead ? (row == 0) : (row < G);
          if (ok) {
            float* cell = v_s + (size_t)(p.per_qhead ? g0 : row) * Npad + key;
            if (key < lim) cell[0] = __fmul_rn(c[u][2 * hr], p.scale) + cell[0];
            if (key + 1 < lim) cell[1] = __fmul_rn(c[u][2 * hr + 1], p.scale) + cell[1];
          }
        }
      }
    }
  }
}

// ---- selection for decode: few query rows against many chunk keys ----------------------------------
// One CTA per (kv-head, batch, query row).  The chunk keys of that head are streamed once (16 lanes per
// key row, 16-byte loads), logits go to shared memory, then log-sum-exp, ranking keys and the same
// sort/merge selection as above, with the candidate tiles spread over the CTA's 8 warps.
template <typename T, int NK, bool kDots>   // kDots: the logits come from topk_decode_dots_kernel's output
__global__ void __launch_bounds__(256, kDots ? 8 : 1) topk_decode_kernel(TopkParams p) {
  extern __shared__ __align__(16) float smem[];
  const int G = p.G, D = p.D, N = p.N, K = p.topk;
  const int Npad = (N + 127) & ~127;
  float* q_s = smem;                         // [G][D]
  float* v_s = q_s + G * D;                  // [G][Npad] selection logits
  float* key_s = v_s + (size_t)G * Npad;     // [Npad]
  float* red_s = key_s + Npad;               // [G][16] partial (max, sum) + [G] lse_total
  u64* list_s = reinterpret_cast<u64*>(red_s + 16 * G + ((G + 1) & ~1));  // 2 KB of selection scratch
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int h = blockIdx.x, b = blockIdx.y, l = blockIdx.z;
  const T* q = static_cast<const T*>(p.q) + ((((int64_t)b * p.L + l) * p.h_kv + h) * G) * D;
  const T* lmks = static_cast<const T*>(p.lmks);
  const int HL = p.per_qhead ? p.h_kv * G : p.h_kv;
  const int lim = row_limit_b(p, b, l);
  float ls_mine = 0.f;                        // thread g < G: lse of the sliding-window branch of member g
  if (tid < G) {
    const int64_t o = (((int64_t)b * p.L + l) * p.h_kv + h) * G + tid;
    ls_mine = (p.lse_dtype == HILS_BF16) ? to_f(static_cast<const bf16*>(p.lse_swa)[o])
                                         : static_cast<const float*>(p.lse_swa)[o];
  }
  // ---- logits ------------------------------------------------------------------------------------
  constexpr bool kIsBf16 = sizeof(T) == 2;
  if constexpr (kDots) {
    // the dots were streamed by topk_decode_dots_kernel: logits = fl(dot * scale) + bias (+ gumbel)
    for (int i = tid; i < G * D; i += 256) q_s[i] = to_f(q[i]);
    const float* dots = p.dots + ((((int64_t)b * p.L + l) * p.h_kv + h) * G) * (int64_t)Npad;
    for (int g = 0; g < G; ++g)
      for (int c = tid; c < Npad; c += 256) {
        float v = -CUDART_INF_F;
        if (c < lim) {
          v = __fmul_rn(dots[(int64_t)g * Npad + c], p.scale);
          if (p.bias) v += p.bias[(((int64_t)b * N + c) * p.h_kv + h) * G + g];
          if (p.gumbel) v += p.gumbel[(int64_t)(h * G + g) * N + c];
        }
        v_s[(size_t)g * Npad + c] = v;
      }
  } else if constexpr (kIsBf16) {
    decode_logits_bf16<NK>(p, reinterpret_cast<const bf16*>(q), reinterpret_cast<const bf16*>(lmks), b, h, lim, G, Npad,
                           HL, q_s, v_s, tid);
  } else {
  for (int i = tid; i < G * D; i += 256) q_s[i] = to_f(q[i]);
  __syncthreads();
  // exact fp32 form: half-warp per chunk key
  const int hw = tid >> 4, sub = tid & 15, per = D / 16;
  const int ng = p.per_qhead ? G : 1;
  for (int cb = 0; cb < Npad; cb += 64) {                 // four key rows in flight per half-warp
    for (int g0 = 0; g0 < ng; ++g0) {
      float kv[4][8];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = cb + u * 16 + hw;
        if (c < lim) {
          const T* krow = lmks + (((int64_t)b * N + c) * HL + (p.per_qhead ? h * G + g0 : h)) * D + sub * per;
          for (int e = 0; e < per; e += 4) {
            const float4 x = load4(krow + e);
            kv[u][e] = x.x; kv[u][e + 1] = x.y; kv[u][e + 2] = x.z; kv[u][e + 3] = x.w;
          }
        }
      }
      const int gl = p.per_qhead ? g0 : 0, gh = p.per_qhead ? g0 + 1 : G;
      for (int g = gl; g < gh; ++g) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int c = cb + u * 16 + hw;
          const bool live = c < lim;
          float acc = 0.f;
          if (live)
            for (int e = 0; e < per; ++e) acc = fmaf(q_s[g * D + sub * per + e], kv[u][e], acc);
#pragma unroll
          for (int o = 8; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
          if (sub == 0 && c < Npad) {
            float v = -CUDART_INF_F;
            if (live) {
              v = acc * p.scale;
              if (p.bias) v += p.bias[(((int64_t)b * N + c) * p.h_kv + h) * G + g];
              if (p.gumbel) v += p.gumbel[(int64_t)(h * G + g) * N + c];
            }
            v_s[(size_t)g * Npad + c] = v;
          }
        }
      }
    }
  }
  }
  __syncthreads();
  // ---- log-sum-exp per group member (one online pass), lse_total ------------------------------------
  for (int g = 0; g < G; ++g) {
    float m = -CUDART_INF_F, sum = 0.f;
    for (int c = tid; c < lim; c += 256) {
      const float v = v_s[(size_t)g * Npad + c];
      if (v > -CUDART_INF_F) {
        const float nm = fmaxf(m, v);
        sum = sum * __expf(m - nm) + __expf(v - nm);
        m = nm;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, sum, o);
      const float nm = fmaxf(m, om);
      sum = (nm > -CUDART_INF_F) ? sum * __expf(m - nm) + os * __expf(om - nm) : 0.f;
      m = nm;
    }
    if (lane == 0) { red_s[g * 16 + warp] = m; red_s[g * 16 + 8 + warp] = sum; }
  }
  __syncthreads();
  if (tid < G) {
    const float* r = red_s + tid * 16;
    float m = r[0];
    for (int w = 1; w < 8; ++w) m = fmaxf(m, r[w]);
    float tot = 0.f;
    if (m > -CUDART_INF_F)
      for (int w = 0; w < 8; ++w) tot += r[8 + w] * expf(r[w] - m);
    const float lh = (tot > 0.f) ? m + logf(tot) : -CUDART_INF_F;
    const float lt = log_add_exp(ls_mine, lh);
    red_s[16 * G + tid] = lt;
    if (p.lse_total) p.lse_total[(((int64_t)b * p.L + l) * p.h_kv + h) * G + tid] = lt;
  }
  __syncthreads();
  // ---- ranking keys, kept as order-preserving bits (0 = not a candidate) -------------------------
  uint32_t* bits_s = reinterpret_cast<uint32_t*>(key_s);
  uint32_t* hist = reinterpret_cast<uint32_t*>(list_s);   // [256]
  uint32_t* wsum = hist + 256;                            // [8]
  uint32_t* ctl = wsum + 8;                               // [4]: prefix, remaining rank, done
  int* sel_ids = reinterpret_cast<int*>(ctl + 4);         // [32]
  for (int c = tid; c < Npad; c += 256) {
    float key = -CUDART_INF_F;
    if (c < lim) {
      for (int g = 0; g < G; ++g) {
        const float v = v_s[(size_t)g * Npad + c];
        if (v > -CUDART_INF_F) key = fmaxf(key, v - red_s[16 * G + g]);
      }
      if (p.drop_mask && p.drop_mask[((int64_t)b * p.L + l) * N + c] != 0) key = -CUDART_INF_F;
    }
    bits_s[c] = (key > -CUDART_INF_F) ? order_bits(key) : 0u;   // false for NaN too
    if (p.rank_keys && c < N) p.rank_keys[(((int64_t)b * p.L + l) * p.h_kv + h) * N + c] = key;
  }
  if (tid < 32) sel_ids[tid] = -1;
  // ---- the K-th largest key by radix select (8 bits per pass, most significant first) ---------------
  // thr = bits of the K-th largest candidate, take = how many candidates equal to thr are selected
  // (those with the lowest chunk ids); fewer than K candidates: thr = 0 and every candidate is taken.
  uint32_t thr = 0u, mask = 0u;
  int take = K;
  for (int shift = 24; shift >= 0; shift -= 8) {
    hist[tid] = 0u;
    __syncthreads();
    for (int c = tid; c < Npad; c += 256) {
      const uint32_t u = bits_s[c];                       // whole warps run this loop together
      const bool act = u != 0u && (u & mask) == thr;
      const uint32_t digit = (u >> shift) & 255u;
      const uint32_t among = __ballot_sync(0xffffffffu, act);
      if (act) {                                          // one atomic per distinct digit in the warp
        const uint32_t peers = __match_any_sync(among, digit);
        if (lane == __ffs(peers) - 1) atomicAdd(&hist[digit], (uint32_t)__popc(peers));
      }
    }
    __syncthreads();
    if (warp == 0) {
      uint32_t cnt[8], tot = 0u;                          // lane 0 holds the 8 highest digits
#pragma unroll
      for (int j = 0; j < 8; ++j) { cnt[j] = hist[255 - (lane * 8 + j)]; tot += cnt[j]; }
      uint32_t inc = tot;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t x = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += x;
      }
      const uint32_t exc = inc - tot;
      const bool here = exc < (uint32_t)take && (uint32_t)take <= inc;
      if (here) {
        uint32_t run = exc;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (run < (uint32_t)take && (uint32_t)take <= run + cnt[j]) {
            ctl[0] = thr | ((uint32_t)(255 - (lane * 8 + j)) << shift);
            ctl[1] = (uint32_t)take - run;
            ctl[2] = 0u;
          }
          run += cnt[j];
        }
      }
      if (!__any_sync(0xffffffffu, here) && lane == 0) { ctl[0] = 0u; ctl[1] = 0u; ctl[2] = 1u; }
    }
    __syncthreads();
    thr = ctl[0]; take = (int)ctl[1];
    mask |= 0xFFu << shift;
    if (ctl[2]) break;
  }
  // ---- compaction in chunk-id order: ids come out ascending ---------------------------------------------
  {
    const int per = (Npad + 255) >> 8, c0 = tid * per, c1 = min(c0 + per, Npad);
    uint32_t n_gt = 0u, n_eq = 0u;
    for (int c = c0; c < c1; ++c) {
      const uint32_t u = bits_s[c];
      n_gt += (u > thr) ? 1u : 0u;
      n_eq += (u == thr && thr != 0u) ? 1u : 0u;
    }
    const uint32_t mine = (n_gt << 16) | n_eq;
    uint32_t inc = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t x = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += x;
    }
    if (lane == 31) wsum[warp] = inc;
    __syncthreads();
    uint32_t before = inc - mine;
    for (int w = 0; w < warp; ++w) before += wsum[w];
    uint32_t eq_rank = before & 0xFFFFu;
    int pos = (int)(before >> 16) + (int)min(eq_rank, (uint32_t)take);
    for (int c = c0; c < c1; ++c) {
      const uint32_t u = bits_s[c];
      bool sel = u > thr;
      if (u == thr && thr != 0u) { sel = eq_rank < (uint32_t)take; ++eq_rank; }
      if (sel && pos < 32) sel_ids[pos++] = c;
    }
  }
  __syncthreads();
  // ---- ids and the raw scores of the selected chunks: eight lanes per chunk, four chunks per warp ------
  for (int k0 = warp * 4; k0 < K; k0 += 32) {
    const int k = k0 + (lane >> 3), sub = lane & 7;
    const int id = (k < K) ? sel_ids[k] : -1;
    if (sub == 0 && k < K) p.indices[(((int64_t)b * p.L + l) * p.h_kv + h) * K + k] = id;
    T* scores = static_cast<T*>(p.scores);
    for (int g = 0; g < G; ++g) {
      float acc = 0.f;
      if (id >= 0) {
        const T* krow = lmks + (((int64_t)b * N + id) * HL + (p.per_qhead ? h * G + g : h)) * D;
        for (int e = sub * 4; e < D; e += 32) {
          const float4 x = load4(krow + e);
          const float* qq = q_s + g * D + e;
          acc = fmaf(qq[0], x.x, acc); acc = fmaf(qq[1], x.y, acc);
          acc = fmaf(qq[2], x.z, acc); acc = fmaf(qq[3], x.w, acc);
        }
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 4);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      if (sub == 0 && k < K) {
        const T sc = from_f<T>(id >= 0 ? acc * p.scale : -CUDART_INF_F);
        scores[((((int64_t)b * p.L + l) * p.h_kv + h) * G + g) * K + k] = sc;
        if (p.weights) v_s[g * 32 + k] = to_f(sc);        // the logits in v_s are no longer needed (K <= 32 here)
      }
    }
  }
  // ---- the step's inter-chunk softmax (glue.cu: chunk_weights_fwd_kernel, same roundings): one warp per member ------
  if (p.weights) {
    if (tid < G) v_s[G * 32 + tid] = ls_mine;             // lse of the window branch, already in the chain's dtype
    __syncthreads();
    const int ncol = K + 1 + (p.softmax1 ? 1 : 0);
    for (int g = warp; g < G; g += 8) {
      float x[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int c = lane + 32 * i;
        x[i] = -CUDART_INF_F;
        if (c < K) {
          x[i] = v_s[g * 32 + c];
          if (p.bias) {
            const float bv = p.bias[(((int64_t)b * N + max(sel_ids[c], 0)) * p.h_kv + h) * G + g];
            x[i] = to_f(from_f<T>(x[i] + to_f(from_f<T>(bv))));
          }
        } else if (c == K) {
          x[i] = v_s[G * 32 + g];
        } else if (c < ncol) {
          x[i] = 0.f;
        }
      }
      const float m = warp_max(fmaxf(x[0], x[1]));
      float e[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) e[i] = (lane + 32 * i < ncol && m > -CUDART_INF_F) ? __expf(x[i] - m) : 0.f;
      const float inv = 1.f / warp_sum(e[0] + e[1]);      // all -inf: 0/0 = NaN, as the reference's softmax
      T* wrow = static_cast<T*>(p.weights) + ((((int64_t)b * p.L + l) * p.h_kv + h) * G + g) * ncol;
#pragma unroll
      for (int i = 0; i < 2; ++i)
        if (lane + 32 * i < ncol) wrow[lane + 32 * i] = from_f<T>(e[i] * inv);
    }
  }
}

template <typename T, int NK>
static int launch_topk_decode(const TopkParams& p, cudaStream_t st) {
  const int Npad = (p.N + 127) & ~127;
  size_t smem = ((size_t)p.G * p.D + (size_t)p.G * Npad + Npad + 16 * p.G + ((p.G + 1) & ~1)) * sizeof(float) +
                8 * 32 * sizeof(u64) + 16;
  if (sizeof(T) == 2) {
    if (p.G > 16) return HILS_ERR_UNSUPPORTED;            // one 16-row A tile holds the group
  }
  if (smem > 200 * 1024) return HILS_ERR_UNSUPPORTED;
  if constexpr (sizeof(T) == 2) {
    if (p.dots) {      // stream the keys once at memory speed, then select from the small fp32 dots array
      const int max_lim = row_limit(p, p.L - 1);
      if (max_lim > 0) {
        constexpr int kStages = (NK == 8) ? 5 : 10;        // ~200 KB of ring per SM
        const size_t ring = (size_t)kStages * (kDotTile + 16) * (NK * 16 + 8) * sizeof(bf16);
        const int ranges = (max_lim + kDotKeys - 1) / kDotKeys;
        const int n_items = p.B * p.L * p.h_kv * (p.per_qhead ? p.G : 1) * ranges;
        static int n_sm = 0;
        if (n_sm == 0) {
          int dev = 0;
          cudaGetDevice(&dev);
          cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
        }
        cudaFuncSetAttribute(topk_decode_dots_kernel<NK, kStages>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ring);
        topk_decode_dots_kernel<NK, kStages><<<std::min(n_items, n_sm), 256, ring, st>>>(p, Npad, n_items, ranges);
        HILS_LAUNCH_CHECK("topk_fwd (decode, key stream)");
      }
    }
  }
  dim3 grid(p.h_kv, p.B, p.L);
  if (sizeof(T) == 2 && p.dots) {
    cudaFuncSetAttribute(topk_decode_kernel<T, NK, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    topk_decode_kernel<T, NK, true><<<grid, 256, smem, st>>>(p);
  } else {
    cudaFuncSetAttribute(topk_decode_kernel<T, NK, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    topk_decode_kernel<T, NK, false><<<grid, 256, smem, st>>>(p);
  }
  HILS_LAUNCH_CHECK("topk_fwd (decode)");
  return HILS_OK;
}

// ---- backward of the returned scores ---------------------------------------------------------
// dq[i,g] = scale * sum_k ds[i,g,k] k'_{id_k};  dk'_c += scale * ds[i,g,k] q[i,g]  (fp32 atomics)
template <typename T>
__global__ void __launch_bounds__(128) topk_bwd_kernel(
    const T* __restrict__ ds, const int32_t* __restrict__ indices, const T* __restrict__ q,
    const T* __restrict__ lmks, T* __restrict__ dq, float* __restrict__ dl, int L, int N, int h_kv, int G,
    int D, int K, int per_qhead, float scale, int64_t rows) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 4 + warp;  // (b, l, h_kv, g)
  if (row >= rows) return;
  const int g = (int)(row % G);
  const int64_t blh = row / G;
  const int h = (int)(blh % h_kv);
  const int64_t bl = blh / h_kv;
  const int64_t b = bl / L;
  const int HL = per_qhead ? h_kv * G : h_kv;
  const int hl = per_qhead ? h * G + g : h;
  const int32_t* ids = indices + blh * K;
  const T* dsr = ds + row * K;
  const T* qr = q + row * D;
  for (int d0 = lane * 4; d0 < D; d0 += 128) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 qv = load4(qr + d0);
    for (int k = 0; k < K; ++k) {
      const int id = ids[k];
      if (id < 0 || id >= N) continue;
      const float s = to_f(dsr[k]) * scale;
      const int64_t off = ((b * N + id) * HL + hl) * D + d0;
      float4 kv = load4(lmks + off);
      acc.x = fmaf(s, kv.x, acc.x); acc.y = fmaf(s, kv.y, acc.y);
      acc.z = fmaf(s, kv.z, acc.z); acc.w = fmaf(s, kv.w, acc.w);
      if (dl) {
        atomicAdd(dl + off + 0, s * qv.x); atomicAdd(dl + off + 1, s * qv.y);
        atomicAdd(dl + off + 2, s * qv.z); atomicAdd(dl + off + 3, s * qv.w);
      }
    }
    store4(dq + row * D + d0, acc);
  }
}

int topk_fwd_tc_launch(const TopkParams& p, cudaStream_t st);   // topk_tc.cu
int topk_bwd_mma_launch(const void* d_scores, const int32_t* indices, const void* q, const void* lmks, void* d_q,
                        float* dl, int B, int L, int N, int h_kv, int G, int D, int topk, int per_qhead, float scale,
                        cudaStream_t st);  // topk_bwd_mma.cu

template <typename T, int KPL>
static int launch_topk(const TopkParams& p, cudaStream_t st) {
  TopkParams pp = p;
  // rows per warp: as many as fit in shared memory
  size_t smem = 0;
  int RW = 4;
  for (; RW >= 1; RW >>= 1) {
    int M = 4 * RW * p.G;
    smem = ((size_t)M * p.D + (size_t)TN * (p.D + 4) + (size_t)M * TN + 2 * (size_t)M + (size_t)p.G * TN) *
               sizeof(float) +
           4 * 32 * KPL * sizeof(int);
    if (smem <= 200 * 1024) break;
  }
  if (RW < 1) {
    set_error("topk_fwd: G*D = %d*%d does not fit in shared memory", p.G, p.D);
    return HILS_ERR_UNSUPPORTED;
  }
  pp.RW = RW;
  cudaError_t e = cudaFuncSetAttribute(topk_fwd_kernel<T, KPL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return cuda_fail(e, "topk_fwd smem attribute");
  dim3 grid(ceil_div(p.L, 4 * RW), p.h_kv, p.B);
  topk_fwd_kernel<T, KPL><<<grid, 128, smem, st>>>(pp);
  HILS_LAUNCH_CHECK("topk_fwd");
  return HILS_OK;
}

}  // namespace hils

using namespace hils;

extern "C" size_t hils_topk_fwd_workspace_bytes(int B, int L, int N, int h_kv, int G, int D, int dtype) {
  // only the bf16 decode shape uses scratch: the raw dot products of every candidate, fp32
  if (dtype != HILS_BF16 || L > 4 || N < 512 || !(D == 64 || D == 128) || G > 16) return 0;
  const size_t Npad = ((size_t)N + 127) & ~(size_t)127;
  return (size_t)B * L * h_kv * G * Npad * sizeof(float);
}

extern "C" int hils_topk_fwd(const void* q, const void* lmks, const void* lse_swa, const float* bias,
                             const float* gumbel, const int32_t* drop_mask, int32_t* indices, void* scores,
                             float* lse_total, float* rank_keys, int B, int L, int N, int h_kv, int G, int D,
                             int topk, int block_size, int window_size, int is_causal, int q_offset,
                             int per_qhead, float sm_scale, int dtype, int lse_dtype, void* workspace,
                             size_t workspace_bytes, void* stream) {
  HILS_REQUIRE(B > 0 && L >= 0 && N >= 0 && h_kv > 0 && G > 0 && D > 0, "topk_fwd: non-positive size");
  HILS_REQUIRE(topk > 0 && topk <= 128, "topk_fwd: topk (%d) must be in [1,128]", topk);
  HILS_REQUIRE(block_size > 0, "topk_fwd: block_size must be positive");
  HILS_REQUIRE(D % 4 == 0, "topk_fwd: D (%d) must be a multiple of 4", D);
  HILS_REQUIRE(dtype == HILS_F32 || dtype == HILS_BF16, "topk_fwd: unknown dtype %d", dtype);
  HILS_REQUIRE(lse_dtype == HILS_F32 || lse_dtype == HILS_BF16, "topk_fwd: unknown lse dtype %d", lse_dtype);
  HILS_REQUIRE(B <= 65535 && h_kv <= 65535, "topk_fwd: B and h_kv must be <= 65535");
  if (L == 0) return HILS_OK;
  HILS_REQUIRE(q && lse_swa && indices && scores, "topk_fwd: null pointer");
  HILS_REQUIRE(N == 0 || lmks, "topk_fwd: null chunk keys");
  TopkParams p;
  p.q = q; p.lmks = lmks; p.lse_swa = lse_swa; p.bias = bias; p.gumbel = gumbel; p.drop_mask = drop_mask;
  p.indices = indices; p.scores = scores; p.lse_total = lse_total; p.rank_keys = rank_keys;
  p.B = B; p.L = L; p.N = N; p.h_kv = h_kv; p.G = G; p.D = D; p.topk = topk; p.block_size = block_size;
  p.window_size = window_size; p.is_causal = is_causal; p.q_offset = q_offset; p.per_qhead = per_qhead;
  p.lse_dtype = lse_dtype; p.RW = 4; p.scale = sm_scale; p.dots = nullptr; p.q_offsets = nullptr;
  p.weights = nullptr; p.softmax1 = 0;
  cudaStream_t st = (cudaStream_t)stream;
  // few query rows against many chunk keys (decode, short chunk-prefill): stream the keys once per row
  if (L <= 4 && N >= 512 && topk <= 32 && (D == 64 || D == 128) && L <= 65535) {
    const size_t need = hils_topk_fwd_workspace_bytes(B, L, N, h_kv, G, D, dtype);
    if (workspace && need > 0 && workspace_bytes >= need && (int64_t)B * h_kv <= 65535)
      p.dots = static_cast<float*>(workspace);
    const int rc = (dtype != HILS_BF16) ? launch_topk_decode<float, 0>(p, st)
                   : (D == 128)         ? launch_topk_decode<bf16, 8>(p, st)
                                        : launch_topk_decode<bf16, 4>(p, st);
    if (rc != HILS_ERR_UNSUPPORTED) return rc;
  }
  // bf16, long candidate lists, one query head per key head: one thread per token, scores by tcgen05
  if (dtype == HILS_BF16 && topk <= N) {
    const int rc = topk_fwd_tc_launch(p, st);
    if (rc != HILS_ERR_UNSUPPORTED) return rc;
  }
  // bf16: scores on the tensor cores, the CTA's scores resident in shared memory
  if (dtype == HILS_BF16 && (D == 64 || D == 128) && G <= 16 && topk <= N && L <= 65535 * 16) {
    const int rc = (D == 128) ? launch_topk_mma<8>(p, st) : launch_topk_mma<4>(p, st);
    if (rc != HILS_ERR_UNSUPPORTED) return rc;
  }
  const int kpl = (topk + 31) / 32;
  if (dtype == HILS_BF16) {
    if (kpl == 1) return launch_topk<bf16, 1>(p, st);
    if (kpl == 2) return launch_topk<bf16, 2>(p, st);
    return launch_topk<bf16, 4>(p, st);
  }
  if (kpl == 1) return launch_topk<float, 1>(p, st);
  if (kpl == 2) return launch_topk<float, 2>(p, st);
  return launch_topk<float, 4>(p, st);
}

namespace hils {
// Selection of the decode step: one new query row per sequence, always on the decode kernels, with the step's
// inter-chunk softmax fused behind it (weights, or null).  q_offsets (device, or null) holds each sequence's position
// when the sequences stand at different ones; q_offset is then the largest of them (host; it sizes the key stream).
// The chunk keys are (B, N, heads, D) with N the row stride of every sequence; rows at or past a sequence's own limit
// are never read.  Shapes the decode kernels do not cover are refused (HILS_ERR_UNSUPPORTED).
int topk_decode_step_launch(const void* q, const void* lmks, const void* lse_swa, const float* bias, int32_t* indices,
                            void* scores, void* weights, int softmax1, const int32_t* q_offsets, int q_offset, int B, int N,
                            int h_kv, int G, int D, int topk, int block_size, int window_size, int per_qhead, float sm_scale,
                            int dtype, int lse_dtype, void* workspace, size_t workspace_bytes, cudaStream_t st) {
  if (!(D == 64 || D == 128) || topk > 32 || B > 65535 || h_kv > 65535 || N <= 0) return HILS_ERR_UNSUPPORTED;
  if (weights && lse_dtype != dtype) return HILS_ERR_UNSUPPORTED;
  TopkParams p;
  p.q = q; p.lmks = lmks; p.lse_swa = lse_swa; p.bias = bias; p.gumbel = nullptr; p.drop_mask = nullptr;
  p.indices = indices; p.scores = scores; p.lse_total = nullptr; p.rank_keys = nullptr;
  p.B = B; p.L = 1; p.N = N; p.h_kv = h_kv; p.G = G; p.D = D; p.topk = topk; p.block_size = block_size;
  p.window_size = window_size; p.is_causal = 1; p.q_offset = q_offset; p.per_qhead = per_qhead;
  p.lse_dtype = lse_dtype; p.RW = 4; p.scale = sm_scale; p.dots = nullptr; p.q_offsets = q_offsets;
  p.weights = weights; p.softmax1 = softmax1;
  const size_t need = hils_topk_fwd_workspace_bytes(B, 1, N, h_kv, G, D, dtype);
  if (workspace && need > 0 && workspace_bytes >= need && (int64_t)B * h_kv <= 65535) p.dots = static_cast<float*>(workspace);
  return (dtype != HILS_BF16) ? launch_topk_decode<float, 0>(p, st)
         : (D == 128)         ? launch_topk_decode<bf16, 8>(p, st)
                              : launch_topk_decode<bf16, 4>(p, st);
}
}  // namespace hils

extern "C" int hils_topk_bwd(const void* d_scores, const int32_t* indices, const void* q, const void* lmks,
                             void* d_q, float* d_lmks_f32, void* d_lmks, int B, int L, int N, int h_kv, int G,
                             int D, int topk, int per_qhead, float sm_scale, int dtype, void* stream) {
  HILS_REQUIRE(B > 0 && L >= 0 && N >= 0 && h_kv > 0 && G > 0 && D > 0 && topk > 0, "topk_bwd: bad size");
  HILS_REQUIRE(D % 4 == 0, "topk_bwd: D (%d) must be a multiple of 4", D);
  HILS_REQUIRE(dtype == HILS_F32 || dtype == HILS_BF16, "topk_bwd: unknown dtype %d", dtype);
  cudaStream_t st = (cudaStream_t)stream;
  const int HL = per_qhead ? h_kv * G : h_kv;
  const int64_t nl = (int64_t)B * N * HL * D;
  if (dtype == HILS_BF16 && nl > 0 && L > 0 && (D == 64 || D == 128) && d_lmks_f32) {
    // dense 64 x 128 tiles of the score gradient in shared memory, both products on the tensor cores
    HILS_REQUIRE(d_scores && indices && q && lmks && d_q && d_lmks, "topk_bwd: null pointer");
    cudaError_t e = cudaMemsetAsync(d_lmks_f32, 0, nl * sizeof(float), st);
    if (e != cudaSuccess) return cuda_fail(e, "topk_bwd memset");
    const int rc = topk_bwd_mma_launch(d_scores, indices, q, lmks, d_q, d_lmks_f32, B, L, N, h_kv, G, D, topk, per_qhead,
                                       sm_scale, st);
    if (rc == HILS_OK) {
      launch_cast_from_f32<bf16>(d_lmks_f32, (bf16*)d_lmks, nl, st);
      HILS_LAUNCH_CHECK("topk_bwd cast");
      return HILS_OK;
    }
    if (rc != HILS_ERR_UNSUPPORTED) return rc;
  }
  if (nl > 0) {
    HILS_REQUIRE(d_lmks_f32 && d_lmks, "topk_bwd: null chunk-key gradient buffers");
    cudaError_t e = cudaMemsetAsync(d_lmks_f32, 0, nl * sizeof(float), st);
    if (e != cudaSuccess) return cuda_fail(e, "topk_bwd memset");
  }
  const int64_t rows = (int64_t)B * L * h_kv * G;
  if (rows > 0) {
    HILS_REQUIRE(d_scores && indices && q && d_q, "topk_bwd: null pointer");
    const int blocks = (int)((rows + 3) / 4);
    if (dtype == HILS_BF16)
      topk_bwd_kernel<bf16><<<blocks, 128, 0, st>>>((const bf16*)d_scores, indices, (const bf16*)q,
                                                   (const bf16*)lmks, (bf16*)d_q, d_lmks_f32, L, N, h_kv, G, D,
                                                   topk, per_qhead, sm_scale, rows);
    else
      topk_bwd_kernel<float><<<blocks, 128, 0, st>>>((const float*)d_scores, indices, (const float*)q,
                                                    (const float*)lmks, (float*)d_q, d_lmks_f32, L, N, h_kv, G,
                                                    D, topk, per_qhead, sm_scale, rows);
    HILS_LAUNCH_CHECK("topk_bwd");
  }
  if (nl > 0) {
    if (dtype == HILS_BF16)
      launch_cast_from_f32<bf16>(d_lmks_f32, (bf16*)d_lmks, nl, st);
    else
      launch_cast_from_f32<float>(d_lmks_f32, (float*)d_lmks, nl, st);
    HILS_LAUNCH_CHECK("topk_bwd cast");
  }
  return HILS_OK;
}


// -------------------------------------------------------------------------------------------------
// Selection backward for callers that must not allocate.
//
// Some hosts of this library cannot obtain device memory at call time: code running while a
// caching allocator is frozen or nearly full, a serving process that pinned all of its memory at
// start-up, or a plugin whose owner forbids cudaMalloc after initialisation.  hils_topk_bwd needs
// an fp32 accumulator with the shape of the chunk keys; this variant keeps that accumulator in a
// fixed array inside the library image, so the caller passes only inputs and outputs.
//
// The array is a file-scope __device__ variable.  In host code its name is only a handle, not a
// device address, so the address is fetched once per device with cudaGetSymbolAddress (with that
// device current) and that pointer is what the kernels receive.
// -------------------------------------------------------------------------------------------------
namespace hils {

constexpr size_t kNoAllocFloats = (size_t)1 << 20;  // 4 MiB of fp32, held by every GPU that loads the library
static __device__ __align__(256) float g_topk_bwd_scratch[kNoAllocFloats];

constexpr int kMaxDevices = 64;
static float* g_scratch_ptr[kMaxDevices] = {nullptr};

// device address of the scratch array on the current device (looked up on the first call per device).
// The cache is written without synchronisation: two host threads that race on a device's first call both look the
// symbol up and both store the same address (an aligned pointer store), so the race is benign.
static int noalloc_scratch(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "topk_bwd_noalloc: cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevices) {
    set_error("topk_bwd_noalloc: device ordinal %d outside [0, %d)", dev, kMaxDevices);
    return HILS_ERR_UNSUPPORTED;
  }
  if (!g_scratch_ptr[dev]) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, g_topk_bwd_scratch);
    if (e != cudaSuccess || !ptr) return cuda_fail(e, "topk_bwd_noalloc: cudaGetSymbolAddress");
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return HILS_OK;
}

}  // namespace hils

extern "C" size_t hils_topk_bwd_noalloc_max_elems(void) { return hils::kNoAllocFloats; }

extern "C" int hils_topk_bwd_noalloc(const void* d_scores, const int32_t* indices, const void* q, const void* lmks,
                                     void* d_q, void* d_lmks, int B, int L, int N, int h_kv, int G, int D, int topk,
                                     int per_qhead, float sm_scale, int dtype, void* stream) {
  HILS_REQUIRE(B > 0 && L >= 0 && N >= 0 && h_kv > 0 && G > 0 && D > 0 && topk > 0, "topk_bwd_noalloc: bad size");
  const int HL = per_qhead ? h_kv * G : h_kv;
  const unsigned long long need = (unsigned long long)B * N * HL * D;
  if (need > hils::kNoAllocFloats) {
    set_error("topk_bwd_noalloc: chunk-key gradient of %llu elements (B*N*heads*D) exceeds the built-in scratch of "
              "%zu elements; use hils_topk_bwd with a caller-provided accumulator", need, hils::kNoAllocFloats);
    return HILS_ERR_WORKSPACE;
  }
  float* scratch = nullptr;
  if (int rc = hils::noalloc_scratch(&scratch)) return rc;
  // hils_topk_bwd zeroes the accumulator itself (cudaMemsetAsync on the stream) before accumulating
  return hils_topk_bwd(d_scores, indices, q, lmks, d_q, scratch, d_lmks, B, L, N, h_kv, G, D, topk, per_qhead,
                       sm_scale, dtype, stream);
}
