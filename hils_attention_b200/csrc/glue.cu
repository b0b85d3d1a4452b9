// Inter-chunk softmax and the combination of the two attention branches, forward and backward.
//
// In the reference these steps are a dozen small PyTorch ops inside the attention module
// (models/FlashHiLS/hils_attention.py:585-610 gather of the prior bias, concatenation with the
// sliding-window log-sum-exp and softmax; :620-629 o = o_hils + w_swa * o_swa).  Here each direction
// is one kernel per step: a warp owns one (batch, token, query head) row, so every tensor is read and
// written once.  Roundings follow the reference's sequence of dtype casts: bias rounded to the score
// dtype, the sum rounded to the score dtype, softmax in fp32 rounded once, gradients of the softmax
// rounded to the score dtype before they fan out.
#include "common.cuh"

namespace hils {

constexpr int kMaxCols = 96;        // K + 2 columns at most; 3 per lane
constexpr int kRowsPerCta = 8;      // one warp per row

constexpr int kBatch = 4;           // rows a warp has in flight
constexpr int kFwdRowsPerCta = 512; // rows one CTA walks: amortises staging the bias table of its batch

// The prior bias of one batch (N x h_q fp32) is staged once per CTA in shared memory, transposed to
// [h_q][N+1] so that the K gathers of a row (ascending chunk ids, one head) fall into different banks;
// gathering it from global memory costs one 32-byte sector per element.
template <typename T>
__global__ void __launch_bounds__(32 * kRowsPerCta)
chunk_weights_fwd_kernel(const T* __restrict__ scores, const int32_t* __restrict__ indices,
                         const float* __restrict__ bias, const T* __restrict__ lse_swa, T* __restrict__ weights,
                         uint32_t rows, int L, int N, int h_q, int h_idx, int K, int softmax1, int bias_in_smem,
                         int rows_per_cta) {
  extern __shared__ float bias_s[];                         // [h_q][N + 1] when bias_in_smem
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t cta_row0 = blockIdx.x * (uint32_t)rows_per_cta;
  const uint32_t cta_row1 = min(rows, cta_row0 + (uint32_t)rows_per_cta);
  const uint32_t rows_per_batch = (uint32_t)L * (uint32_t)h_q;
  const uint32_t b0 = cta_row0 / rows_per_batch;
  if (bias && bias_in_smem) {
    const float* src = bias + (int64_t)b0 * N * h_q;
    for (int i = threadIdx.x; i < N * h_q; i += 32 * kRowsPerCta) {
      const int c = i / h_q, hq = i - c * h_q;
      bias_s[hq * (N + 1) + c] = src[i];
    }
    __syncthreads();
  }
  const int g = h_q / h_idx;
  const int ncol = K + 1 + (softmax1 ? 1 : 0);
  const int ni = (ncol + 31) >> 5;                          // 32-column groups in use (1..3)
  for (uint32_t r0 = cta_row0 + warp * kBatch; r0 < cta_row1; r0 += kRowsPerCta * kBatch) {
    float x[kBatch][3];
    int id[kBatch][3];
    uint32_t hq_of[kBatch], b_of[kBatch];
    // all loads of the batch first, then the arithmetic
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const uint32_t r = min(r0 + j, rows - 1);
      const uint32_t bl = r / (uint32_t)h_q, hq = r - bl * (uint32_t)h_q;
      hq_of[j] = hq;
      b_of[j] = bl / (uint32_t)L;
      const int32_t* idx = indices + ((int64_t)bl * h_idx + hq / g) * K;
#pragma unroll
      for (int i = 0; i < 3; ++i) {
        x[j][i] = -CUDART_INF_F;
        id[j][i] = 0;
        if (i < ni) {
          const int c = lane + 32 * i;
          if (c < K) {
            x[j][i] = to_f(scores[(int64_t)r * K + c]);
            if (bias) id[j][i] = max(idx[c], 0);
          } else if (c == K) {
            x[j][i] = to_f(lse_swa[r]);
          } else if (c < ncol) {
            x[j][i] = 0.f;
          }
        }
      }
    }
    if (bias) {
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        const bool staged = bias_in_smem && b_of[j] == b0;      // a CTA may straddle two batches
#pragma unroll
        for (int i = 0; i < 3; ++i)
          if (i < ni && lane + 32 * i < K) {
            const float bv = staged ? bias_s[hq_of[j] * (N + 1) + id[j][i]]
                                    : bias[((int64_t)b_of[j] * N + id[j][i]) * h_q + hq_of[j]];
            x[j][i] = to_f(from_f<T>(x[j][i] + to_f(from_f<T>(bv))));
          }
      }
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      if (r0 + j >= cta_row1) break;                        // warp-uniform
      const float m = warp_max(fmaxf(fmaxf(x[j][0], x[j][1]), x[j][2]));
      float e[3], sum = 0.f;
#pragma unroll
      for (int i = 0; i < 3; ++i) {
        e[i] = (i < ni && lane + 32 * i < ncol && m > -CUDART_INF_F) ? __expf(x[j][i] - m) : 0.f;
        sum += e[i];
      }
      sum = warp_sum(sum);
      const float inv = 1.f / sum;                           // all -inf: 0/0 = NaN, as the reference's softmax
#pragma unroll
      for (int i = 0; i < 3; ++i) {
        const int c = lane + 32 * i;
        if (i < ni && c < ncol) weights[(int64_t)(r0 + j) * ncol + c] = from_f<T>(e[i] * inv);
      }
    }
  }
}

// Same computation for K <= 32, K % 4 == 0 (the common top-k sizes): eight lanes per row, four columns per
// lane with vector loads, so one warp instruction serves four rows; reductions take three shuffles.
template <typename T>
__global__ void __launch_bounds__(32 * kRowsPerCta)
chunk_weights_fwd8_kernel(const T* __restrict__ scores, const int32_t* __restrict__ indices,
                          const float* __restrict__ bias, const T* __restrict__ lse_swa, T* __restrict__ weights,
                          uint32_t rows, int L, int N, int h_q, int h_idx, int K, int softmax1, int bias_in_smem,
                          int rows_per_cta) {
  extern __shared__ float bias_s[];                         // [h_q][N + 1] when bias_in_smem
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane & 7, rq = lane >> 3;
  const uint32_t cta_row0 = blockIdx.x * (uint32_t)rows_per_cta;
  const uint32_t cta_row1 = min(rows, cta_row0 + (uint32_t)rows_per_cta);
  const uint32_t rows_per_batch = (uint32_t)L * (uint32_t)h_q;
  const uint32_t b0 = cta_row0 / rows_per_batch;
  if (bias && bias_in_smem) {
    const float* src = bias + (int64_t)b0 * N * h_q;
    for (int i = threadIdx.x; i < N * h_q; i += 32 * kRowsPerCta) {
      const int c = i / h_q, hq = i - c * h_q;
      bias_s[hq * (N + 1) + c] = src[i];
    }
    __syncthreads();
  }
  const int g = h_q / h_idx;
  const int ncol = K + 1 + (softmax1 ? 1 : 0);
  const bool has_cols = 4 * sub < K;
  for (uint32_t r0 = cta_row0 + warp * 8; r0 < cta_row1; r0 += kRowsPerCta * 8) {   // two row groups in flight
    float4 sc[2];
    int4 id[2];
    float ls[2];
    uint32_t hq_of[2], b_of[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const uint32_t r = min(r0 + 4 * j + rq, rows - 1);
      const uint32_t bl = r / (uint32_t)h_q, hq = r - bl * (uint32_t)h_q;
      hq_of[j] = hq;
      b_of[j] = bl / (uint32_t)L;
      sc[j] = make_float4(-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F);
      id[j] = make_int4(0, 0, 0, 0);
      if (has_cols) {
        sc[j] = load4(scores + (int64_t)r * K + 4 * sub);
        if (bias) id[j] = *reinterpret_cast<const int4*>(indices + ((int64_t)bl * h_idx + hq / g) * K + 4 * sub);
      }
      ls[j] = to_f(lse_swa[r]);
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const uint32_t r = r0 + 4 * j + rq;
      float x[4] = {sc[j].x, sc[j].y, sc[j].z, sc[j].w};
      if (bias && has_cols) {
        const int ids[4] = {max(id[j].x, 0), max(id[j].y, 0), max(id[j].z, 0), max(id[j].w, 0)};
        const bool staged = bias_in_smem && b_of[j] == b0;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float bv = staged ? bias_s[hq_of[j] * (N + 1) + ids[e]]
                                  : bias[((int64_t)b_of[j] * N + ids[e]) * h_q + hq_of[j]];
          x[e] = to_f(from_f<T>(x[e] + to_f(from_f<T>(bv))));
        }
      }
      float m = fmaxf(fmaxf(x[0], x[1]), fmaxf(x[2], x[3]));
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 4));
      m = fmaxf(m, ls[j]);
      if (softmax1) m = fmaxf(m, 0.f);
      float e4[4], sum = 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        e4[e] = (m > -CUDART_INF_F) ? __expf(x[e] - m) : 0.f;
        sum += e4[e];
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      sum += __shfl_xor_sync(0xffffffffu, sum, 4);
      const float e_l = (m > -CUDART_INF_F) ? __expf(ls[j] - m) : 0.f;
      const float e_z = (softmax1 && m > -CUDART_INF_F) ? __expf(-m) : 0.f;
      sum += e_l + e_z;
      const float inv = 1.f / sum;                           // all -inf: 0/0 = NaN, as the reference's softmax
      if (r < cta_row1) {
        T* wrow = weights + (int64_t)r * ncol;
        if (has_cols) {
#pragma unroll
          for (int e = 0; e < 4; ++e) wrow[4 * sub + e] = from_f<T>(e4[e] * inv);
        }
        if (sub == 0) {
          wrow[K] = from_f<T>(e_l * inv);
          if (softmax1) wrow[K + 1] = from_f<T>(e_z * inv);
        }
      }
    }
  }
}

// d_x = w * (d_w - sum(w * d_w)), rounded to T; columns [0,K) -> d_scores and (scattered) d_bias,
// column K -> d_lse.  A CTA owns kTokPerCta tokens of one (batch, query head): the bias gradient is
// accumulated per chunk id in shared memory and leaves the CTA as one atomic per touched chunk.
constexpr int kTokPerCta = 128;

template <typename T>
__global__ void __launch_bounds__(32 * kRowsPerCta)
chunk_weights_bwd_kernel(const T* __restrict__ weights, const T* __restrict__ d_weights,
                         const int32_t* __restrict__ indices, T* __restrict__ d_scores, T* __restrict__ d_lse,
                         float* __restrict__ d_bias, int L, int N, int h_q, int h_idx, int K, int softmax1,
                         int bias_in_smem) {
  extern __shared__ float acc_s[];                          // [N] when bias_in_smem
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int hq = blockIdx.y;
  const int64_t b = blockIdx.z;
  const int l0 = blockIdx.x * kTokPerCta, l1 = min(l0 + kTokPerCta, L);
  const int g = h_q / h_idx;
  const int ncol = K + 1 + (softmax1 ? 1 : 0);
  if (bias_in_smem) {
    for (int c = threadIdx.x; c < N; c += 32 * kRowsPerCta) acc_s[c] = 0.f;
    __syncthreads();
  }
  for (int lb = l0 + warp * kBatch; lb < l1; lb += kRowsPerCta * kBatch) {
    float w[kBatch][3], dw[kBatch][3];
    int id[kBatch][3];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {                     // all loads of the batch first
      const int l = min(lb + j, l1 - 1);
      const int64_t bl = b * L + l, r = bl * h_q + hq;
      const int32_t* idx = indices + (bl * h_idx + hq / g) * K;
#pragma unroll
      for (int i = 0; i < 3; ++i) {
        const int c = lane + 32 * i;
        w[j][i] = (c < ncol) ? to_f(weights[r * ncol + c]) : 0.f;
        dw[j][i] = (c < ncol) ? to_f(d_weights[r * ncol + c]) : 0.f;
        id[j][i] = (d_bias && c < K) ? idx[c] : -1;
      }
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      if (lb + j >= l1) break;                              // warp-uniform
      const int64_t r = (b * L + lb + j) * h_q + hq;
      float dot = fmaf(w[j][0], dw[j][0], fmaf(w[j][1], dw[j][1], w[j][2] * dw[j][2]));
      dot = warp_sum(dot);
#pragma unroll
      for (int i = 0; i < 3; ++i) {
        const int c = lane + 32 * i;
        if (c >= ncol) continue;
        const T dx = from_f<T>(w[j][i] * (dw[j][i] - dot));
        if (c < K) {
          d_scores[r * K + c] = dx;
          if (id[j][i] >= 0) {
            if (bias_in_smem) atomicAdd(acc_s + id[j][i], to_f(dx));
            else atomicAdd(d_bias + (b * N + id[j][i]) * h_q + hq, to_f(dx));
          }
        } else if (c == K) {
          d_lse[r] = dx;
        }
      }
    }
  }
  if (bias_in_smem) {
    __syncthreads();
    for (int c = threadIdx.x; c < N; c += 32 * kRowsPerCta) {
      const float x = acc_s[c];
      if (x != 0.f) atomicAdd(d_bias + (b * N + c) * h_q + hq, x);
    }
  }
}

// Backward for K <= 32, K % 4 == 0: eight lanes per row, four columns per lane (see the forward variant).
template <typename T>
__global__ void __launch_bounds__(32 * kRowsPerCta)
chunk_weights_bwd8_kernel(const T* __restrict__ weights, const T* __restrict__ d_weights,
                          const int32_t* __restrict__ indices, T* __restrict__ d_scores, T* __restrict__ d_lse,
                          float* __restrict__ d_bias, int L, int N, int h_q, int h_idx, int K, int softmax1,
                          int bias_in_smem) {
  extern __shared__ float acc_s[];                          // [N] when bias_in_smem
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane & 7, rq = lane >> 3;
  const int hq = blockIdx.y;
  const int64_t b = blockIdx.z;
  const int l0 = blockIdx.x * kTokPerCta, l1 = min(l0 + kTokPerCta, L);
  const int g = h_q / h_idx;
  const int ncol = K + 1 + (softmax1 ? 1 : 0);
  const bool has_cols = 4 * sub < K;
  if (bias_in_smem) {
    for (int c = threadIdx.x; c < N; c += 32 * kRowsPerCta) acc_s[c] = 0.f;
    __syncthreads();
  }
  for (int lb = l0 + warp * 8; lb < l1; lb += kRowsPerCta * 8) {       // two groups of four tokens in flight
    float w[2][4], dw[2][4], wx[2][2], dwx[2][2];
    int4 id[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {                            // all loads first
      const int l = min(lb + 4 * j + rq, l1 - 1);
      const int64_t bl = b * L + l, r = bl * h_q + hq;
      const T* wr = weights + r * ncol;
      const T* dr = d_weights + r * ncol;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        w[j][e] = has_cols ? to_f(wr[4 * sub + e]) : 0.f;
        dw[j][e] = has_cols ? to_f(dr[4 * sub + e]) : 0.f;
      }
      // the window column (and the zero column) are handled by the first lane of the group
      wx[j][0] = (sub == 0) ? to_f(wr[K]) : 0.f;
      dwx[j][0] = (sub == 0) ? to_f(dr[K]) : 0.f;
      wx[j][1] = (sub == 0 && softmax1) ? to_f(wr[K + 1]) : 0.f;
      dwx[j][1] = (sub == 0 && softmax1) ? to_f(dr[K + 1]) : 0.f;
      id[j] = make_int4(-1, -1, -1, -1);
      if (d_bias && has_cols) id[j] = *reinterpret_cast<const int4*>(indices + (bl * h_idx + hq / g) * K + 4 * sub);
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int l = lb + 4 * j + rq;
      float dot = fmaf(wx[j][0], dwx[j][0], wx[j][1] * dwx[j][1]);
#pragma unroll
      for (int e = 0; e < 4; ++e) dot = fmaf(w[j][e], dw[j][e], dot);
      dot += __shfl_xor_sync(0xffffffffu, dot, 1);
      dot += __shfl_xor_sync(0xffffffffu, dot, 2);
      dot += __shfl_xor_sync(0xffffffffu, dot, 4);
      if (l < l1) {
        const int64_t r = (b * L + l) * h_q + hq;
        if (has_cols) {
          const int ids[4] = {id[j].x, id[j].y, id[j].z, id[j].w};
          float dx[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            dx[e] = to_f(from_f<T>(w[j][e] * (dw[j][e] - dot)));
            if (ids[e] >= 0) {
              if (bias_in_smem) atomicAdd(acc_s + ids[e], dx[e]);
              else atomicAdd(d_bias + (b * N + ids[e]) * h_q + hq, dx[e]);
            }
          }
          store4(d_scores + r * K + 4 * sub, make_float4(dx[0], dx[1], dx[2], dx[3]));
        }
        if (sub == 0) d_lse[r] = from_f<T>(wx[j][0] * (dwx[j][0] - dot));
      }
    }
  }
  if (bias_in_smem) {
    __syncthreads();
    for (int c = threadIdx.x; c < N; c += 32 * kRowsPerCta) {
      const float x = acc_s[c];
      if (x != 0.f) atomicAdd(d_bias + (b * N + c) * h_q + hq, x);
    }
  }
}

// Both combine kernels give a row to a group of 2^lg lanes (4 elements per lane and step) and keep
// kBatch rows per group in flight.
// o = o_hils + o_swa * w[:, swa_col]
template <typename T>
__global__ void __launch_bounds__(256)
combine_fwd_kernel(const T* o_h, const T* __restrict__ o_swa, const T* __restrict__ weights,
                   T* o,   // o may alias o_h (in place)
                   uint32_t rows, int D, int ncol, int swa_col, int lg) {
  const uint32_t gid = blockIdx.x * 256u + threadIdx.x;
  const uint32_t r0 = (gid >> lg) * kBatch;
  const int d0 = (int)(gid & ((1u << lg) - 1u)) * 4, dstep = 4 << lg;
  if (r0 >= rows) return;
  for (int d = d0; d < D; d += dstep) {
    float4 a[kBatch], x[kBatch];
    float w[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const int64_t r = min(r0 + j, rows - 1);
      a[j] = load4(o_h + r * D + d);
      x[j] = load4(o_swa + r * D + d);
      w[j] = to_f(weights[r * ncol + swa_col]);
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j)
      if (r0 + j < rows)
        store4(o + (int64_t)(r0 + j) * D + d, make_float4(fmaf(x[j].x, w[j], a[j].x), fmaf(x[j].y, w[j], a[j].y),
                                                          fmaf(x[j].z, w[j], a[j].z), fmaf(x[j].w, w[j], a[j].w)));
  }
}

// d_o_swa = d_o * w_swa;  d_w[:, swa_col] = sum_d d_o * o_swa
template <typename T>
__global__ void __launch_bounds__(256)
combine_bwd_kernel(const T* __restrict__ d_o, const T* __restrict__ o_swa, const T* __restrict__ weights,
                   T* __restrict__ d_o_swa, T* __restrict__ d_weights, uint32_t rows, int D, int ncol, int swa_col,
                   int lg) {
  const uint32_t gid = blockIdx.x * 256u + threadIdx.x;
  const uint32_t r0 = (gid >> lg) * kBatch;
  const int d0 = (int)(gid & ((1u << lg) - 1u)) * 4, dstep = 4 << lg;
  float dot[kBatch];
#pragma unroll
  for (int j = 0; j < kBatch; ++j) dot[j] = 0.f;
  if (r0 < rows) {
    for (int d = d0; d < D; d += dstep) {
      float4 g[kBatch], x[kBatch];
      float w[kBatch];
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        const int64_t r = min(r0 + j, rows - 1);
        g[j] = load4(d_o + r * D + d);
        x[j] = load4(o_swa + r * D + d);
        w[j] = to_f(weights[r * ncol + swa_col]);
      }
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        dot[j] = fmaf(g[j].x, x[j].x, fmaf(g[j].y, x[j].y, fmaf(g[j].z, x[j].z, fmaf(g[j].w, x[j].w, dot[j]))));
        if (r0 + j < rows)
          store4(d_o_swa + (int64_t)(r0 + j) * D + d,
                 make_float4(g[j].x * w[j], g[j].y * w[j], g[j].z * w[j], g[j].w * w[j]));
      }
    }
  }
  // groups are aligned inside the warp: reduce over the 2^lg lanes of a group
#pragma unroll
  for (int j = 0; j < kBatch; ++j) {
    for (int o = 1; o < (1 << lg); o <<= 1) dot[j] += __shfl_xor_sync(0xffffffffu, dot[j], o);
    if (d0 == 0 && r0 + j < rows) d_weights[(int64_t)(r0 + j) * ncol + swa_col] = from_f<T>(dot[j]);
  }
}

}  // namespace hils

using namespace hils;

extern "C" int hils_chunk_weights_fwd(const void* scores, const int32_t* indices, const float* bias,
                                      const void* lse_swa, void* weights, int B, int L, int N, int h_q, int h_idx,
                                      int K, int softmax1, int dtype, void* stream) {
  HILS_REQUIRE(dtype == HILS_BF16 || dtype == HILS_F32, "chunk_weights_fwd: dtype must be bf16 or fp32");
  HILS_REQUIRE(K >= 1 && K + 2 <= kMaxCols, "chunk_weights_fwd: topk must be in [1, 94]");
  HILS_REQUIRE(h_idx >= 1 && h_q % h_idx == 0, "chunk_weights_fwd: h_q must be a multiple of the index heads");
  const int64_t rows = (int64_t)B * L * h_q;
  if (rows == 0) return HILS_OK;
  HILS_REQUIRE(scores && indices && lse_swa && weights, "chunk_weights_fwd: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  HILS_REQUIRE(rows < (int64_t)1 << 31, "chunk_weights_fwd: more than 2^31 rows");
  const size_t table = (size_t)h_q * (N + 1) * sizeof(float);
  const int in_smem = bias && table <= 96 * 1024 && rows >= 4 * (int64_t)kFwdRowsPerCta;
  const int rpc = in_smem ? kFwdRowsPerCta : kRowsPerCta * kBatch;
  const unsigned grid = (unsigned)((rows + rpc - 1) / rpc);
  const size_t smem = in_smem ? table : 0;
  if (K <= 32 && K % 4 == 0 && ((((uintptr_t)scores) | ((uintptr_t)indices)) & 15) == 0) {
    // eight lanes per row
    const int rpc8 = in_smem ? kFwdRowsPerCta : kRowsPerCta * 8;
    const unsigned grid8 = (unsigned)((rows + rpc8 - 1) / rpc8);
    if (dtype == HILS_BF16) {
      if (smem > 48 * 1024)
        cudaFuncSetAttribute(chunk_weights_fwd8_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      chunk_weights_fwd8_kernel<bf16><<<grid8, 32 * kRowsPerCta, smem, st>>>(
          (const bf16*)scores, indices, bias, (const bf16*)lse_swa, (bf16*)weights, (uint32_t)rows, L, N, h_q, h_idx, K,
          softmax1, in_smem, rpc8);
    } else {
      if (smem > 48 * 1024)
        cudaFuncSetAttribute(chunk_weights_fwd8_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      chunk_weights_fwd8_kernel<float><<<grid8, 32 * kRowsPerCta, smem, st>>>(
          (const float*)scores, indices, bias, (const float*)lse_swa, (float*)weights, (uint32_t)rows, L, N, h_q, h_idx, K,
          softmax1, in_smem, rpc8);
    }
    HILS_LAUNCH_CHECK("chunk_weights_fwd");
    return HILS_OK;
  }
  if (dtype == HILS_BF16) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(chunk_weights_fwd_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    chunk_weights_fwd_kernel<bf16><<<grid, 32 * kRowsPerCta, smem, st>>>(
        (const bf16*)scores, indices, bias, (const bf16*)lse_swa, (bf16*)weights, (uint32_t)rows, L, N, h_q, h_idx, K,
        softmax1, in_smem, rpc);
  } else {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(chunk_weights_fwd_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    chunk_weights_fwd_kernel<float><<<grid, 32 * kRowsPerCta, smem, st>>>(
        (const float*)scores, indices, bias, (const float*)lse_swa, (float*)weights, (uint32_t)rows, L, N, h_q, h_idx, K,
        softmax1, in_smem, rpc);
  }
  HILS_LAUNCH_CHECK("chunk_weights_fwd");
  return HILS_OK;
}

extern "C" int hils_chunk_weights_bwd(const void* weights, const void* d_weights, const int32_t* indices,
                                      void* d_scores, void* d_lse, float* d_bias, int B, int L, int N, int h_q,
                                      int h_idx, int K, int softmax1, int dtype, void* stream) {
  HILS_REQUIRE(dtype == HILS_BF16 || dtype == HILS_F32, "chunk_weights_bwd: dtype must be bf16 or fp32");
  HILS_REQUIRE(K >= 1 && K + 2 <= kMaxCols, "chunk_weights_bwd: topk must be in [1, 94]");
  HILS_REQUIRE(h_idx >= 1 && h_q % h_idx == 0, "chunk_weights_bwd: h_q must be a multiple of the index heads");
  const int64_t rows = (int64_t)B * L * h_q;
  cudaStream_t st = (cudaStream_t)stream;
  if (d_bias) {
    const cudaError_t e = cudaMemsetAsync(d_bias, 0, sizeof(float) * (size_t)B * N * h_q, st);
    if (e != cudaSuccess) return cuda_fail(e, "chunk_weights_bwd (memset)");
  }
  if (rows == 0) return HILS_OK;
  HILS_REQUIRE(weights && d_weights && indices && d_scores && d_lse, "chunk_weights_bwd: null pointer");
  HILS_REQUIRE(h_q <= 65535 && B <= 65535, "chunk_weights_bwd: more than 65535 heads or sequences");
  const int in_smem = d_bias && (size_t)N * 4 <= 96 * 1024;
  const size_t smem = in_smem ? (size_t)N * 4 : 0;
  dim3 grid((L + kTokPerCta - 1) / kTokPerCta, h_q, B);
  if (K <= 32 && K % 4 == 0 && ((((uintptr_t)d_scores) | ((uintptr_t)indices)) & 15) == 0) {
    if (dtype == HILS_BF16) {
      if (smem > 48 * 1024)
        cudaFuncSetAttribute(chunk_weights_bwd8_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      chunk_weights_bwd8_kernel<bf16><<<grid, 32 * kRowsPerCta, smem, st>>>(
          (const bf16*)weights, (const bf16*)d_weights, indices, (bf16*)d_scores, (bf16*)d_lse, d_bias, L, N, h_q, h_idx,
          K, softmax1, in_smem);
    } else {
      if (smem > 48 * 1024)
        cudaFuncSetAttribute(chunk_weights_bwd8_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      chunk_weights_bwd8_kernel<float><<<grid, 32 * kRowsPerCta, smem, st>>>(
          (const float*)weights, (const float*)d_weights, indices, (float*)d_scores, (float*)d_lse, d_bias, L, N, h_q,
          h_idx, K, softmax1, in_smem);
    }
    HILS_LAUNCH_CHECK("chunk_weights_bwd");
    return HILS_OK;
  }
  if (dtype == HILS_BF16) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(chunk_weights_bwd_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    chunk_weights_bwd_kernel<bf16><<<grid, 32 * kRowsPerCta, smem, st>>>(
        (const bf16*)weights, (const bf16*)d_weights, indices, (bf16*)d_scores, (bf16*)d_lse, d_bias, L, N, h_q, h_idx,
        K, softmax1, in_smem);
  } else {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(chunk_weights_bwd_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    chunk_weights_bwd_kernel<float><<<grid, 32 * kRowsPerCta, smem, st>>>(
        (const float*)weights, (const float*)d_weights, indices, (float*)d_scores, (float*)d_lse, d_bias, L, N, h_q,
        h_idx, K, softmax1, in_smem);
  }
  HILS_LAUNCH_CHECK("chunk_weights_bwd");
  return HILS_OK;
}

static int lanes_log2(int D) {            // lanes per row: the smallest power of two >= D/4, at most 32
  int lg = 0;
  while ((4 << lg) < D && lg < 5) ++lg;
  return lg;
}

extern "C" int hils_combine_fwd(const void* o_hils, const void* o_swa, const void* weights, void* o, int B, int L,
                                int h_q, int D, int num_weights, int swa_col, int dtype, void* stream) {
  HILS_REQUIRE(dtype == HILS_BF16 || dtype == HILS_F32, "combine_fwd: dtype must be bf16 or fp32");
  HILS_REQUIRE(D % 4 == 0, "combine_fwd: D must be a multiple of 4");
  HILS_REQUIRE(swa_col >= 0 && swa_col < num_weights, "combine_fwd: swa_col out of range");
  const int64_t rows = (int64_t)B * L * h_q;
  if (rows == 0) return HILS_OK;
  HILS_REQUIRE(rows < (int64_t)1 << 31, "combine_fwd: more than 2^31 rows");
  HILS_REQUIRE(o_hils && o_swa && weights && o, "combine_fwd: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  const int lg = lanes_log2(D);
  const int64_t threads = ((rows + kBatch - 1) / kBatch) << lg;
  const unsigned grid = (unsigned)((threads + 255) / 256);
  if (dtype == HILS_BF16)
    combine_fwd_kernel<bf16><<<grid, 256, 0, st>>>((const bf16*)o_hils, (const bf16*)o_swa, (const bf16*)weights,
                                                   (bf16*)o, (uint32_t)rows, D, num_weights, swa_col, lg);
  else
    combine_fwd_kernel<float><<<grid, 256, 0, st>>>((const float*)o_hils, (const float*)o_swa, (const float*)weights,
                                                    (float*)o, (uint32_t)rows, D, num_weights, swa_col, lg);
  HILS_LAUNCH_CHECK("combine_fwd");
  return HILS_OK;
}

extern "C" int hils_combine_bwd(const void* d_o, const void* o_swa, const void* weights, void* d_o_swa,
                                void* d_weights, int B, int L, int h_q, int D, int num_weights, int swa_col,
                                int dtype, void* stream) {
  HILS_REQUIRE(dtype == HILS_BF16 || dtype == HILS_F32, "combine_bwd: dtype must be bf16 or fp32");
  HILS_REQUIRE(D % 4 == 0, "combine_bwd: D must be a multiple of 4");
  HILS_REQUIRE(swa_col >= 0 && swa_col < num_weights, "combine_bwd: swa_col out of range");
  const int64_t rows = (int64_t)B * L * h_q;
  if (rows == 0) return HILS_OK;
  HILS_REQUIRE(rows < (int64_t)1 << 31, "combine_bwd: more than 2^31 rows");
  HILS_REQUIRE(d_o && o_swa && weights && d_o_swa && d_weights, "combine_bwd: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  const int lg = lanes_log2(D);
  const int64_t threads = ((rows + kBatch - 1) / kBatch) << lg;
  const unsigned grid = (unsigned)((threads + 255) / 256);
  if (dtype == HILS_BF16)
    combine_bwd_kernel<bf16><<<grid, 256, 0, st>>>((const bf16*)d_o, (const bf16*)o_swa, (const bf16*)weights,
                                                   (bf16*)d_o_swa, (bf16*)d_weights, (uint32_t)rows, D, num_weights,
                                                   swa_col, lg);
  else
    combine_bwd_kernel<float><<<grid, 256, 0, st>>>((const float*)d_o, (const float*)o_swa, (const float*)weights,
                                                    (float*)d_o_swa, (float*)d_weights, (uint32_t)rows, D, num_weights,
                                                    swa_col, lg);
  HILS_LAUNCH_CHECK("combine_bwd");
  return HILS_OK;
}
