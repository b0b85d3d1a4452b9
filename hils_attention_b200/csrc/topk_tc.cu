// Chunk selection for LONG candidate lists on the 5th-generation tensor cores (tcgen05 + TMEM + TMA), bf16,
// one query head per key head (G = 1).  Same contract as topk.cu (ops/topk_head_softmax.py:15-154, kernels :192-971):
//   v[c]   = fl32(fl32(<q, k'_c>) * scale) + bias[c];  lse_total = logaddexp(lse_swa, logsumexp_c v[c])
//   key[c] = v[c] - lse_total;  the K largest keys win, ties go to the smaller chunk id, ids ascending, -1 padded
//
// With a thousand and more candidates per token the warp-per-token selector of topk.cu spends thousands of
// instructions per token and re-streams the chunk keys for every 16 tokens.  Here one CTA owns 128 consecutive
// tokens of one (batch, head) and ONE THREAD owns one token: the scores of a tile of 128 chunk keys are a single
// 128 x 128 tcgen05 product whose accumulator row a thread reads straight from its TMEM lane, so every step of the
// selection is 128 tokens wide and free of cross-lane traffic.  The scores are never stored: the key tiles are
// streamed twice (they are small and L2-resident) and the product is recomputed, which costs the tensor pipe next
// to nothing:
//   pass 0  log-sum-exp of the row (running maximum and sum per 32 columns) AND the row's 32 largest values v, exactly.
//           key = v - lse_total is a non-decreasing function of v, so the K-th largest key and the number of keys
//           strictly above it follow from the 32 largest v once lse_total is known.  A value enters the list only if
//           it beats the current K-th value: such values (a share of K/n of the stream after n candidates) are
//           appended to a 16-entry buffer per token in shared memory, and only when some token's buffer would
//           overflow does the warp sort the buffered values in registers (bitonic network) and merge them into the
//           running sorted lists (max(list[i], sorted[31-i]) is the top half of the union, one half-cleaner stage
//           sorts it); the 32 columns that caused the overflow go through the same network.  Sorting every 32
//           columns unconditionally, as an earlier version did, cost three times the instructions: some lane of a
//           warp has a qualifying value in almost every group, so a data-dependent skip never fires;
//   pass 1  candidates are scanned in id order; those whose key is above the K-th key, and the first ones equal to
//           it, are written out with their raw scores: ids come out ascending without a sort.
// All mbarrier waits are bounded; on expiry the kernel records a status word, every role leaves its loop, TMEM is
// released and the CTA returns.
#include "common.cuh"
#include "topk_params.cuh"
#include "umma.cuh"

namespace hils {

using namespace umma;

static __device__ int g_sel_status = 0;

__device__ __forceinline__ bool sel_wait(uint64_t* b, uint32_t parity) {
  const uint32_t addr = smem_u32(b);
  for (int it = 0; it < (1 << 20); ++it) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.b32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(addr), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ void sel_fail(int code) { atomicCAS(&g_sel_status, 0, code); }

__device__ __forceinline__ int sel_row_limit(const TopkParams& p, int l) {
  if (l >= p.L) return 0;
  if (!p.is_causal) return p.N;
  const int t = p.q_offset + l;
  const int lim = (p.window_size > 0) ? floor_div(t - p.window_size + 1, p.block_size) : floor_div(t, p.block_size);
  return max(0, min(lim, p.N));
}
__device__ __forceinline__ float sel_log_add_exp(float a, float b) {
  if (isinf(a) && a == b) return a;
  const float mx = fmaxf(a, b), mn = fminf(a, b);
  return mx + log1pf(expf(mn - mx));
}

constexpr int kSelTcThreads = 192;   // row warpgroup + MMA warp + TMA warp
constexpr float kSelLog2e = 1.4426950408889634f;

// descending bitonic sort of 32 registers (240 compare-exchanges, all indices static)
__device__ __forceinline__ void sel_sort32_desc(float (&x)[32]) {
#pragma unroll
  for (int k = 2; k <= 32; k <<= 1)
#pragma unroll
    for (int j = k >> 1; j > 0; j >>= 1)
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const int l = i ^ j;
        if (l > i) {
          const bool desc = (i & k) == 0;
          const float a = x[i], c = x[l];
          x[i] = desc ? fmaxf(a, c) : fminf(a, c);
          x[l] = desc ? fminf(a, c) : fmaxf(a, c);
        }
      }
}
// top[] (sorted descending) <- the 32 largest of top[] and c[] (sorted descending)
__device__ __forceinline__ void sel_merge_top32(float (&top)[32], const float (&c)[32]) {
#pragma unroll
  for (int i = 0; i < 32; ++i) top[i] = fmaxf(top[i], c[31 - i]);   // the top half of the union, a bitonic sequence
#pragma unroll
  for (int j = 16; j > 0; j >>= 1)
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const int l = i ^ j;
      if (l > i) {
        const float a = top[i], d = top[l];
        top[i] = fmaxf(a, d);
        top[l] = fminf(a, d);
      }
    }
}

// descending bitonic sort of 16 registers (80 compare-exchanges)
__device__ __forceinline__ void sel_sort16_desc(float (&x)[16]) {
#pragma unroll
  for (int k = 2; k <= 16; k <<= 1)
#pragma unroll
    for (int j = k >> 1; j > 0; j >>= 1)
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int l = i ^ j;
        if (l > i) {
          const bool desc = (i & k) == 0;
          const float a = x[i], c = x[l];
          x[i] = desc ? fmaxf(a, c) : fminf(a, c);
          x[l] = desc ? fminf(a, c) : fmaxf(a, c);
        }
      }
}
// top[] (sorted descending) <- the 32 largest of top[] and the 16 values c[] (sorted descending)
__device__ __forceinline__ void sel_merge_top32_16(float (&top)[32], const float (&c)[16]) {
#pragma unroll
  for (int i = 16; i < 32; ++i) top[i] = fmaxf(top[i], c[31 - i]);
#pragma unroll
  for (int j = 16; j > 0; j >>= 1)
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const int l = i ^ j;
      if (l > i) {
        const float a = top[i], d = top[l];
        top[i] = fmaxf(a, d);
        top[l] = fminf(a, d);
      }
    }
}
// the K-th entry of a descending list (K is not a compile-time constant: a select chain, no local memory)
__device__ __forceinline__ float sel_kth(const float (&top)[32], int K) {
  float kth = top[0];
#pragma unroll
  for (int j = 1; j < 32; ++j) kth = (j == K - 1) ? top[j] : kth;
  return kth;
}

constexpr int kSelCap = 16;   // buffered qualifying values per token between two merges
constexpr int kSelDirectTiles = 4;   // tiles at the head of a row's stream that are sorted unconditionally (measured best)

// the first n buffered values of this token (entry j at cand[j * 128]) -> its sorted list
__device__ __forceinline__ void sel_flush(float (&top)[32], const float* cand, int n) {
  float c16[16];
#pragma unroll
  for (int j = 0; j < kSelCap; ++j) c16[j] = (j < n) ? cand[j * 128] : -CUDART_INF_F;
  sel_sort16_desc(c16);
  sel_merge_top32_16(top, c16);
}

template <int D>
__global__ void __launch_bounds__(kSelTcThreads, 2) topk_fwd_tc_kernel(TopkParams p, const __grid_constant__ CUtensorMap tmQ,
                                                                      const __grid_constant__ CUtensorMap tmK) {
  constexpr int DB = D / 64;
  constexpr int TBYTES = DB * 16384;     // a [128 x D] bf16 tile (queries or chunk keys)
  constexpr int NST = (D == 64) ? 3 : 2; // key tile ring
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* Qs = smem;
  uint8_t* Ks = Qs + TBYTES;             // NST stages

  __shared__ uint64_t q_full, kv_full[3], kv_free[3], s_full[2], s_free[2], bias_full[2];
  __shared__ float bias_s[2][128];
  __shared__ float cand_s[kSelCap * 128];   // [entry][token]: conflict-free for a warp's 32 tokens
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int blk = gridDim.x - 1 - blockIdx.x;            // the last token blocks see the most chunks: they start first
  const int l0 = blk * 128, h = blockIdx.y, b = blockIdx.z;
  const int K = p.topk;
  const int cta_limit = sel_row_limit(p, min(l0 + 127, p.L - 1));   // limits do not decrease with the position
  const int ntile = (cta_limit + 127) >> 7;
  const int nitem = 2 * ntile;

  if (ntile == 0 || *reinterpret_cast<volatile int*>(&g_sel_status) != 0) {
    // no candidates for any token of the block: empty lists, lse_total = lse of the window branch
    if (tid < 128 && l0 + tid < p.L && ntile == 0) {
      const int64_t row = ((int64_t)b * p.L + l0 + tid) * p.h_kv + h;
      for (int k = 0; k < K; ++k) {
        p.indices[row * K + k] = -1;
        static_cast<bf16*>(p.scores)[row * K + k] = __float2bfloat16_rn(-CUDART_INF_F);
      }
      if (p.lse_total)
        p.lse_total[row] = (p.lse_dtype == HILS_BF16) ? to_f(static_cast<const bf16*>(p.lse_swa)[row])
                                                      : static_cast<const float*>(p.lse_swa)[row];
      if (p.rank_keys)
        for (int c = 0; c < p.N; ++c) p.rank_keys[row * p.N + c] = -CUDART_INF_F;
    }
    return;
  }

  if (tid == 0) {
    mbar_init(&q_full, 1);
    for (int s = 0; s < NST; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_free[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_free[s], 128);
      mbar_init(&bias_full[s], 1);
    }
    mbar_init_fence();
    abort_s = 0;
  }
  if (warp == 4) tmem_alloc(&tmem_base_s, 256);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  const bool has_bias = p.bias != nullptr;

  if (warp == 5) {
    // =============================== TMA producer (+ bias tiles) =================================
    bool ok = true;
    if (lane == 0) {
      mbar_expect_tx(&q_full, TBYTES);
#pragma unroll
      for (int db = 0; db < DB; ++db) tma_load_2d(Qs + db * 16384, &tmQ, &q_full, h * D + db * 64, b * p.L + l0);
    }
    for (int i = 0; i < nitem; ++i) {
      const int st = i % NST, t = i % ntile, sb = i & 1;
      if (__any_sync(0xffffffffu, abort_s != 0)) { ok = false; break; }
      if (lane == 0) {
        if (i >= NST) ok = sel_wait(&kv_free[st], ((i / NST) - 1) & 1);
        if (ok) {
          mbar_expect_tx(&kv_full[st], TBYTES);
#pragma unroll
          for (int db = 0; db < DB; ++db)
            tma_load_2d(Ks + st * TBYTES + db * 16384, &tmK, &kv_full[st], h * D + db * 64, b * p.N + t * 128);
        }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) { if (lane == 0) sel_fail(6010000 + i); break; }
      if (has_bias) {
        // the bias of the tile's 128 chunks -> slot of the item's S buffer, once the rows have left that slot
        if (i >= 2) {
          ok = __all_sync(0xffffffffu, sel_wait(&s_free[sb], ((i >> 1) - 1) & 1));
          if (!ok) { if (lane == 0) sel_fail(6011000 + i); break; }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int c = t * 128 + j * 32 + lane;
          bias_s[sb][j * 32 + lane] = c < p.N ? __ldg(p.bias + ((int64_t)b * p.N + c) * p.h_kv + h) : 0.f;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&bias_full[sb]);
      }
    }
    if (!ok && lane == 0) abort_s = 1;
  } else if (warp == 4) {
    // =============================== MMA issuer ==================================================
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_bf16(128, 128, 0);
      const DescWords q_d = desc_words_sw128(smem_u32(Qs), 16, 1024), k_d = desc_words_sw128(smem_u32(Ks), 16, 1024);
      bool ok = sel_wait(&q_full, 0);
      for (int i = 0; ok && i < nitem; ++i) {
        const int st = i % NST, sb = i & 1;
        if (abort_s) { ok = false; break; }
        ok = sel_wait(&kv_full[st], (i / NST) & 1);
        if (ok && i >= 2) ok = sel_wait(&s_free[sb], ((i >> 1) - 1) & 1);
        if (!ok) { sel_fail(6020000 + i); break; }
        tc_fence_after();
        const uint32_t kb = k_d.lo + st * (TBYTES >> 4);
        mma_ss_w<false>(tmem + sb * 128, q_d.lo, q_d.hi, kb, k_d.hi, idesc);
#pragma unroll
        for (int kk = 1; kk < D / 16; ++kk)
          mma_ss_w<true>(tmem + sb * 128, q_d.lo + (((kk >> 2) * 16384 + (kk & 3) * 32) >> 4), q_d.hi,
                         kb + (((kk >> 2) * 16384 + (kk & 3) * 32) >> 4), k_d.hi, idesc);
        mma_commit(&s_full[sb]);
        mma_commit(&kv_free[st]);
      }
      if (!ok) abort_s = 1;
    }
  } else {
    // =============================== rows: one thread per token =================================
    const int r = tid, l = l0 + r;
    const int lim = sel_row_limit(p, l);                   // 0 for rows past the end of the sequence
    const int64_t row = ((int64_t)b * p.L + (l < p.L ? l : 0)) * p.h_kv + h;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    float lse_w = 0.f;
    if (l < p.L)
      lse_w = (p.lse_dtype == HILS_BF16) ? to_f(static_cast<const bf16*>(p.lse_swa)[row])
                                         : static_cast<const float*>(p.lse_swa)[row];
    float m_run = -CUDART_INF_F, s_run = 0.f;               // pass 0: running maximum and sum
    float top[32];                                          // pass 0: the 32 largest values so far, descending
#pragma unroll
    for (int j = 0; j < 32; ++j) top[j] = -CUDART_INF_F;
    float thrv = -CUDART_INF_F;                             // the K-th largest value so far
    int cnt = 0;                                            // buffered values of this token
    float* cand = cand_s + r;
    float lt = 0.f, thr = -CUDART_INF_F, cut = -CUDART_INF_F;
    int take = 0, eq_seen = 0, n_out = 0;
    int32_t* out_ids = p.indices + row * K;
    bf16* out_sc = static_cast<bf16*>(p.scores) + row * K;
    float* rk = (p.rank_keys && l < p.L) ? p.rank_keys + row * p.N : nullptr;
    bool ok = true;
    for (int i = 0; i < nitem; ++i) {
      const int pass = i / ntile, t = i - pass * ntile, sb = i & 1;
      ok = sel_wait(&s_full[sb], (i >> 1) & 1);
      if (ok && has_bias) ok = sel_wait(&bias_full[sb], (i >> 1) & 1);
      if (!ok) sel_fail(6030000 + i);
      ok = __all_sync(0xffffffffu, ok) && !abort_s;
      if (!ok) break;
      tc_fence_after();
      if (t == 0 && pass == 1) {
        // between the passes: lse_total, the lists of values become lists of keys, the K-th key and the ties to take
        sel_flush(top, cand, cnt);
        const float lh = (s_run > 0.f) ? m_run + logf(s_run) : -CUDART_INF_F;
        lt = sel_log_add_exp(lse_w, lh);
        if (p.lse_total && l < p.L) p.lse_total[row] = lt;
#pragma unroll
        for (int j = 0; j < 32; ++j) top[j] = top[j] - lt;   // -inf stays -inf
        thr = sel_kth(top, K);                               // -inf with fewer than K candidates (all win)
        int gt = 0;
#pragma unroll
        for (int j = 0; j < 32; ++j) gt += (j < K && top[j] > thr) ? 1 : 0;
        take = (thr > -CUDART_INF_F) ? K - gt : 0;
        // u >= cut is necessary for key >= thr: the margin is far above the few ulps of lse_total and of the K-th key
        // that the roundings of fl(fl(s scale) + bias) - lse_total can move a key by
        cut = (thr + lt) - 1e-5f * (fabsf(lt) + fabsf(thr) + 1.f);
      }
#pragma unroll 1
      for (int cb = 0; cb < 4; ++cb) {
        float sv[32];
        __syncwarp();
        tmem_ld32(tmem + lane_base + sb * 128 + cb * 32, sv);
        tmem_ld_wait();
        const int c0 = t * 128 + cb * 32;
        if (pass == 0) {
          if (c0 < lim) {
            float cm[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
            if (c0 + 32 <= lim) {                      // the whole group lies inside the row's range: no column test
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                float v = __fmul_rn(sv[j], p.scale);
                if (has_bias) v += bias_s[sb][cb * 32 + j];
                sv[j] = v;
                cm[j & 3] = fmaxf(cm[j & 3], v);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                float v = __fmul_rn(sv[j], p.scale);
                if (has_bias) v += bias_s[sb][cb * 32 + j];
                v = (c0 + j < lim) ? v : -CUDART_INF_F;
                sv[j] = v;
                cm[j & 3] = fmaxf(cm[j & 3], v);
              }
            }
            const float m_new = fmaxf(m_run, fmaxf(fmaxf(cm[0], cm[1]), fmaxf(cm[2], cm[3])));
            const float nb = -m_new * kSelLog2e;
            float ad[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int j = 0; j < 32; ++j) ad[j & 3] += ex2(fmaf(sv[j], kSelLog2e, nb));
            s_run = s_run * ex2(fmaf(m_run, kSelLog2e, nb)) + ((ad[0] + ad[1]) + (ad[2] + ad[3]));   // ex2(-inf) = 0 at first
            m_run = m_new;
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) sv[j] = -CUDART_INF_F;   // nothing of this row here (the tile serves other rows)
          }
          // The first tiles of a row's stream go through the sorting network directly (most values still qualify);
          // later, values that beat the K-th value so far wait in the buffer.
          const bool direct = t < kSelDirectTiles;
          const int cnt0 = cnt;
          if (!direct) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const bool q = sv[j] > thrv;
              if (q && cnt < kSelCap) cand[cnt * 128] = sv[j];
              cnt += q ? 1 : 0;
            }
          }
          if (direct || __any_sync(0xffffffffu, cnt > kSelCap)) {
            // some token's buffer cannot take this group: merge what was buffered before it, then the group itself
            if (!direct) {
              sel_flush(top, cand, cnt0);
              cnt = 0;
            }
            sel_sort32_desc(sv);
            sel_merge_top32(top, sv);
            thrv = sel_kth(top, K);
          }
        } else {
          // Emit pass.  Only ~K of a row's candidates are selected, so the exact key (two roundings and a subtraction)
          // is formed for the few that a one-instruction bound lets through: u = fma(s, scale, bias) against
          // cut = K-th key + lse_total minus a margin that covers every rounding between u and the key.  Those few are
          // buffered (score, column) and handled after the group.  Groups with columns beyond a row's limit, rows that
          // take every candidate (fewer than K) and diagnostic runs take the exact path for all 32 columns.
          bool fast = !rk && thr > -CUDART_INF_F && c0 + 32 <= lim;
          fast = __all_sync(0xffffffffu, fast);
          int nb = 0;
          if (fast) {
            // The buffer keeps the layout of the first pass - thread r owns the floats r + 128 e - because the row warps
            // of a CTA can be one tile apart: a warp that is already emitting must not touch the slots in which a
            // slower warp still holds first-pass values.  Entry n = (score at e = 2 n, column at e = 2 n + 1).
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float u = has_bias ? fmaf(sv[j], p.scale, bias_s[sb][cb * 32 + j]) : sv[j] * p.scale;
              const bool q = u >= cut;
              if (q && nb < kSelCap / 2) {
                cand[(2 * nb) * 128] = sv[j];
                cand[(2 * nb + 1) * 128] = __int_as_float(cb * 32 + j);
              }
              nb += q ? 1 : 0;
            }
            fast = !__any_sync(0xffffffffu, nb > kSelCap / 2);         // a buffer overflowed: the exact path redoes the group
            if (fast) {
              for (int e = 0; e < nb; ++e) {
                const int col = __float_as_int(cand[(2 * e + 1) * 128]) & 127;
                const float raw = __fmul_rn(cand[(2 * e) * 128], p.scale);
                float v = raw;
                if (has_bias) v += bias_s[sb][col];
                const float key = v - lt;
                const bool is_eq = key == thr;
                const bool sel = key > thr || (is_eq && eq_seen < take);
                eq_seen += is_eq ? 1 : 0;
                if (sel && n_out < K) {
                  out_ids[n_out] = t * 128 + col;
                  out_sc[n_out] = __float2bfloat16_rn(raw);
                  ++n_out;
                }
              }
            }
          }
          if (!fast) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float raw = __fmul_rn(sv[j], p.scale);
              float v = raw;
              if (has_bias) v += bias_s[sb][cb * 32 + j];
              const bool valid = c0 + j < lim;
              const float key = valid ? v - lt : -CUDART_INF_F;
              if (rk && c0 + j < p.N) rk[c0 + j] = key;
              const bool is_eq = valid && key == thr && thr > -CUDART_INF_F;
              const bool sel = valid && key > -CUDART_INF_F && (key > thr || (is_eq && eq_seen < take));
              eq_seen += is_eq ? 1 : 0;
              if (sel && n_out < K) {
                out_ids[n_out] = c0 + j;
                out_sc[n_out] = __float2bfloat16_rn(raw);
                ++n_out;
              }
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&s_free[sb]);
    }
    if (ok && l < p.L) {
      for (int k = n_out; k < K; ++k) {
        out_ids[k] = -1;
        out_sc[k] = __float2bfloat16_rn(-CUDART_INF_F);
      }
      if (rk)                                              // keys of the chunks beyond the block's last tile
        for (int c = ntile * 128; c < p.N; ++c) rk[c] = -CUDART_INF_F;
    }
    if (!ok && lane == 0) { abort_s = 1; sel_fail(6039999); }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem, 256);
}

// Returns HILS_ERR_UNSUPPORTED (without setting an error text) when the call is outside this path.
int topk_fwd_tc_launch(const TopkParams& p, cudaStream_t st) {
  const int D = p.D;
  if (p.G != 1 || (D != 64 && D != 128) || p.topk > 32 || p.drop_mask || p.gumbel || p.N < 512 || p.L <= 4) return HILS_ERR_UNSUPPORTED;
  if (((uintptr_t)p.q | (uintptr_t)p.lmks) & 15) return HILS_ERR_UNSUPPORTED;
  if ((int64_t)p.B * p.L >= (1ll << 31) || (int64_t)p.B * p.N >= (1ll << 31)) return HILS_ERR_UNSUPPORTED;
  CUtensorMap tmQ, tmK;
  if (int rc = make_tmap_bf16_rows(&tmQ, p.q, (uint64_t)p.B * p.L, (uint64_t)p.h_kv * D, (uint64_t)p.h_kv * D, 128)) return rc;
  if (int rc = make_tmap_bf16_rows(&tmK, p.lmks, (uint64_t)p.B * p.N, (uint64_t)p.h_kv * D, (uint64_t)p.h_kv * D, 128)) return rc;
  const int NST = (D == 64) ? 3 : 2;
  const size_t smem = 1024 + (size_t)(1 + NST) * (D / 64) * 16384;
  dim3 grid((p.L + 127) / 128, p.h_kv, p.B);
  if (D == 64) {
    cudaFuncSetAttribute(topk_fwd_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    topk_fwd_tc_kernel<64><<<grid, kSelTcThreads, smem, st>>>(p, tmQ, tmK);
  } else {
    cudaFuncSetAttribute(topk_fwd_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    topk_fwd_tc_kernel<128><<<grid, kSelTcThreads, smem, st>>>(p, tmQ, tmK);
  }
  HILS_LAUNCH_CHECK("topk_fwd (one thread per token, tcgen05 scores)");
  return HILS_OK;
}

// device-side error word of this file's kernel (0 = none); synchronises and clears
int take_status_topk_tc() {
  int v = 0, zero = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  if (cudaMemcpyFromSymbol(&v, g_sel_status, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(g_sel_status, &zero, sizeof(int));
  return v;
}

}  // namespace hils
