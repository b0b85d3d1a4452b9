// Sliding-window branch on the tensor cores (tcgen05 + TMEM + TMA), bf16, head dims 64 and 128.
//
// Forward: one CTA owns 128 rows (128/G query tokens x G heads of one kv head) and the 64-key tiles
// its window touches.  It walks the tiles twice:
//   sweep 1: S = Q K^T, each row only tracks its masked maximum;
//   sweep 2: S again, P = exp2(scale*S - max) with the mask applied, O += P V in TMEM, row sums.
// Knowing the maximum before the second sweep removes the rescaling of O that a one-sweep online
// softmax needs; the window is short (<= ~12 tiles) so the extra Q K^T is cheap.
// Backward: the same two atomic-free passes as the sparse attention: a query-major pass for dQ
// (dQ accumulates in TMEM over the block's tiles) and a key-major pass for dK/dV (one CTA per
// 64-key tile walks the query blocks that see it; M = 64 accumulators in TMEM).
//   P = exp2(scale*S - lse), dS = P (dP - Delta) scale, Delta = <o, dO> - dlse
// (ops/flex_attn_tilelang.py:124-133 tile range, :155-216 masks, :685-702 Delta, :374-588 backward).
#include "tc_rows.cuh"
#include "umma.cuh"

namespace hils {

static __device__ int g_device_status = 0;

using namespace umma;

struct SwaTcParams {
  const bf16* q; const bf16* k; const bf16* v; bf16* o; float* lse; const bf16* d_o; const float* d_lse;
  bf16* d_q; bf16* d_k; bf16* d_v; float* delta;
  int B, Lq, Lk, h_q, h_kv, W, S, mask_lmk, expand, kv_start;
  float scale;
};

constexpr int kThreads = 192;
constexpr float kLn2 = 0.6931471805599453f;

// raw key range [lo, hi] visible from query row i (empty when lo > hi)
__device__ __forceinline__ void row_range(const SwaTcParams& p, int i, int& lo, int& hi) {
  const int t = p.kv_start + (p.Lk - p.Lq) + i;
  int start = t - p.W + 1;
  if (p.expand) start = floor_div(start, p.S) * p.S;
  lo = max(0, start - p.kv_start);
  hi = min(p.Lk - 1, t - p.kv_start);
}
// bit jj set when key column j0 + jj is a landmark column ((absolute position + 1) % S == 0)
__device__ __forceinline__ unsigned long long lmk_bits(const SwaTcParams& p, int j0) {
  if (!p.mask_lmk) return 0ull;
  unsigned long long m = 0ull;
  const int rem = (p.kv_start + j0 + 1) % p.S;
  for (int pos = (p.S - rem) % p.S; pos < 64; pos += p.S) m |= 1ull << pos;
  return m;
}

// ================================================================================================
template <int D>
__global__ void __launch_bounds__(kThreads, (D == 64) ? 3 : 2) swa_fwd_tc_kernel(SwaTcParams p, const __grid_constant__ CUtensorMap tmK,
                                                              const __grid_constant__ CUtensorMap tmV) {
  constexpr int DB = D / 64;
  constexpr int QBYTES = DB * 16384;
  constexpr int KVBYTES = DB * 8192;
  // A block's window is ~10 key tiles swept twice, so CTA prologue, pipeline fill and epilogue weigh as much
  // as the loop: at D = 64 three CTAs share an SM (one S accumulator, one P tile, 128 TMEM columns and
  // 65 KB of shared memory each) and hide them for one another; at D = 128 two do (256 TMEM columns each).  Two CTAs of
  // D = 128 have 115,712 bytes each and the tiles alone take 114,688: the barriers live behind the tiles in the dynamic
  // region, which starts on a 1 KB boundary because nothing static precedes it, so no alignment gap is lost.
  constexpr int NSB = 1;
  // (No alignment attribute: it would apply to the dynamic region of every kernel of this file and cost the backward
  // kernels, which budget their shared memory to the byte, their second CTA.  With nothing static in front, the region
  // starts at the CTA's shared-memory window, which is 1 KB aligned; the kernel verifies it.)
  extern __shared__ uint8_t swa_fwd_smem[];
  uint8_t* Qs = swa_fwd_smem;
  uint8_t* Ks = Qs + QBYTES;
  uint8_t* Vs = Ks + 2 * KVBYTES;
  uint8_t* Ps = Vs + 2 * KVBYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(Ps + NSB * 16384);
  uint64_t* kv_full = bars;          // [2]
  uint64_t* s_full = bars + 2;       // [2]
  uint64_t* p_full = bars + 4;       // [2]
  uint64_t* pv_done = bars + 6;      // [2]
  uint32_t& tmem_base_s = *reinterpret_cast<uint32_t*>(bars + 8);
  volatile int& abort_s = *reinterpret_cast<volatile int*>(reinterpret_cast<uint32_t*>(bars + 8) + 1);
  if ((reinterpret_cast<uintptr_t>(swa_fwd_smem) & 1023) != 0) {   // the tiles need the 1 KB alignment of their swizzle
    if (threadIdx.x == 0) atomicExch(&g_device_status, 405);
    return;
  }

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = p.h_q / p.h_kv, QB = 128 / G;
  const int blk = gridDim.x - 1 - blockIdx.x;
  const int q0 = blk * QB, h = blockIdx.y, b = blockIdx.z;

  if (tid == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 128);
      mbar_init(&pv_done[s], 1);
    }
    mbar_init_fence();
    abort_s = 0;
  }
  if (warp == 4) tmem_alloc(&tmem_base_s, D == 64 ? 128 : 256);

  const int r = tid, ql = r / G, g = r % G, i = q0 + ql;
  const bool is_row = tid < 128;
  const bool valid = is_row && i < p.Lq;
  const int hq = h * G + g;
  const int64_t rowi = ((int64_t)b * p.Lq + (valid ? i : 0)) * p.h_q + hq;
  if (is_row) load_row_to_tile<D>(Qs, r, p.q + rowi * D, valid);
  // tiles touched by the block: first row's lower edge .. last valid row's upper edge
  int blo, bhi, tmp;
  row_range(p, q0, blo, tmp);
  row_range(p, min(q0 + QB, p.Lq) - 1, tmp, bhi);
  const int jt0 = blo >> 6;
  const int nt = (bhi >= blo) ? (bhi >> 6) - jt0 + 1 : 0;
  const int n = 2 * nt;
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  const uint32_t tS = tmem, tO = tmem + NSB * 64;

  if (warp == 5) {
    if (lane == 0) {
      for (int it = 0; it < n; ++it) {
        const int s = it & 1, u = it >> 1;
        if (abort_s) break;
        if (it >= 2 && !mbar_wait(&pv_done[s], (u - 1) & 1)) { abort_s = 1; atomicExch(&g_device_status, 401); break; }
        const bool second = it >= nt;
        const int jt = jt0 + (second ? it - nt : it);
        mbar_expect_tx(&kv_full[s], second ? 2 * KVBYTES : KVBYTES);
#pragma unroll
        for (int db = 0; db < DB; ++db) {
          tma_load_2d(Ks + s * KVBYTES + db * 8192, &tmK, &kv_full[s], h * D + db * 64, b * p.Lk + jt * 64);
          if (second) tma_load_2d(Vs + s * KVBYTES + db * 8192, &tmV, &kv_full[s], h * D + db * 64, b * p.Lk + jt * 64);
        }
      }
    }
  } else if (warp == 4) {
    if (lane == 0 && n > 0) {
      constexpr uint32_t idesc_qk = idesc_bf16(128, 64, 0);
      constexpr uint32_t idesc_pv = idesc_bf16(128, D, 1);
      // descriptor words built once; inside the loops an operand is addressed by adding to the low word
      const DescWords q_d = desc_words_sw128(smem_u32(Qs), 16, 1024), k_d = desc_words_sw128(smem_u32(Ks), 16, 1024),
                      p_d = desc_words_sw128(smem_u32(Ps), 16, 1024), v_d = desc_words_sw128(smem_u32(Vs), 8192, 1024);
      auto issue_qk = [&](int it) {
        const int s = it & 1;
        const uint32_t kb = k_d.lo + s * (KVBYTES >> 4);
        const uint32_t ts = tS + (NSB == 2 ? s : 0) * 64;
        mma_ss_w<false>(ts, q_d.lo, q_d.hi, kb, k_d.hi, idesc_qk);
#pragma unroll
        for (int kk = 1; kk < D / 16; ++kk)
          mma_ss_w<true>(ts, q_d.lo + (((kk >> 2) * 16384 + (kk & 3) * 32) >> 4), q_d.hi,
                         kb + (((kk >> 2) * 8192 + (kk & 3) * 32) >> 4), k_d.hi, idesc_qk);
        mma_commit(&s_full[s]);
      };
      bool ok = mbar_wait(&kv_full[0], 0);
      if (ok) { tc_fence_after(); issue_qk(0); }
      for (int it = 0; ok && it < n; ++it) {
        const int s = it & 1, u = it >> 1;
        if (abort_s) break;
        if (NSB == 2 && it + 1 < n) {
          ok = mbar_wait(&kv_full[(it + 1) & 1], ((it + 1) >> 1) & 1);
          if (!ok) break;
          tc_fence_after();
          issue_qk(it + 1);
        }
        ok = mbar_wait(&p_full[s], u & 1);
        if (!ok) break;
        tc_fence_after();
        if (it >= nt) {
          const uint32_t a0 = p_d.lo + (NSB == 2 ? s : 0) * (16384 >> 4), b0 = v_d.lo + s * (KVBYTES >> 4);
          mma_ss_wr(tO, a0, p_d.hi, b0, v_d.hi, idesc_pv, it > nt ? 1u : 0u);
#pragma unroll
          for (int kk = 1; kk < 4; ++kk)
            mma_ss_w<true>(tO, a0 + ((kk * 32) >> 4), p_d.hi, b0 + ((kk * 2048) >> 4), v_d.hi, idesc_pv);
        }
        mma_commit(&pv_done[s]);
        if (NSB == 1 && it + 1 < n) {   // S was consumed before the arrival on p_full waited for above
          ok = mbar_wait(&kv_full[(it + 1) & 1], ((it + 1) >> 1) & 1);
          if (!ok) break;
          tc_fence_after();
          issue_qk(it + 1);
        }
      }
      if (!ok) { abort_s = 1; atomicExch(&g_device_status, 402); }
    }
  } else {
    const float sl2 = p.scale * kLog2e;
    int lo = 1, hi = 0;
    if (valid) row_range(p, i, lo, hi);
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    float m = -CUDART_INF_F, l = 0.f;
    bool ok = true;
    for (int it = 0; it < n; ++it) {
      const int s = it & 1, u = it >> 1;
      const bool second = it >= nt;
      const int j0 = (jt0 + (second ? it - nt : it)) * 64;
      ok = mbar_wait(&s_full[s], u & 1);
      if (it >= 2) ok = mbar_wait(&pv_done[s], (u - 1) & 1) && ok;
      ok = __all_sync(0xffffffffu, ok) && !abort_s;
      if (!ok) break;
      tc_fence_after();
      float sv[64];
      tmem_ld32(tS + lane_base + (NSB == 2 ? s : 0) * 64, sv);
      tmem_ld32(tS + lane_base + (NSB == 2 ? s : 0) * 64 + 32, sv + 32);
      tmem_ld_wait();
      const int a = lo - j0, e = hi - j0;
      const unsigned long long lm = lmk_bits(p, j0);
      if (!second) {
#pragma unroll
        for (int jj = 0; jj < 64; ++jj)
          if (jj >= a && jj <= e && !((lm >> jj) & 1ull)) m = fmaxf(m, sv[jj]);
      } else {
        const float mb = (m > -CUDART_INF_F) ? m * sl2 : 0.f;
        float part = 0.f;
#pragma unroll
        for (int jj = 0; jj < 64; ++jj) {
          const bool vis = jj >= a && jj <= e && !((lm >> jj) & 1ull);
          sv[jj] = vis ? ex2(fmaf(sv[jj], sl2, -mb)) : 0.f;
          part += sv[jj];
        }
        l += part;
        store_row_bf16_sw128(Ps + (NSB == 2 ? s : 0) * 16384, r, sv);
      }
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(&p_full[s]);
    }
    if (ok && n > 0) {
      ok = mbar_wait(&pv_done[(n - 1) & 1], ((n - 1) >> 1) & 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok && lane == 0) { abort_s = 1; atomicExch(&g_device_status, 403); }
    } else if (!ok && lane == 0) {
      abort_s = 1;
      atomicExch(&g_device_status, 404);
    }
    const float inv = (l > 0.f) ? 1.f / l : 0.f;
    if (ok) tc_fence_after();
#pragma unroll
    for (int cb = 0; cb < D / 32; ++cb) {
      float ov[32];
      if (ok && n > 0) {
        tmem_ld32(tO + lane_base + cb * 32, ov);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) ov[j] *= inv;
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) ov[j] = 0.f;
      }
      if (valid) store32_bf16(p.o + rowi * D + cb * 32, ov);
    }
    if (valid) p.lse[rowi] = (l > 0.f) ? m * p.scale + __logf(l) : -CUDART_INF_F;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem, D == 64 ? 128 : 256);
}

// Backward row arithmetic in two phases, so that the dP row can still be in flight from TMEM while the
// first phase works on the S row.  Phase A: sv <- P = exp2(scale*S - lse), masked.
__device__ __forceinline__ void swa_bwd_row_p(float* sv, float sl2, float lse_l2, int a, int e, unsigned long long lm) {
#pragma unroll
  for (int jj = 0; jj < 64; ++jj) {
    const bool vis = jj >= a && jj <= e && !((lm >> jj) & 1ull);
    sv[jj] = vis ? ex2(fmaf(sv[jj], sl2, -lse_l2)) : 0.f;
  }
}
// Phase B: sv <- dS = scale * P * (dP - delta), dp <- P
__device__ __forceinline__ void swa_bwd_row_ds(float* sv, float* dp, float delta, float scale) {
  const float nds = -delta * scale;
#pragma unroll
  for (int jj = 0; jj < 64; ++jj) {
    const float pj = sv[jj];
    sv[jj] = pj * fmaf(dp[jj], scale, nds);
    dp[jj] = pj;
  }
}

// ================================================================================================
template <int D>
__global__ void __launch_bounds__(kThreads, (D == 64) ? 2 : 1) swa_bwd_dq_tc_kernel(SwaTcParams p, const __grid_constant__ CUtensorMap tmK,
                                                                    const __grid_constant__ CUtensorMap tmV) {
  constexpr int DB = D / 64;
  constexpr int QBYTES = DB * 16384;
  constexpr int KVBYTES = DB * 8192;
  // A block's window is only ~10 key tiles, so a CTA's prologue, pipeline fill and epilogue weigh as much
  // as its loop.  At D = 64 two CTAs share an SM and hide them for each other: one S/dP accumulator per
  // CTA (256 TMEM columns), products issued after the previous tile's dS.  D = 128 needs the whole shared
  // memory for one CTA and double-buffers the accumulator instead.
  constexpr int NSB = (D == 64) ? 1 : 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* Qs = smem;
  uint8_t* dOs = Qs + QBYTES;
  uint8_t* Ks = dOs + QBYTES;
  uint8_t* Vs = Ks + 2 * KVBYTES;
  uint8_t* dSs = Vs + 2 * KVBYTES;

  __shared__ uint64_t kv_full[2], sdp_full[2], ds_full[2], dq_done[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = p.h_q / p.h_kv, QB = 128 / G;
  const int blk = gridDim.x - 1 - blockIdx.x;
  const int q0 = blk * QB, h = blockIdx.y, b = blockIdx.z;

  if (tid == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&sdp_full[s], 1);
      mbar_init(&ds_full[s], 128);
      mbar_init(&dq_done[s], 1);
    }
    mbar_init_fence();
    abort_s = 0;
  }
  if (warp == 4) tmem_alloc(&tmem_base_s, NSB == 1 ? 256 : 512);

  const int r = tid, ql = r / G, g = r % G, i = q0 + ql;
  const bool is_row = tid < 128;
  const bool valid = is_row && i < p.Lq;
  const int hq = h * G + g;
  const int64_t rowi = ((int64_t)b * p.Lq + (valid ? i : 0)) * p.h_q + hq;
  float delta = 0.f, lse_l2 = 0.f;
  bool live = false;
  if (is_row) {
    load_row_to_tile<D>(Qs, r, p.q + rowi * D, valid);
    load_row_to_tile<D>(dOs, r, p.d_o + rowi * D, valid);
    if (valid) {
      const bf16* orow = p.o + rowi * D;
      const bf16* dorow = p.d_o + rowi * D;
      float acc = 0.f;
#pragma unroll
      for (int d = 0; d < D; d += 4) {
        float4 x = load4(orow + d), y = load4(dorow + d);
        acc += x.x * y.x + x.y * y.y + x.z * y.z + x.w * y.w;
      }
      delta = acc - (p.d_lse ? p.d_lse[rowi] : 0.f);
      const float lse = p.lse[rowi];
      live = lse > -CUDART_INF_F;
      lse_l2 = live ? lse * kLog2e : 0.f;
      p.delta[rowi] = delta;
    }
  }
  int blo, bhi, tmp;
  row_range(p, q0, blo, tmp);
  row_range(p, min(q0 + QB, p.Lq) - 1, tmp, bhi);
  const int jt0 = blo >> 6;
  const int n = (bhi >= blo) ? (bhi >> 6) - jt0 + 1 : 0;
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  const uint32_t tdQ = tmem + NSB * 128;

  if (warp == 5) {
    if (lane == 0) {
      for (int it = 0; it < n; ++it) {
        const int s = it & 1, u = it >> 1;
        if (abort_s) break;
        if (it >= 2 && !mbar_wait(&dq_done[s], (u - 1) & 1)) { abort_s = 1; atomicExch(&g_device_status, 411); break; }
        mbar_expect_tx(&kv_full[s], 2 * KVBYTES);
#pragma unroll
        for (int db = 0; db < DB; ++db) {
          tma_load_2d(Ks + s * KVBYTES + db * 8192, &tmK, &kv_full[s], h * D + db * 64, b * p.Lk + (jt0 + it) * 64);
          tma_load_2d(Vs + s * KVBYTES + db * 8192, &tmV, &kv_full[s], h * D + db * 64, b * p.Lk + (jt0 + it) * 64);
        }
      }
    }
  } else if (warp == 4) {
    if (lane == 0 && n > 0) {
      constexpr uint32_t idesc_s = idesc_bf16(128, 64, 0);
      constexpr uint32_t idesc_dq = idesc_bf16(128, D, 1);
      // descriptor words built once; inside the loops an operand is addressed by adding to the low word
      const DescWords q_d = desc_words_sw128(smem_u32(Qs), 16, 1024), do_d = desc_words_sw128(smem_u32(dOs), 16, 1024),
                      k_d = desc_words_sw128(smem_u32(Ks), 16, 1024), v_d = desc_words_sw128(smem_u32(Vs), 16, 1024),
                      ds_d = desc_words_sw128(smem_u32(dSs), 16, 1024), kmn_d = desc_words_sw128(smem_u32(Ks), 8192, 1024);
      auto issue_sdp = [&](int it) {
        const int s = it & 1;
        const uint32_t kb = k_d.lo + s * (KVBYTES >> 4), vb = v_d.lo + s * (KVBYTES >> 4);
        const uint32_t ts = tmem + (NSB == 2 ? s : 0) * 128;
        mma_ss_w<false>(ts, q_d.lo, q_d.hi, kb, k_d.hi, idesc_s);
#pragma unroll
        for (int kk = 1; kk < D / 16; ++kk)
          mma_ss_w<true>(ts, q_d.lo + (((kk >> 2) * 16384 + (kk & 3) * 32) >> 4), q_d.hi,
                         kb + (((kk >> 2) * 8192 + (kk & 3) * 32) >> 4), k_d.hi, idesc_s);
        mma_ss_w<false>(ts + 64, do_d.lo, do_d.hi, vb, v_d.hi, idesc_s);
#pragma unroll
        for (int kk = 1; kk < D / 16; ++kk)
          mma_ss_w<true>(ts + 64, do_d.lo + (((kk >> 2) * 16384 + (kk & 3) * 32) >> 4), do_d.hi,
                         vb + (((kk >> 2) * 8192 + (kk & 3) * 32) >> 4), v_d.hi, idesc_s);
        mma_commit(&sdp_full[NSB == 2 ? s : 0]);
      };
      bool ok = mbar_wait(&kv_full[0], 0);
      if (ok) { tc_fence_after(); issue_sdp(0); }
      for (int it = 0; ok && it < n; ++it) {
        const int s = it & 1, u = it >> 1;
        if (abort_s) break;
        if (NSB == 2 && it + 1 < n) {
          ok = mbar_wait(&kv_full[(it + 1) & 1], ((it + 1) >> 1) & 1);
          if (!ok) break;
          tc_fence_after();
          issue_sdp(it + 1);
        }
        ok = mbar_wait(&ds_full[s], u & 1);
        if (!ok) break;
        tc_fence_after();
        {
          const uint32_t a0 = ds_d.lo + s * (16384 >> 4), b0 = kmn_d.lo + s * (KVBYTES >> 4);
          mma_ss_wr(tdQ, a0, ds_d.hi, b0, kmn_d.hi, idesc_dq, it > 0 ? 1u : 0u);
#pragma unroll
          for (int kk = 1; kk < 4; ++kk)
            mma_ss_w<true>(tdQ, a0 + ((kk * 32) >> 4), ds_d.hi, b0 + ((kk * 2048) >> 4), kmn_d.hi, idesc_dq);
        }
        mma_commit(&dq_done[s]);
        if (NSB == 1 && it + 1 < n) {   // the single accumulator was consumed before the dS arrival above
          ok = mbar_wait(&kv_full[(it + 1) & 1], ((it + 1) >> 1) & 1);
          if (!ok) break;
          tc_fence_after();
          issue_sdp(it + 1);
        }
      }
      if (!ok) { abort_s = 1; atomicExch(&g_device_status, 412); }
    }
  } else {
    const float sl2 = p.scale * kLog2e;
    int lo = 1, hi = 0;
    if (valid && live) row_range(p, i, lo, hi);
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    bool ok = true;
    for (int it = 0; it < n; ++it) {
      const int s = it & 1, u = it >> 1;
      const int j0 = (jt0 + it) * 64;
      ok = (NSB == 2) ? mbar_wait(&sdp_full[s], u & 1) : mbar_wait(&sdp_full[0], it & 1);
      if (it >= 2) ok = mbar_wait(&dq_done[s], (u - 1) & 1) && ok;
      ok = __all_sync(0xffffffffu, ok) && !abort_s;
      if (!ok) break;
      tc_fence_after();
      float sv[64], dp[64];
      const uint32_t tsd = tmem + lane_base + (NSB == 2 ? s : 0) * 128;
      tmem_ld32(tsd, sv);
      tmem_ld32(tsd + 32, sv + 32);
      tmem_ld_wait();
      tmem_ld32(tsd + 64, dp);        // in flight while P is formed
      tmem_ld32(tsd + 96, dp + 32);
      swa_bwd_row_p(sv, sl2, lse_l2, lo - j0, hi - j0, lmk_bits(p, j0));
      tmem_ld_wait64(dp);
      swa_bwd_row_ds(sv, dp, delta, p.scale);
      store_row_bf16_sw128(dSs + s * 16384, r, sv);
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(&ds_full[s]);
    }
    if (ok && n > 0) {
      ok = mbar_wait(&dq_done[(n - 1) & 1], ((n - 1) >> 1) & 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok && lane == 0) { abort_s = 1; atomicExch(&g_device_status, 413); }
    } else if (!ok && lane == 0) {
      abort_s = 1;
      atomicExch(&g_device_status, 414);
    }
    if (ok) tc_fence_after();
#pragma unroll
    for (int cb = 0; cb < D / 32; ++cb) {
      float ov[32];
      if (ok && n > 0) {
        tmem_ld32(tdQ + lane_base + cb * 32, ov);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) ov[j] = 0.f;
      }
      if (valid) store32_bf16(p.d_q + rowi * D + cb * 32, ov);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem, NSB == 1 ? 256 : 512);
}

// ================================================================================================
// key-major pass (training layout: Lq == Lk, kv_start == 0, so query i sits at position i)
template <int D>
__global__ void __launch_bounds__(kThreads, (D == 64) ? 2 : 1) swa_bwd_dkv_tc_kernel(SwaTcParams p, const __grid_constant__ CUtensorMap tmK,
                                                                     const __grid_constant__ CUtensorMap tmV,
                                                                     const __grid_constant__ CUtensorMap tmQ,
                                                                     const __grid_constant__ CUtensorMap tmdO) {
  constexpr int DB = D / 64;
  constexpr int QBYTES = DB * 16384;
  constexpr int KVBYTES = DB * 8192;
  // Only ~6 query blocks see a key tile, so at D = 64 two CTAs share an SM (see the query-major pass): one
  // S/dP accumulator (256 TMEM columns) and one dS / P buffer per CTA.
  constexpr int NDS = 1;
  constexpr int NSB = (D == 64) ? 1 : 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* Qs = smem;
  uint8_t* dOs = Qs + 2 * QBYTES;
  uint8_t* Ks = dOs + 2 * QBYTES;
  uint8_t* Vs = Ks + KVBYTES;
  uint8_t* dSs = Vs + KVBYTES;
  uint8_t* Pws = dSs + NDS * 16384;
  {
    // the launch sizes the dynamic region for the static variables in front of it (see the host side):
    // refuse to run rather than write past it if the layout is ever different
    uint32_t dyn_bytes;
    asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_bytes));
    if ((size_t)(Pws + NDS * 16384 - smem_raw) > dyn_bytes) {
      if (threadIdx.x == 0) atomicExch(&g_device_status, 425);
      return;
    }
  }

  __shared__ uint64_t kv_full, qdo_full[2], sdp_full[2], dsp_full[2], dkv_done[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int jt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int G = p.h_q / p.h_kv, QB = 128 / G;
  const int L = p.Lq;

  if (tid == 0) {
    mbar_init(&kv_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&qdo_full[s], 1);
      mbar_init(&sdp_full[s], 1);
      mbar_init(&dsp_full[s], 128);
      mbar_init(&dkv_done[s], 1);
    }
    mbar_init_fence();
    abort_s = 0;
  }
  if (warp == 4) tmem_alloc(&tmem_base_s, NSB == 1 ? 256 : 512);
  // queries that can see a key of this tile: i in [j_first, i_hi(j_last)]
  const int j_first = jt * 64, j_last = min(j_first + 63, L - 1);
  int i_hi = p.expand ? (j_last / p.S + 1) * p.S + p.W - 2 : j_last + p.W - 1;
  i_hi = min(i_hi, L - 1);
  const int blk0 = j_first / QB;
  const int m = (i_hi >= j_first) ? i_hi / QB - blk0 + 1 : 0;
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  const uint32_t tdK = tmem + NSB * 128, tdV = tmem + NSB * 128 + D;

  if (warp == 5) {
    if (lane == 0 && m > 0) {
      mbar_expect_tx(&kv_full, 2 * KVBYTES);
#pragma unroll
      for (int db = 0; db < DB; ++db) {
        tma_load_2d(Ks + db * 8192, &tmK, &kv_full, h * D + db * 64, b * L + jt * 64);
        tma_load_2d(Vs + db * 8192, &tmV, &kv_full, h * D + db * 64, b * L + jt * 64);
      }
      for (int j = 0; j < m; ++j) {
        const int s = j & 1, u = j >> 1;
        if (abort_s) break;
        if (j >= 2 && !mbar_wait(&dkv_done[s], (u - 1) & 1)) { abort_s = 1; atomicExch(&g_device_status, 421); break; }
        mbar_expect_tx(&qdo_full[s], 2 * QBYTES);
#pragma unroll
        for (int db = 0; db < DB; ++db) {
          tma_load_3d(Qs + s * QBYTES + db * 16384, &tmQ, &qdo_full[s], db * 64, h * G, b * L + (blk0 + j) * QB);
          tma_load_3d(dOs + s * QBYTES + db * 16384, &tmdO, &qdo_full[s], db * 64, h * G, b * L + (blk0 + j) * QB);
        }
      }
    }
  } else if (warp == 4) {
    if (lane == 0 && m > 0) {
      constexpr uint32_t idesc_s = idesc_bf16(128, 64, 0);
      constexpr uint32_t idesc_dkv = idesc_bf16(64, D, 1, 1);
      // D = 64: dK and dV of a block come from one product of M = 128, N = 128: A = [dS^T ; P^T] (64-row
      // blocks of an MN-major operand, one tile apart), B = [Q | dO] (64-column blocks two stages apart);
      // dK is the block (rows 0..63, columns 0..63) of the accumulator, dV the block (rows 64..127,
      // columns 64..127).  Half the MMA instructions for the same operand bytes.
      constexpr bool kStacked = (D == 64);
      constexpr uint32_t idesc_st = idesc_bf16(128, 128, 1, 1);
      const DescWords ast_d = desc_words_sw128(smem_u32(dSs), NDS * 16384, 1024),
                      bst_d = desc_words_sw128(smem_u32(Qs), 2 * QBYTES, 1024);
      // descriptor words built once; the Q / dO tiles are read K-major for S and dP and MN-major for dK and dV
      const DescWords q_d = desc_words_sw128(smem_u32(Qs), 16, 1024), do_d = desc_words_sw128(smem_u32(dOs), 16, 1024),
                      k_d = desc_words_sw128(smem_u32(Ks), 16, 1024), v_d = desc_words_sw128(smem_u32(Vs), 16, 1024),
                      qmn_d = desc_words_sw128(smem_u32(Qs), 16384, 1024), domn_d = desc_words_sw128(smem_u32(dOs), 16384, 1024),
                      ds_d = desc_words_sw128(smem_u32(dSs), 16384, 1024), pw_d = desc_words_sw128(smem_u32(Pws), 16384, 1024);
      auto issue_sdp = [&](int j) {
        const int s = j & 1;
        const uint32_t qb = q_d.lo + s * (QBYTES >> 4), dob = do_d.lo + s * (QBYTES >> 4);
        const uint32_t ts = tmem + (NSB == 2 ? s : 0) * 128;
        mma_ss_w<false>(ts, qb, q_d.hi, k_d.lo, k_d.hi, idesc_s);
#pragma unroll
        for (int kk = 1; kk < D / 16; ++kk)
          mma_ss_w<true>(ts, qb + (((kk >> 2) * 16384 + (kk & 3) * 32) >> 4), q_d.hi,
                         k_d.lo + (((kk >> 2) * 8192 + (kk & 3) * 32) >> 4), k_d.hi, idesc_s);
        mma_ss_w<false>(ts + 64, dob, do_d.hi, v_d.lo, v_d.hi, idesc_s);
#pragma unroll
        for (int kk = 1; kk < D / 16; ++kk)
          mma_ss_w<true>(ts + 64, dob + (((kk >> 2) * 16384 + (kk & 3) * 32) >> 4), do_d.hi,
                         v_d.lo + (((kk >> 2) * 8192 + (kk & 3) * 32) >> 4), v_d.hi, idesc_s);
        mma_commit(&sdp_full[NSB == 2 ? s : 0]);
      };
      bool ok = mbar_wait(&kv_full, 0) && mbar_wait(&qdo_full[0], 0);
      if (ok) { tc_fence_after(); issue_sdp(0); }
      for (int j = 0; ok && j < m; ++j) {
        const int s = j & 1, u = j >> 1, sb = j % NDS;
        if (abort_s) break;
        if (NSB == 2 && j + 1 < m) {
          ok = mbar_wait(&qdo_full[(j + 1) & 1], ((j + 1) >> 1) & 1);
          if (!ok) break;
          tc_fence_after();
          issue_sdp(j + 1);
        }
        ok = mbar_wait(&dsp_full[s], u & 1);
        if (!ok) break;
        tc_fence_after();
        {
          const uint32_t dsb = ds_d.lo + sb * (16384 >> 4), pwb = pw_d.lo + sb * (16384 >> 4);
          const uint32_t qb = qmn_d.lo + s * (QBYTES >> 4), dob = domn_d.lo + s * (QBYTES >> 4);
          if (kStacked) {
            const uint32_t a0 = ast_d.lo + sb * (16384 >> 4), b0 = bst_d.lo + s * (QBYTES >> 4);
            mma_ss_wr(tdK, a0, ast_d.hi, b0, bst_d.hi, idesc_st, j > 0 ? 1u : 0u);
#pragma unroll
            for (int kk = 1; kk < 8; ++kk)
              mma_ss_w<true>(tdK, a0 + ((kk * 2048) >> 4), ast_d.hi, b0 + ((kk * 2048) >> 4), bst_d.hi, idesc_st);
          } else {
            mma_ss_wr(tdK, dsb, ds_d.hi, qb, qmn_d.hi, idesc_dkv, j > 0 ? 1u : 0u);
            mma_ss_wr(tdV, pwb, pw_d.hi, dob, domn_d.hi, idesc_dkv, j > 0 ? 1u : 0u);
#pragma unroll
            for (int kk = 1; kk < 8; ++kk) {
              mma_ss_w<true>(tdK, dsb + ((kk * 2048) >> 4), ds_d.hi, qb + ((kk * 2048) >> 4), qmn_d.hi, idesc_dkv);
              mma_ss_w<true>(tdV, pwb + ((kk * 2048) >> 4), pw_d.hi, dob + ((kk * 2048) >> 4), domn_d.hi, idesc_dkv);
            }
          }
        }
        mma_commit(&dkv_done[s]);
        if (NSB == 1 && j + 1 < m) {   // the single accumulator was consumed before the dS arrival above
          ok = mbar_wait(&qdo_full[(j + 1) & 1], ((j + 1) >> 1) & 1);
          if (!ok) break;
          tc_fence_after();
          issue_sdp(j + 1);
        }
      }
      if (!ok) { abort_s = 1; atomicExch(&g_device_status, 422); }
    }
  } else {
    const int r = tid, ql = r / G, g = r % G, hq = h * G + g;
    const float sl2 = p.scale * kLog2e;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    const unsigned long long lm = lmk_bits(p, j_first);
    bool ok = true;
    for (int j = 0; j < m; ++j) {
      const int s = j & 1, u = j >> 1, sb = j % NDS;
      const int i = (blk0 + j) * QB + ql;
      int lo = 1, hi = 0;
      float delta = 0.f, lse_l2 = 0.f;
      if (i < L) {
        const int64_t rowi = ((int64_t)b * L + i) * p.h_q + hq;
        const float lse = p.lse[rowi];
        if (lse > -CUDART_INF_F) {
          row_range(p, i, lo, hi);
          lse_l2 = lse * kLog2e;
          delta = p.delta[rowi];
        }
      }
      ok = (NSB == 2) ? mbar_wait(&sdp_full[s], u & 1) : mbar_wait(&sdp_full[0], j & 1);
      if (j >= NDS) ok = mbar_wait(&dkv_done[(j - NDS) & 1], ((j - NDS) >> 1) & 1) && ok;
      ok = __all_sync(0xffffffffu, ok) && !abort_s;
      if (!ok) break;
      tc_fence_after();
      float sv[64], dp[64];
      const uint32_t tsd = tmem + lane_base + (NSB == 2 ? s : 0) * 128;
      tmem_ld32(tsd, sv);
      tmem_ld32(tsd + 32, sv + 32);
      tmem_ld_wait();
      tmem_ld32(tsd + 64, dp);        // in flight while P is formed
      tmem_ld32(tsd + 96, dp + 32);
      swa_bwd_row_p(sv, sl2, lse_l2, lo - j_first, hi - j_first, lm);
      tmem_ld_wait64(dp);
      swa_bwd_row_ds(sv, dp, delta, p.scale);
      store_row_bf16_sw128(dSs + sb * 16384, r, sv);
      store_row_bf16_sw128(Pws + sb * 16384, r, dp);
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(&dsp_full[s]);
    }
    if (ok && m > 0) {
      ok = mbar_wait(&dkv_done[(m - 1) & 1], ((m - 1) >> 1) & 1);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok && lane == 0) { abort_s = 1; atomicExch(&g_device_status, 423); }
    } else if (!ok && lane == 0) {
      abort_s = 1;
      atomicExch(&g_device_status, 424);
    }
    const int krow = 16 * warp + lane;           // M = 64 accumulator: lanes 0..15 of each warp hold rows
    const int tokj = j_first + krow;
    const int64_t tok = (int64_t)b * L + tokj;
    if (ok) tc_fence_after();
    if (D == 64) {
      // stacked accumulator (M = 128): TMEM lane = row; warps 0, 1 hold the dK rows (columns 0..63), warps
      // 2, 3 the dV rows (columns 64..127)
      const bool is_v = warp >= 2;
      const int tokr = j_first + 32 * (warp & 1) + lane;
#pragma unroll
      for (int cb = 0; cb < 2; ++cb) {
        float ov[32];
        if (ok && m > 0) {
          tmem_ld32(tdK + lane_base + (is_v ? 64 : 0) + cb * 32, ov);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int jj = 0; jj < 32; ++jj) ov[jj] = 0.f;
        }
        if (tokr < L) store32_bf16((is_v ? p.d_v : p.d_k) + (((int64_t)b * L + tokr) * p.h_kv + h) * D + cb * 32, ov);
      }
    } else
#pragma unroll
    for (int which = 0; which < 2; ++which) {
#pragma unroll
      for (int cb = 0; cb < D / 32; ++cb) {
        float ov[32];
        if (ok && m > 0) {
          tmem_ld32((which ? tdV : tdK) + lane_base + cb * 32, ov);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int jj = 0; jj < 32; ++jj) ov[jj] = 0.f;
        }
        if (lane < 16 && tokj < L) store32_bf16((which ? p.d_v : p.d_k) + (tok * p.h_kv + h) * D + cb * 32, ov);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem, NSB == 1 ? 256 : 512);
}

// ---- host side ---------------------------------------------------------------------------------
static bool swa_tc_shape_ok(int B, int Lq, int Lk, int h_q, int h_kv, int D, int Dv, int S) {
  if (D != Dv || (D != 64 && D != 128)) return false;
  const int G = h_q / h_kv;
  if (G > 128 || (128 % G) != 0) return false;
  if (S <= 0 || Lq <= 0 || Lk <= 0) return false;
  if ((int64_t)B * Lk >= (1ll << 31) || (int64_t)B * Lq >= (1ll << 31)) return false;
  return true;
}

static SwaTcParams make_swa(const void* q, const void* k, const void* v, int B, int Lq, int Lk, int h_q, int h_kv, int W,
                            int S, int mask_lmk, int expand, int kv_start, float scale) {
  SwaTcParams p;
  p.q = (const bf16*)q; p.k = (const bf16*)k; p.v = (const bf16*)v; p.o = nullptr; p.lse = nullptr; p.d_o = nullptr;
  p.d_lse = nullptr; p.d_q = nullptr; p.d_k = nullptr; p.d_v = nullptr; p.delta = nullptr;
  p.B = B; p.Lq = Lq; p.Lk = Lk; p.h_q = h_q; p.h_kv = h_kv; p.W = W; p.S = S; p.mask_lmk = mask_lmk;
  p.expand = expand; p.kv_start = kv_start; p.scale = scale;
  return p;
}

int swa_fwd_tc_launch(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Lq, int Lk, int h_q,
                      int h_kv, int D, int Dv, int W, int S, int mask_lmk, int expand, float scale, int kv_start,
                      cudaStream_t st) {
  if (!swa_tc_shape_ok(B, Lq, Lk, h_q, h_kv, D, Dv, S)) return HILS_ERR_UNSUPPORTED;
  if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)o) & 15) return HILS_ERR_UNSUPPORTED;
  SwaTcParams p = make_swa(q, k, v, B, Lq, Lk, h_q, h_kv, W, S, mask_lmk, expand, kv_start, scale);
  p.o = (bf16*)o; p.lse = lse;
  CUtensorMap tmK, tmV;
  if (int rc = make_tmap_bf16_rows(&tmK, k, (uint64_t)B * Lk, (uint64_t)h_kv * D, (uint64_t)h_kv * D, 64)) return rc;
  if (int rc = make_tmap_bf16_rows(&tmV, v, (uint64_t)B * Lk, (uint64_t)h_kv * D, (uint64_t)h_kv * D, 64)) return rc;
  const int QB = 128 / (h_q / h_kv);
  const size_t smem = (size_t)(D / 64) * 16384 + 4 * (size_t)(D / 64) * 8192 + 16384 + 128;   // tiles + barriers
  dim3 grid(ceil_div(Lq, QB), h_kv, B);
  if (D == 64) {
    cudaFuncSetAttribute(swa_fwd_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    swa_fwd_tc_kernel<64><<<grid, kThreads, smem, st>>>(p, tmK, tmV);
  } else {
    cudaFuncSetAttribute(swa_fwd_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    swa_fwd_tc_kernel<128><<<grid, kThreads, smem, st>>>(p, tmK, tmV);
  }
  HILS_LAUNCH_CHECK("swa_fwd (tensor-core path)");
  return HILS_OK;
}

// fp32 scratch of the tensor-core backward: Delta per (batch, token, q-head); 0 = shape outside this path
size_t swa_bwd_tc_workspace(int B, int L, int h_q, int h_kv, int D, int Dv, int S) {
  if (!swa_tc_shape_ok(B, L, L, h_q, h_kv, D, Dv, S)) return 0;
  return (size_t)B * L * h_q * sizeof(float);
}

int swa_bwd_tc_launch(const void* q, const void* k, const void* v, const void* o, const float* lse, const void* d_o,
                      const float* d_lse, void* d_q, void* d_k, void* d_v, void* workspace, int B, int L, int h_q, int h_kv,
                      int D, int Dv, int W, int S, int mask_lmk, int expand, float scale, cudaStream_t st) {
  if (swa_bwd_tc_workspace(B, L, h_q, h_kv, D, Dv, S) == 0) return HILS_ERR_UNSUPPORTED;
  if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)o | (uintptr_t)d_o | (uintptr_t)d_q | (uintptr_t)d_k |
       (uintptr_t)d_v) & 15)
    return HILS_ERR_UNSUPPORTED;
  SwaTcParams p = make_swa(q, k, v, B, L, L, h_q, h_kv, W, S, mask_lmk, expand, 0, scale);
  p.o = (bf16*)const_cast<void*>(o); p.lse = const_cast<float*>(lse); p.d_o = (const bf16*)d_o; p.d_lse = d_lse;
  p.d_q = (bf16*)d_q; p.d_k = (bf16*)d_k; p.d_v = (bf16*)d_v; p.delta = static_cast<float*>(workspace);
  const int G = h_q / h_kv, QB = 128 / G;
  CUtensorMap tmK, tmV, tmQ, tmdO;
  if (int rc = make_tmap_bf16_rows(&tmK, k, (uint64_t)B * L, (uint64_t)h_kv * D, (uint64_t)h_kv * D, 64)) return rc;
  if (int rc = make_tmap_bf16_rows(&tmV, v, (uint64_t)B * L, (uint64_t)h_kv * D, (uint64_t)h_kv * D, 64)) return rc;
  if (int rc = make_tmap_bf16_thd(&tmQ, q, (uint64_t)B * L, h_q, D, G, QB)) return rc;
  if (int rc = make_tmap_bf16_thd(&tmdO, d_o, (uint64_t)B * L, h_q, D, G, QB)) return rc;
  const int NDS = 1;
  const size_t smem_dq = 1024 + 2 * (size_t)(D / 64) * 16384 + 4 * (size_t)(D / 64) * 8192 + 2 * 16384;
  // D = 64: two CTAs per SM need (228 KB / 2 - 1 KB reserved) = 115,712 bytes each, static variables (80 bytes) included.
  // The tiles take 114,688; the static variables sit in front of the dynamic
  // region, so 944 bytes of slack reach the next 1 KB boundary (the kernel checks that they do).
  const size_t smem_dkv = (D == 64 ? 944 : 1024) + 4 * (size_t)(D / 64) * 16384 + 2 * (size_t)(D / 64) * 8192 +
                          2 * (size_t)NDS * 16384;
  dim3 grid_q(ceil_div(L, QB), h_kv, B), grid_k(ceil_div(L, 64), h_kv, B);
  if (D == 64) {
    cudaFuncSetAttribute(swa_bwd_dq_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_dq);
    cudaFuncSetAttribute(swa_bwd_dkv_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_dkv);
    swa_bwd_dq_tc_kernel<64><<<grid_q, kThreads, smem_dq, st>>>(p, tmK, tmV);
    swa_bwd_dkv_tc_kernel<64><<<grid_k, kThreads, smem_dkv, st>>>(p, tmK, tmV, tmQ, tmdO);
  } else {
    cudaFuncSetAttribute(swa_bwd_dq_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_dq);
    cudaFuncSetAttribute(swa_bwd_dkv_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_dkv);
    swa_bwd_dq_tc_kernel<128><<<grid_q, kThreads, smem_dq, st>>>(p, tmK, tmV);
    swa_bwd_dkv_tc_kernel<128><<<grid_k, kThreads, smem_dkv, st>>>(p, tmK, tmV, tmQ, tmdO);
  }
  HILS_LAUNCH_CHECK("swa_bwd (tensor-core path)");
  return HILS_OK;
}

int take_status_swa_tc() {
  int v = 0, zero = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  if (cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));
  return v;
}

}  // namespace hils
