// Exact per-chunk log Z, forward and backward, on the 5th-generation tensor cores (tcgen05 + TMEM + TMA): bf16,
// chunk size 64.
//
// Contract (ops/exact_chunk_log_z_tilelang.py:89-112):
//   logZ[b,i,h,c] = logsumexp_{j in chunk c [, (j+1)%S != 0]} scale <q_i, k_j>   when i >= (c+1)S + W - 1, else -inf.
// A chunk that is defined for row i lies wholly before the row's window, so no causal or length test is left inside
// it: log Z of (row, chunk) is the log-sum-exp of one 64-column block of Q K^T.  One CTA owns 128 rows = 128/G tokens
// x the G query heads of one kv head; key tiles of 128 keys (two chunks) stream through a TMA ring, S = Q K^T is one
// tcgen05 product per tile into TMEM (double buffered), and the thread that owns a row reads its 2 x 64 scores from
// its TMEM lane and writes the two log-masses.  The output (B, L, H, ceil(L/64)) fp32 is written exactly once; chunks
// that are not defined for a row get -inf.
//
// Backward (ops/exact_chunk_log_z_tilelang.py:148-262 dQ, :273-391 dK): with p_ij = exp(scale s_ij - logZ[i, c(j)]),
//   dS_ij = scale * dlogZ[i, c(j)] * p_ij,   dQ = dS K,   dK = dS^T Q
// in the two atomic-free passes of the sliding-window and sparse kernels: a query-major pass (one CTA = 128 rows walks
// the chunks defined for them, dQ accumulates in TMEM) and a key-major pass (one CTA = one chunk walks the 128-row
// query blocks that see it, dK accumulates in TMEM as an M = 64 product of two MN-major operands).  The row's thread
// forms dS from its S row in TMEM and the two scalars logZ, dlogZ of (row, chunk).  All mbarrier waits are bounded.
#include "common.cuh"
#include "tc_rows.cuh"
#include "umma.cuh"

namespace hils {

using namespace umma;

static __device__ int g_logz_status = 0;

struct LogzTcParams {
  const void* q; const void* k; float* log_z;
  int B, L, h_q, h_kv, W, mask_lmk, n_chunk;
  float scale;
};

__device__ __forceinline__ bool lz_wait(uint64_t* b, uint32_t parity) {
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

// chunks defined for the row at position i: c < floor((i - W + 1) / 64), at least 0
__device__ __forceinline__ int lz_remote_chunks(int i, int W, int n_full) {
  return max(0, min(floor_div(i - W + 1, 64), n_full));
}

constexpr int kLzThreads = 192;   // row warpgroup + MMA warp + TMA warp

template <int D>
__global__ void __launch_bounds__(kLzThreads, 2) logz_fwd_tc_kernel(LogzTcParams p, const __grid_constant__ CUtensorMap tmQ,
                                                                   const __grid_constant__ CUtensorMap tmK) {
  constexpr int DB = D / 64;
  constexpr int TBYTES = DB * 16384;
  constexpr int NST = (D == 64) ? 3 : 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* Qs = smem;
  uint8_t* Ks = Qs + TBYTES;

  __shared__ uint64_t q_full, kv_full[3], kv_free[3], s_full[2], s_free[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = p.h_q / p.h_kv, gs = 31 - __clz(G), QB = 128 >> gs;
  const int blk = gridDim.x - 1 - blockIdx.x;            // the last token blocks see the most chunks: they start first
  const int l0 = blk * QB, h = blockIdx.y, b = blockIdx.z;
  const int n_full = p.L / 64;
  const int nch = lz_remote_chunks(min(l0 + QB - 1, p.L - 1), p.W, n_full);
  const int ntile = (nch + 1) >> 1;
  const float ninf = -CUDART_INF_F;

  // this thread's row and the tail of its output row that no tile covers
  const int r = tid & 127, tok = l0 + (r >> gs), hq = h * G + (r & (G - 1));
  float* out = p.log_z + (((int64_t)b * p.L + (tok < p.L ? tok : 0)) * p.h_q + hq) * p.n_chunk;
  if (tid < 128 && tok < p.L)
    for (int c = 2 * ntile; c < p.n_chunk; ++c) out[c] = ninf;
  if (ntile == 0 || *reinterpret_cast<volatile int*>(&g_logz_status) != 0) return;

  if (tid == 0) {
    mbar_init(&q_full, 1);
    for (int s = 0; s < NST; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_free[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_free[s], 128);
    }
    mbar_init_fence();
    abort_s = 0;
  }
  if (warp == 4) tmem_alloc(&tmem_base_s, 256);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;

  if (warp == 5) {
    if (lane == 0) {
      mbar_expect_tx(&q_full, TBYTES);
#pragma unroll
      for (int db = 0; db < DB; ++db) tma_load_3d(Qs + db * 16384, &tmQ, &q_full, db * 64, h * G, b * p.L + l0);
      for (int i = 0; i < ntile; ++i) {
        const int st = i % NST;
        if (abort_s) break;
        if (i >= NST && !lz_wait(&kv_free[st], ((i / NST) - 1) & 1)) { abort_s = 1; atomicCAS(&g_logz_status, 0, 7010000 + i); break; }
        mbar_expect_tx(&kv_full[st], TBYTES);
#pragma unroll
        for (int db = 0; db < DB; ++db)
          tma_load_2d(Ks + st * TBYTES + db * 16384, &tmK, &kv_full[st], h * D + db * 64, b * p.L + i * 128);
      }
    }
  } else if (warp == 4) {
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_bf16(128, 128, 0);
      const DescWords q_d = desc_words_sw128(smem_u32(Qs), 16, 1024), k_d = desc_words_sw128(smem_u32(Ks), 16, 1024);
      bool ok = lz_wait(&q_full, 0);
      for (int i = 0; ok && i < ntile; ++i) {
        const int st = i % NST, sb = i & 1;
        if (abort_s) { ok = false; break; }
        ok = lz_wait(&kv_full[st], (i / NST) & 1);
        if (ok && i >= 2) ok = lz_wait(&s_free[sb], ((i >> 1) - 1) & 1);
        if (!ok) { atomicCAS(&g_logz_status, 0, 7020000 + i); break; }
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
    const int lim = tok < p.L ? lz_remote_chunks(tok, p.W, n_full) : 0;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    const float sl2 = p.scale * 1.4426950408889634f;
    const bool pair_ok = (p.n_chunk & 1) == 0;              // rows start 8-byte aligned: two masses per store
    bool ok = true;
    for (int i = 0; i < ntile; ++i) {
      const int sb = i & 1;
      ok = lz_wait(&s_full[sb], (i >> 1) & 1);
      if (!ok) atomicCAS(&g_logz_status, 0, 7030000 + i);
      ok = __all_sync(0xffffffffu, ok) && !abort_s;
      if (!ok) break;
      tc_fence_after();
      float res[2];
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        float sv[64];
        tmem_ld32(tmem + lane_base + sb * 128 + half * 64, sv);
        tmem_ld32(tmem + lane_base + sb * 128 + half * 64 + 32, sv + 32);
        tmem_ld_wait();
        if (p.mask_lmk) sv[63] = ninf;
        float m4[4] = {sv[0], sv[1], sv[2], sv[3]};
#pragma unroll
        for (int j = 4; j < 64; ++j) m4[j & 3] = fmaxf(m4[j & 3], sv[j]);
        const float m = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
        const float mb = m * sl2;
        float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < 64; ++j) s4[j & 3] += ex2(fmaf(sv[j], sl2, -mb));
        const float sum = (s4[0] + s4[1]) + (s4[2] + s4[3]);
        res[half] = (2 * i + half < lim) ? fmaf(m, p.scale, logf(sum)) : ninf;
      }
      tc_fence_before();
      mbar_arrive(&s_free[sb]);
      if (tok < p.L) {
        const int c = 2 * i;
        if (pair_ok) {
          *reinterpret_cast<float2*>(out + c) = make_float2(res[0], res[1]);
        } else {
          out[c] = res[0];
          if (c + 1 < p.n_chunk) out[c + 1] = res[1];
        }
      }
    }
    if (!ok && lane == 0) abort_s = 1;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem, 256);
}

// Returns HILS_ERR_UNSUPPORTED (without setting an error text) when the call is outside this path.
int logz_fwd_tc_launch(const void* q, const void* k, float* log_z, int B, int L, int h_q, int h_kv, int D, int chunk_size,
                       int window_size, float sm_scale, int mask_lmk, cudaStream_t st) {
  if (chunk_size != 64 || (D != 64 && D != 128) || L < 64) return HILS_ERR_UNSUPPORTED;
  const int G = h_q / h_kv;
  if (G > 128 || (128 % G) != 0) return HILS_ERR_UNSUPPORTED;
  if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)log_z) & 15) return HILS_ERR_UNSUPPORTED;
  if ((int64_t)B * L >= (1ll << 31)) return HILS_ERR_UNSUPPORTED;
  LogzTcParams p;
  p.q = q; p.k = k; p.log_z = log_z; p.B = B; p.L = L; p.h_q = h_q; p.h_kv = h_kv; p.W = window_size;
  p.mask_lmk = mask_lmk; p.n_chunk = (L + 63) / 64; p.scale = sm_scale;
  const int QB = 128 / G;
  CUtensorMap tmQ, tmK;
  if (int rc = make_tmap_bf16_thd(&tmQ, q, (uint64_t)B * L, h_q, D, G, QB)) return rc;
  if (int rc = make_tmap_bf16_rows(&tmK, k, (uint64_t)B * L, (uint64_t)h_kv * D, (uint64_t)h_kv * D, 128)) return rc;
  const int NST = (D == 64) ? 3 : 2;
  const size_t smem = 1024 + (size_t)(1 + NST) * (D / 64) * 16384;
  dim3 grid((L + QB - 1) / QB, h_kv, B);
  if (D == 64) {
    cudaFuncSetAttribute(logz_fwd_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    logz_fwd_tc_kernel<64><<<grid, kLzThreads, smem, st>>>(p, tmQ, tmK);
  } else {
    cudaFuncSetAttribute(logz_fwd_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    logz_fwd_tc_kernel<128><<<grid, kLzThreads, smem, st>>>(p, tmQ, tmK);
  }
  HILS_LAUNCH_CHECK("chunk_logz_fwd (tcgen05 path)");
  return HILS_OK;
}

// =================================================================================================
// backward
// =================================================================================================
struct LogzBwdParams {
  const bf16* q; const bf16* k; const float* log_z; const float* d_log_z; bf16* d_q; bf16* d_k;
  int B, L, h_q, h_kv, W, n_chunk;
  float scale;
};

__device__ __forceinline__ void lz_fail(int code) { atomicCAS(&g_logz_status, 0, code); }

// dS row of one chunk from the S row: sv[j] <- scale * dz * exp2(sv[j] * sl2 - lz * log2e); zeros when the chunk is not
// defined for the row
__device__ __forceinline__ void lz_row_ds(float (&sv)[64], bool on, float sl2, float lz, float dz_scaled) {
  if (on) {
    const float nb = -lz * 1.4426950408889634f;
#pragma unroll
    for (int j = 0; j < 64; ++j) sv[j] = dz_scaled * ex2(fmaf(sv[j], sl2, nb));
  } else {
#pragma unroll
    for (int j = 0; j < 64; ++j) sv[j] = 0.f;
  }
}

// ---- query-major pass: dQ --------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(kLzThreads, 2) logz_bwd_dq_tc_kernel(LogzBwdParams p, const __grid_constant__ CUtensorMap tmK) {
  constexpr int DB = D / 64;
  constexpr int QBYTES = DB * 16384;
  constexpr int KBYTES = DB * 8192;       // one chunk's keys, 64 x D
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* Qs = smem;
  uint8_t* Ks = Qs + QBYTES;              // 2 stages
  uint8_t* dSs = Ks + 2 * KBYTES;         // 2 x [128 x 64] bf16

  __shared__ uint64_t k_full[2], s_full[2], ds_full[2], dq_done[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = p.h_q / p.h_kv, gs = 31 - __clz(G), QB = 128 >> gs;
  const int blk = gridDim.x - 1 - blockIdx.x;            // the last token blocks see the most chunks: they start first
  const int l0 = blk * QB, h = blockIdx.y, b = blockIdx.z;
  const int n_full = p.L / 64;
  const int n = lz_remote_chunks(min(l0 + QB - 1, p.L - 1), p.W, n_full);   // chunks this block walks

  const int r = tid & 127, tok = l0 + (r >> gs), hq = h * G + (r & (G - 1));
  const bool is_row = tid < 128, valid = is_row && tok < p.L;
  const int64_t rowi = ((int64_t)b * p.L + (valid ? tok : 0)) * p.h_q + hq;
  if (n == 0 || *reinterpret_cast<volatile int*>(&g_logz_status) != 0) {
    if (valid && n == 0) {
      float z[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) z[j] = 0.f;
      for (int cb = 0; cb < D / 32; ++cb) store32_bf16(p.d_q + rowi * D + cb * 32, z);
    }
    return;
  }
  if (tid == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&ds_full[s], 128);
      mbar_init(&dq_done[s], 1);
    }
    mbar_init_fence();
    abort_s = 0;
  }
  if (warp == 4) tmem_alloc(&tmem_base_s, 256);
  if (is_row) load_row_to_tile<D>(Qs, r, p.q + rowi * D, valid);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  const uint32_t tdQ = tmem + 128;

  if (warp == 5) {
    if (lane == 0) {
      for (int it = 0; it < n; ++it) {
        const int s = it & 1, u = it >> 1;
        if (abort_s) break;
        if (it >= 2 && !lz_wait(&dq_done[s], (u - 1) & 1)) { abort_s = 1; lz_fail(7110000 + it); break; }
        mbar_expect_tx(&k_full[s], KBYTES);
#pragma unroll
        for (int db = 0; db < DB; ++db) tma_load_2d(Ks + s * KBYTES + db * 8192, &tmK, &k_full[s], h * D + db * 64, b * p.L + it * 64);
      }
    }
  } else if (warp == 4) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = idesc_bf16(128, 64, 0);
      constexpr uint32_t idesc_dq = idesc_bf16(128, D, 1);
      const DescWords q_d = desc_words_sw128(smem_u32(Qs), 16, 1024), k_d = desc_words_sw128(smem_u32(Ks), 16, 1024),
                      ds_d = desc_words_sw128(smem_u32(dSs), 16, 1024), kmn_d = desc_words_sw128(smem_u32(Ks), 8192, 1024);
      auto issue_s = [&](int it) {
        const int s = it & 1;
        const uint32_t kb = k_d.lo + s * (KBYTES >> 4), ts = tmem + s * 64;
        mma_ss_w<false>(ts, q_d.lo, q_d.hi, kb, k_d.hi, idesc_s);
#pragma unroll
        for (int kk = 1; kk < D / 16; ++kk)
          mma_ss_w<true>(ts, q_d.lo + (((kk >> 2) * 16384 + (kk & 3) * 32) >> 4), q_d.hi,
                         kb + (((kk >> 2) * 8192 + (kk & 3) * 32) >> 4), k_d.hi, idesc_s);
        mma_commit(&s_full[s]);
      };
      bool ok = lz_wait(&k_full[0], 0);
      if (ok) { tc_fence_after(); issue_s(0); }
      for (int it = 0; ok && it < n; ++it) {
        const int s = it & 1, u = it >> 1;
        if (abort_s) break;
        if (it + 1 < n) {                 // S of the next chunk: its accumulator was read before the dS arrival of tile it - 1
          ok = lz_wait(&k_full[(it + 1) & 1], ((it + 1) >> 1) & 1);
          if (!ok) break;
          tc_fence_after();
          issue_s(it + 1);
        }
        ok = lz_wait(&ds_full[s], u & 1);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a0 = ds_d.lo + s * (16384 >> 4), b0 = kmn_d.lo + s * (KBYTES >> 4);
        mma_ss_wr(tdQ, a0, ds_d.hi, b0, kmn_d.hi, idesc_dq, it > 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 1; kk < 4; ++kk) mma_ss_w<true>(tdQ, a0 + ((kk * 32) >> 4), ds_d.hi, b0 + ((kk * 2048) >> 4), kmn_d.hi, idesc_dq);
        mma_commit(&dq_done[s]);
      }
      if (!ok) { abort_s = 1; lz_fail(7120000); }
    }
  } else {
    const int lim = valid ? lz_remote_chunks(tok, p.W, n_full) : 0;
    const float sl2 = p.scale * 1.4426950408889634f;
    const float* lzr = p.log_z + rowi * p.n_chunk;
    const float* dzr = p.d_log_z + rowi * p.n_chunk;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    bool ok = true;
    for (int it = 0; it < n; ++it) {
      const int s = it & 1, u = it >> 1;
      const bool on = it < lim;
      const float lz = on ? lzr[it] : 0.f, dz = on ? dzr[it] * p.scale : 0.f;
      ok = lz_wait(&s_full[s], u & 1);
      if (it >= 2) ok = lz_wait(&dq_done[s], (u - 1) & 1) && ok;   // the dS buffer's previous product has run
      ok = __all_sync(0xffffffffu, ok) && !abort_s;
      if (!ok) break;
      tc_fence_after();
      float sv[64];
      tmem_ld32(tmem + lane_base + s * 64, sv);
      tmem_ld32(tmem + lane_base + s * 64 + 32, sv + 32);
      tmem_ld_wait();
      lz_row_ds(sv, on, sl2, lz, dz);
      store_row_bf16_sw128(dSs + s * 16384, r, sv);
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(&ds_full[s]);
    }
    if (ok) {
      ok = lz_wait(&dq_done[(n - 1) & 1], ((n - 1) >> 1) & 1);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (!ok && lane == 0) { abort_s = 1; lz_fail(7130000); }
    if (ok) tc_fence_after();
#pragma unroll
    for (int cb = 0; cb < D / 32; ++cb) {
      float ov[32];
      if (ok) {
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
  if (warp == 4) tmem_dealloc(tmem, 256);
}

// ---- key-major pass: dK ----------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(kLzThreads, 2) logz_bwd_dk_tc_kernel(LogzBwdParams p, const __grid_constant__ CUtensorMap tmK,
                                                                      const __grid_constant__ CUtensorMap tmQ) {
  constexpr int DB = D / 64;
  constexpr int QBYTES = DB * 16384;
  constexpr int KBYTES = DB * 8192;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* Qs = smem;                     // 2 stages
  uint8_t* Ks = Qs + 2 * QBYTES;
  uint8_t* dSs = Ks + KBYTES;             // 2 x [128 x 64] bf16
  {
    // At D = 128 two CTAs per SM need the tiles, the static variables in front of them and the alignment gap to fit
    // 115,712 bytes, which the launch sizes to the byte: refuse to run rather than write past the dynamic region if
    // the layout is ever different.
    uint32_t dyn_bytes;
    asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_bytes));
    if ((size_t)(dSs + 2 * 16384 - smem_raw) > dyn_bytes) {
      if (threadIdx.x == 0) atomicCAS(&g_logz_status, 0, 7200001);
      return;
    }
  }

  __shared__ uint64_t k_full, q_full[2], s_full[2], ds_full[2], dk_done[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;   // early chunks are seen by the most queries and start first
  const int G = p.h_q / p.h_kv, gs = 31 - __clz(G), QB = 128 >> gs;
  const int L = p.L;
  // rows that see chunk c: tokens i >= (c + 1) * 64 + W - 1; chunks behind the last full one are never defined
  const int i_first = (c + 1) * 64 + p.W - 1;
  const bool any = c < L / 64 && i_first < L;
  const int blk0 = any ? i_first / QB : 0;
  const int m = any ? (L - 1) / QB - blk0 + 1 : 0;
  const int krow = 16 * warp + lane;          // M = 64 accumulator: lanes 0..15 of each row warp hold key rows
  const int tokj = c * 64 + krow;
  if (m == 0 || *reinterpret_cast<volatile int*>(&g_logz_status) != 0) {
    if (m == 0 && warp < 4 && lane < 16 && tokj < L) {
      float z[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) z[j] = 0.f;
      for (int cb = 0; cb < D / 32; ++cb) store32_bf16(p.d_k + (((int64_t)b * L + tokj) * p.h_kv + h) * D + cb * 32, z);
    }
    return;
  }
  if (tid == 0) {
    mbar_init(&k_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&ds_full[s], 128);
      mbar_init(&dk_done[s], 1);
    }
    mbar_init_fence();
    abort_s = 0;
  }
  if (warp == 4) tmem_alloc(&tmem_base_s, 256);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  const uint32_t tdK = tmem + 128;

  if (warp == 5) {
    if (lane == 0) {
      mbar_expect_tx(&k_full, KBYTES);
#pragma unroll
      for (int db = 0; db < DB; ++db) tma_load_2d(Ks + db * 8192, &tmK, &k_full, h * D + db * 64, b * L + c * 64);
      for (int j = 0; j < m; ++j) {
        const int s = j & 1, u = j >> 1;
        if (abort_s) break;
        if (j >= 2 && !lz_wait(&dk_done[s], (u - 1) & 1)) { abort_s = 1; lz_fail(7210000 + j); break; }
        mbar_expect_tx(&q_full[s], QBYTES);
#pragma unroll
        for (int db = 0; db < DB; ++db) tma_load_3d(Qs + s * QBYTES + db * 16384, &tmQ, &q_full[s], db * 64, h * G, b * L + (blk0 + j) * QB);
      }
    }
  } else if (warp == 4) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = idesc_bf16(128, 64, 0);
      constexpr uint32_t idesc_dk = idesc_bf16(64, D, 1, 1);
      const DescWords q_d = desc_words_sw128(smem_u32(Qs), 16, 1024), k_d = desc_words_sw128(smem_u32(Ks), 16, 1024),
                      qmn_d = desc_words_sw128(smem_u32(Qs), 16384, 1024), ds_d = desc_words_sw128(smem_u32(dSs), 16384, 1024);
      auto issue_s = [&](int j) {
        const int s = j & 1;
        const uint32_t qb = q_d.lo + s * (QBYTES >> 4), ts = tmem + s * 64;
        mma_ss_w<false>(ts, qb, q_d.hi, k_d.lo, k_d.hi, idesc_s);
#pragma unroll
        for (int kk = 1; kk < D / 16; ++kk)
          mma_ss_w<true>(ts, qb + (((kk >> 2) * 16384 + (kk & 3) * 32) >> 4), q_d.hi,
                         k_d.lo + (((kk >> 2) * 8192 + (kk & 3) * 32) >> 4), k_d.hi, idesc_s);
        mma_commit(&s_full[s]);
      };
      bool ok = lz_wait(&k_full, 0) && lz_wait(&q_full[0], 0);
      if (ok) { tc_fence_after(); issue_s(0); }
      for (int j = 0; ok && j < m; ++j) {
        const int s = j & 1, u = j >> 1;
        if (abort_s) break;
        if (j + 1 < m) {
          ok = lz_wait(&q_full[(j + 1) & 1], ((j + 1) >> 1) & 1);
          if (!ok) break;
          tc_fence_after();
          issue_s(j + 1);
        }
        ok = lz_wait(&ds_full[s], u & 1);
        if (!ok) break;
        tc_fence_after();
        const uint32_t dsb = ds_d.lo + s * (16384 >> 4), qb = qmn_d.lo + s * (QBYTES >> 4);
        mma_ss_wr(tdK, dsb, ds_d.hi, qb, qmn_d.hi, idesc_dk, j > 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 1; kk < 8; ++kk) mma_ss_w<true>(tdK, dsb + ((kk * 2048) >> 4), ds_d.hi, qb + ((kk * 2048) >> 4), qmn_d.hi, idesc_dk);
        mma_commit(&dk_done[s]);
      }
      if (!ok) { abort_s = 1; lz_fail(7220000); }
    }
  } else {
    const int r = tid, ql = r >> gs, hq = h * G + (r & (G - 1));
    const float sl2 = p.scale * 1.4426950408889634f;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    bool ok = true;
    for (int j = 0; j < m; ++j) {
      const int s = j & 1, u = j >> 1;
      const int i = (blk0 + j) * QB + ql;
      const bool on = i >= i_first && i < L;
      float lz = 0.f, dz = 0.f;
      if (on) {
        const int64_t off = (((int64_t)b * L + i) * p.h_q + hq) * p.n_chunk + c;
        lz = p.log_z[off];
        dz = p.d_log_z[off] * p.scale;
      }
      ok = lz_wait(&s_full[s], u & 1);
      if (j >= 2) ok = lz_wait(&dk_done[s], (u - 1) & 1) && ok;    // the dS buffer's previous product has run
      ok = __all_sync(0xffffffffu, ok) && !abort_s;
      if (!ok) break;
      tc_fence_after();
      float sv[64];
      tmem_ld32(tmem + lane_base + s * 64, sv);
      tmem_ld32(tmem + lane_base + s * 64 + 32, sv + 32);
      tmem_ld_wait();
      lz_row_ds(sv, on, sl2, lz, dz);
      store_row_bf16_sw128(dSs + s * 16384, r, sv);
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(&ds_full[s]);
    }
    if (ok) {
      ok = lz_wait(&dk_done[(m - 1) & 1], ((m - 1) >> 1) & 1);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (!ok && lane == 0) { abort_s = 1; lz_fail(7230000); }
    if (ok) tc_fence_after();
#pragma unroll
    for (int cb = 0; cb < D / 32; ++cb) {
      float ov[32];
      if (ok) {
        tmem_ld32(tdK + lane_base + cb * 32, ov);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) ov[jj] = 0.f;
      }
      if (lane < 16 && tokj < L) store32_bf16(p.d_k + (((int64_t)b * L + tokj) * p.h_kv + h) * D + cb * 32, ov);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem, 256);
}

// Returns HILS_ERR_UNSUPPORTED (without setting an error text) when the call is outside this path.
int logz_bwd_tc_launch(const void* q, const void* k, const float* log_z, const float* d_log_z, void* d_q, void* d_k, int B, int L,
                       int h_q, int h_kv, int D, int chunk_size, int window_size, float sm_scale, cudaStream_t st) {
  if (chunk_size != 64 || (D != 64 && D != 128) || L < 64) return HILS_ERR_UNSUPPORTED;
  const int G = h_q / h_kv;
  if (G > 128 || (128 % G) != 0) return HILS_ERR_UNSUPPORTED;
  if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)d_q | (uintptr_t)d_k) & 15) return HILS_ERR_UNSUPPORTED;
  if ((int64_t)B * L >= (1ll << 31)) return HILS_ERR_UNSUPPORTED;
  LogzBwdParams p;
  p.q = (const bf16*)q; p.k = (const bf16*)k; p.log_z = log_z; p.d_log_z = d_log_z; p.d_q = (bf16*)d_q; p.d_k = (bf16*)d_k;
  p.B = B; p.L = L; p.h_q = h_q; p.h_kv = h_kv; p.W = window_size; p.n_chunk = (L + 63) / 64; p.scale = sm_scale;
  const int QB = 128 / G;
  CUtensorMap tmK, tmQ;
  if (int rc = make_tmap_bf16_rows(&tmK, k, (uint64_t)B * L, (uint64_t)h_kv * D, (uint64_t)h_kv * D, 64)) return rc;
  if (int rc = make_tmap_bf16_thd(&tmQ, q, (uint64_t)B * L, h_q, D, G, QB)) return rc;
  const size_t DBb = (size_t)(D / 64);
  const size_t smem_dq = 1024 + DBb * 16384 + 2 * DBb * 8192 + 2 * 16384;
  // key-major pass at D = 128: two CTAs per SM have (228 KB / 2 - 1 KB reserved) = 115,712 bytes each, static variables
  // (80 bytes, in front of the dynamic region) included; the tiles take 114,688, so the gap to the next 1 KB boundary
  // is 944 bytes, not 1024 (the kernel checks that the layout fits)
  const size_t smem_dk = (D == 128 ? 944 : 1024) + 2 * DBb * 16384 + DBb * 8192 + 2 * 16384;
  dim3 grid_q((L + QB - 1) / QB, h_kv, B), grid_k((L + 63) / 64, h_kv, B);
  if (D == 64) {
    cudaFuncSetAttribute(logz_bwd_dq_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_dq);
    cudaFuncSetAttribute(logz_bwd_dk_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_dk);
    logz_bwd_dq_tc_kernel<64><<<grid_q, kLzThreads, smem_dq, st>>>(p, tmK);
    logz_bwd_dk_tc_kernel<64><<<grid_k, kLzThreads, smem_dk, st>>>(p, tmK, tmQ);
  } else {
    cudaFuncSetAttribute(logz_bwd_dq_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_dq);
    cudaFuncSetAttribute(logz_bwd_dk_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_dk);
    logz_bwd_dq_tc_kernel<128><<<grid_q, kLzThreads, smem_dq, st>>>(p, tmK);
    logz_bwd_dk_tc_kernel<128><<<grid_k, kLzThreads, smem_dk, st>>>(p, tmK, tmQ);
  }
  HILS_LAUNCH_CHECK("chunk_logz_bwd (tcgen05 path)");
  return HILS_OK;
}

int take_status_logz_tc() {
  int v = 0, zero = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  if (cudaMemcpyFromSymbol(&v, g_logz_status, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(g_logz_status, &zero, sizeof(int));
  return v;
}

}  // namespace hils
