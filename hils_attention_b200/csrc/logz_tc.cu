// Exact per-chunk log Z, forward, on the 5th-generation tensor cores (tcgen05 + TMEM + TMA): bf16, chunk size 64.
//
// Contract (ops/exact_chunk_log_z_tilelang.py:89-112):
//   logZ[b,i,h,c] = logsumexp_{j in chunk c [, (j+1)%S != 0]} scale <q_i, k_j>   when i >= (c+1)S + W - 1, else -inf.
// A chunk that is defined for row i lies wholly before the row's window, so no causal or length test is left inside
// it: log Z of (row, chunk) is the log-sum-exp of one 64-column block of Q K^T.  One CTA owns 128 rows = 128/G tokens
// x the G query heads of one kv head; key tiles of 128 keys (two chunks) stream through a TMA ring, S = Q K^T is one
// tcgen05 product per tile into TMEM (double buffered), and the thread that owns a row reads its 2 x 64 scores from
// its TMEM lane and writes the two log-masses.  The output (B, L, H, ceil(L/64)) fp32 is written exactly once; chunks
// that are not defined for a row get -inf.  All mbarrier waits are bounded.
#include "common.cuh"
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

int take_status_logz_tc() {
  int v = 0, zero = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  if (cudaMemcpyFromSymbol(&v, g_logz_status, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(g_logz_status, &zero, sizeof(int));
  return v;
}

}  // namespace hils
