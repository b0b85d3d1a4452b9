// Gradient of the chunk keys in the selection backward, on the tensor cores (tcgen05), bf16.
//
//   dk'[c] = scale * sum_{(token, g) that selected c at slot k} dscore[token, g, k] * q[token, g]
// (ops/topk_head_softmax.py:1040-1092 forms this with a dense (B,h,G,L,N) scatter and a bmm.)
// Here one CTA owns a tile of 64 chunks of one key head and walks all 128-row query blocks.  For a
// block, each row thread scatters its K dscore values into a zeroed [128 rows x 64 chunks] bf16 tile
// in shared memory (the dense slice of that scatter, never materialised in HBM); the Q tile arrives
// by TMA; one M=64 MMA chain adds tile^T * Q into the TMEM accumulator.  The result is written once:
// no atomics, no fp32 accumulator in HBM, deterministic.
#include "tc_rows.cuh"
#include "umma.cuh"

namespace hils {

static __device__ int g_device_status = 0;

using namespace umma;

struct TopkBwdTcParams {
  const bf16* ds; const int32_t* idx; bf16* d_lmks;
  int B, L, N, h_kv, G, K, per_qhead;
  float scale;
};

template <int D>
__global__ void __launch_bounds__(192, 1) topk_bwd_dk_tc_kernel(TopkBwdTcParams p, const __grid_constant__ CUtensorMap tmQ) {
  constexpr int DB = D / 64;
  constexpr int QBYTES = DB * 16384;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* Qs = smem;                 // 2 stages
  uint8_t* As = Qs + 2 * QBYTES;      // 2 x [128 rows x 64 chunks] bf16

  __shared__ uint64_t q_full[2], a_full[2], mma_done[2], all_done;
  __shared__ uint32_t tmem_base_s;
  __shared__ volatile int abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c0 = blockIdx.x * 64, hl = blockIdx.y, b = blockIdx.z;
  // rows of a block: (token, group member) for shared keys, tokens of one q-head for per-q-head keys
  const int Gr = p.per_qhead ? 1 : p.G;
  const int QB = 128 / Gr;
  const int hq0 = p.per_qhead ? hl : hl * p.G;          // first q head of the rows
  const int hk = p.per_qhead ? hl / p.G : hl;           // kv head whose id lists apply
  const int h_q = p.h_kv * p.G;
  const int HL = p.per_qhead ? h_q : p.h_kv;
  const int nblk = (p.L + QB - 1) / QB;

  if (tid == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&a_full[s], 128);
      mbar_init(&mma_done[s], 1);
    }
    mbar_init(&all_done, 1);
    mbar_init_fence();
    abort_s = 0;
  }
  if (warp == 4) tmem_alloc(&tmem_base_s, 128);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;

  if (warp == 5) {
    if (lane == 0) {
      for (int j = 0; j < nblk; ++j) {
        const int s = j & 1, u = j >> 1;
        if (abort_s) break;
        if (j >= 2 && !mbar_wait(&mma_done[s], (u - 1) & 1)) { abort_s = 1; atomicExch(&g_device_status, 501); break; }
        mbar_expect_tx(&q_full[s], QBYTES);
#pragma unroll
        for (int db = 0; db < DB; ++db)
          tma_load_3d(Qs + s * QBYTES + db * 16384, &tmQ, &q_full[s], db * 64, hq0, b * p.L + j * QB);
      }
    }
  } else if (warp == 4) {
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_bf16(64, D, 1, 1);
      const uint32_t q_addr = smem_u32(Qs), a_addr = smem_u32(As);
      bool ok = true;
      for (int j = 0; ok && j < nblk; ++j) {
        const int s = j & 1, u = j >> 1;
        if (abort_s) break;
        ok = mbar_wait(&q_full[s], u & 1) && mbar_wait(&a_full[s], u & 1);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          mma_ss(tmem, desc_sw128(a_addr + s * 16384 + kk * 2048, 16384, 1024),
                 desc_sw128(q_addr + s * QBYTES + kk * 2048, 16384, 1024), idesc, (j > 0 || kk > 0) ? 1u : 0u);
        mma_commit(&mma_done[s]);
      }
      if (ok) mma_commit(&all_done);
      else { abort_s = 1; atomicExch(&g_device_status, 502); }
    }
  } else {
    const int r = tid, ql = r / Gr, g = r % Gr, hq = hq0 + g;
    bool ok = true;
    for (int j = 0; j < nblk; ++j) {
      const int s = j & 1, u = j >> 1;
      const int t = j * QB + ql;
      if (j >= 2) ok = mbar_wait(&mma_done[s], (u - 1) & 1);
      ok = __all_sync(0xffffffffu, ok) && !abort_s;
      if (!ok) break;
      uint8_t* tile = As + s * 16384;
      store_row_zero_sw128(tile, r);
      if (t < p.L) {
        const int32_t* ids = p.idx + (((int64_t)b * p.L + t) * p.h_kv + hk) * p.K;
        const bf16* dsr = p.ds + (((int64_t)b * p.L + t) * h_q + hq) * p.K;
        for (int k = 0; k < p.K; ++k) {
          const int id = __ldg(ids + k);
          if (id < 0) break;
          const int col = id - c0;
          if (col >= 0 && col < 64 && id < p.N) {
            // equal ids in one row add up (written by this thread only, so read-modify-write is safe)
            bf16* cell = reinterpret_cast<bf16*>(tile + sw128_off(r, col >> 3)) + (col & 7);
            *cell = __float2bfloat16_rn(__bfloat162float(*cell) + __bfloat162float(dsr[k]));
          }
        }
      }
      fence_async_smem();
      mbar_arrive(&a_full[s]);
    }
    if (ok) {
      ok = mbar_wait(&all_done, 0);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok && lane == 0) { abort_s = 1; atomicExch(&g_device_status, 503); }
    } else if (lane == 0) {
      abort_s = 1;
      atomicExch(&g_device_status, 504);
    }
    // M = 64 accumulator: chunk row 16*warp + lane lives in TMEM lane 32*warp + lane (lanes 0..15)
    const int crow = c0 + 16 * warp + lane;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    if (ok) tc_fence_after();
#pragma unroll
    for (int cb = 0; cb < D / 32; ++cb) {
      float ov[32];
      if (ok) {
        tmem_ld32(tmem + lane_base + cb * 32, ov);
        tmem_ld_wait();
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) ov[jj] *= p.scale;
      } else {
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) ov[jj] = 0.f;
      }
      if (lane < 16 && crow < p.N) store32_bf16(p.d_lmks + (((int64_t)b * p.N + crow) * HL + hl) * D + cb * 32, ov);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem, 128);
}

// HILS_ERR_UNSUPPORTED when the shape is outside this path
int topk_bwd_dk_tc_launch(const void* d_scores, const int32_t* indices, const void* q, void* d_lmks, int B, int L, int N,
                          int h_kv, int G, int D, int topk, int per_qhead, float scale, cudaStream_t st) {
  if (D != 64 && D != 128) return HILS_ERR_UNSUPPORTED;
  const int Gr = per_qhead ? 1 : G;
  if (Gr > 128 || (128 % Gr) != 0 || N <= 0 || L <= 0) return HILS_ERR_UNSUPPORTED;
  if ((int64_t)B * L >= (1ll << 31)) return HILS_ERR_UNSUPPORTED;
  if (((uintptr_t)q | (uintptr_t)d_lmks) & 15) return HILS_ERR_UNSUPPORTED;
  TopkBwdTcParams p;
  p.ds = (const bf16*)d_scores; p.idx = indices; p.d_lmks = (bf16*)d_lmks;
  p.B = B; p.L = L; p.N = N; p.h_kv = h_kv; p.G = G; p.K = topk; p.per_qhead = per_qhead; p.scale = scale;
  CUtensorMap tmQ;
  if (int rc = make_tmap_bf16_thd(&tmQ, q, (uint64_t)B * L, (uint64_t)h_kv * G, D, Gr, 128 / Gr)) return rc;
  const int HL = per_qhead ? h_kv * G : h_kv;
  const size_t smem = 1024 + 2 * (size_t)(D / 64) * 16384 + 2 * 16384;
  dim3 grid((N + 63) / 64, HL, B);
  if (D == 64) {
    cudaFuncSetAttribute(topk_bwd_dk_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    topk_bwd_dk_tc_kernel<64><<<grid, 192, smem, st>>>(p, tmQ);
  } else {
    cudaFuncSetAttribute(topk_bwd_dk_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    topk_bwd_dk_tc_kernel<128><<<grid, 192, smem, st>>>(p, tmQ);
  }
  HILS_LAUNCH_CHECK("topk_bwd (tensor-core chunk-key gradient)");
  return HILS_OK;
}

int take_status_topk_tc() {
  int v = 0, zero = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  if (cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));
  return v;
}

}  // namespace hils
