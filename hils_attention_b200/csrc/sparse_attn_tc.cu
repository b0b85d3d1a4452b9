// Sparse chunk attention forward on the 5th-generation tensor cores (tcgen05 + TMEM + TMA), bf16.
//
// One CTA owns 128 rows = 128/G consecutive query tokens x the G query heads of one kv head.  The
// chunks selected by any of its tokens form a sorted union list (bitmap in shared memory); the CTA
// walks that list once.  For every chunk c of the union:
//   TMA warp     : K_c and V_c tiles [64 x D] -> shared memory (128-byte swizzle), 2-stage ring
//   MMA warp     : S = Q K_c^T  (tcgen05.mma, fp32 accumulator in TMEM, double buffered)
//   softmax warps: one thread per row reads its S row from TMEM; a row that selected c forms
//                  P = w * softmax(scale * S) (own softmax per chunk, last key masked), other rows
//                  write zeros; P goes to shared memory as the A operand of the second product
//   MMA warp     : O += P V_c   (accumulates over the whole union in TMEM)
// The epilogue converts the O rows to bf16 and stores them.  Rows are independent per chunk
// (ops/hils_fwd_bwd_head.py:404-485), so no running maximum or rescaling of O is needed.
//
// A row's id list is consumed with a moving pointer when every list of the block is ascending
// (what the selection kernel emits); otherwise each row scans its K ids per chunk.  Equal ids in
// one row add their weights.  All mbarrier waits are bounded; on expiry the kernel records a status
// word, every role leaves its loop, TMEM is released and the kernel returns.
#include "sparse_attn_generic.cuh"
#include "umma.cuh"
#include "tc_rows.cuh"

namespace hils {

static __device__ int g_device_status = 0;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The tensor-map encoder is a driver-API call and needs a context current on the calling host
// thread; a thread that has made no runtime call yet (e.g. an autograd worker) has none until the
// runtime binds the primary context, which this does once per thread.
static void bind_context_once() {
  static thread_local bool done = false;
  if (!done) {
    cudaFree(nullptr);
    done = true;
  }
}

int make_tmap_bf16_rows(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride_elems,
                        uint32_t box_rows) {
  bind_context_once();
  static EncodeTiledFn enc = nullptr;
  if (!enc) {
    cudaDriverEntryPointQueryResult q;
    void* fn = nullptr;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || !fn) return cuda_fail(e, "cuTensorMapEncodeTiled lookup");
    enc = (EncodeTiledFn)fn;
  }
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_stride_elems * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t es[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, es,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with %d", (int)r);
    return HILS_ERR_CUDA;
  }
  return HILS_OK;
}

int make_tmap_bf16_thd(CUtensorMap* map, const void* base, uint64_t tokens, uint64_t heads, uint64_t D,
                       uint32_t box_heads, uint32_t box_tokens) {
  bind_context_once();
  static EncodeTiledFn enc = nullptr;
  if (!enc) {
    cudaDriverEntryPointQueryResult q;
    void* fn = nullptr;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || !fn) return cuda_fail(e, "cuTensorMapEncodeTiled lookup");
    enc = (EncodeTiledFn)fn;
  }
  cuuint64_t dims[3] = {D, heads, tokens};
  cuuint64_t strides[2] = {D * 2, heads * D * 2};
  cuuint32_t box[3] = {64, box_heads, box_tokens};
  cuuint32_t es[3] = {1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, es,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled (3-D) failed with %d", (int)r);
    return HILS_ERR_CUDA;
  }
  return HILS_OK;
}

using namespace umma;

constexpr int kBwdThreads = 320;  // 2 row warpgroups + MMA warp + TMA warp
constexpr int kFwdStages = 3;     // K/V ring depth of the forward kernel

template <int D>
__global__ void __launch_bounds__(kBwdThreads, 2) sparse_fwd_tc_kernel(SparseParams p, const __grid_constant__ CUtensorMap tmK,
                                                                   const __grid_constant__ CUtensorMap tmV) {
  constexpr int DB = D / 64;             // 64-wide column blocks of a [rows x D] tile
  constexpr int QBYTES = DB * 16384;     // Q tile 128 x D
  constexpr int KVBYTES = DB * 8192;     // K or V tile 64 x D
  constexpr int NST = kFwdStages;        // K/V ring depth (loads run ahead of the MMAs)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* Qs = smem;
  uint8_t* Ks = Qs + QBYTES;             // NST stages
  uint8_t* Vs = Ks + NST * KVBYTES;      // NST stages
  uint8_t* Ps = Vs + NST * KVBYTES;        // 2 x [128 x 64] bf16
  int* union_s = reinterpret_cast<int*>(Ps + 2 * 16384);
  const int nchunk = p.T / 64;
  const int nwords = (nchunk + 31) >> 5;
  const int G = p.h_q / p.h_kv, QB = 128 / G;
  const int umax = min(nchunk, QB * p.K);
  uint32_t* bitmap_s = reinterpret_cast<uint32_t*>(union_s + umax);

  __shared__ uint64_t kv_full[4], kv_free[4], s_full[2], p_full[2], pv_done[2], all_done;
  __shared__ uint32_t tmem_base_s;
  __shared__ int n_union_s, warp_tot_s[4];
  __shared__ volatile int abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int blk = gridDim.x - 1 - blockIdx.x;  // heaviest (latest) query blocks first
  const int q0 = blk * QB, h = blockIdx.y, b = blockIdx.z;

  if (tid == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 128);
      mbar_init(&pv_done[s], 1);
    }
    for (int st = 0; st < NST; ++st) {
      mbar_init(&kv_full[st], 1);
      mbar_init(&kv_free[st], 1);
    }
    mbar_init(&all_done, 1);
    mbar_init_fence();
    abort_s = 0;
  }
  if (warp == 8) tmem_alloc(&tmem_base_s, 256);
  for (int w = tid; w < nwords; w += kBwdThreads) bitmap_s[w] = 0u;
  __syncthreads();

  // ---- per-row setup: Q row into shared memory, chunk ids into the bitmap -----------------------
  // two row warpgroups (threads 0..127, 128..255) each own all 128 rows and alternate over the union
  const int r = tid & 127, wg = tid >> 7;
  const int ql = r / G, g = r % G, t = q0 + ql;
  const bool is_row = tid < 256, is_loader = tid < 128;
  const bool valid = is_row && t < p.L;
  const int hq = h * G + g;
  const int32_t* ids = p.idx + (((int64_t)b * p.L + (valid ? t : 0)) * p.h_kv + h) * p.K;
  const bf16* wrow = static_cast<const bf16*>(p.w) + (((int64_t)b * p.L + (valid ? t : 0)) * p.h_q + hq) * p.num_weights;
  int nvalid = 0;
  int my_unsorted = 0;
  if (is_loader) {
    const bf16* qrow = static_cast<const bf16*>(p.q) + (((int64_t)b * p.L + (valid ? t : 0)) * p.h_q + hq) * D;
#pragma unroll
    for (int c = 0; c < D / 8; ++c) {
      uint4 x = make_uint4(0u, 0u, 0u, 0u);
      if (valid) x = *reinterpret_cast<const uint4*>(qrow + c * 8);
      *reinterpret_cast<uint4*>(Qs + (c >> 3) * 16384 + sw128_off(r, c & 7)) = x;
    }
  }
  if (valid) {
    int prev = -1;
    for (int k = 0; k < p.K; ++k) {
      const int id = __ldg(ids + k);
      if (id < 0) break;
      ++nvalid;
      if (id < prev) my_unsorted = 1;
      prev = id;
      if (is_loader && g == 0 && id < nchunk) atomicOr(&bitmap_s[id >> 5], 1u << (id & 31));
    }
  }
  const int unsorted = __syncthreads_or(my_unsorted);

  // ---- bitmap -> ascending union list ------------------------------------------------------------
  {
    const int wpt = (nwords + 127) / 128;
    int cnt = 0;
    if (is_loader)
      for (int w = tid * wpt; w < min(nwords, (tid + 1) * wpt); ++w) cnt += __popc(bitmap_s[w]);
    int inc = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int n = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += n;
    }
    if (is_loader && lane == 31) warp_tot_s[warp] = inc;
    __syncthreads();
    if (is_loader) {
      int base = inc - cnt;
      for (int w = 0; w < warp; ++w) base += warp_tot_s[w];
      for (int w = tid * wpt; w < min(nwords, (tid + 1) * wpt); ++w) {
        uint32_t bits = bitmap_s[w];
        while (bits) {
          const int bpos = __ffs(bits) - 1;
          bits &= bits - 1;
          if (base < umax) union_s[base] = w * 32 + bpos;
          ++base;
        }
      }
      if (tid == 127) n_union_s = min(base, umax);
    }
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const int n = n_union_s;
  const uint32_t tmem = tmem_base_s;
  const uint32_t tS = tmem, tO = tmem + 128;

  if (warp == 9) {
    // =============================== TMA producer ===============================================
    if (lane == 0) {
      for (int i = 0; i < n; ++i) {
        const int s = i % NST;
        if (abort_s) break;
        if (i >= NST && !mbar_wait(&kv_free[s], ((i / NST) - 1) & 1)) { abort_s = 1; atomicExch(&g_device_status, 101); break; }
        const int c = union_s[i];
        mbar_expect_tx(&kv_full[s], 2 * KVBYTES);
#pragma unroll
        for (int db = 0; db < DB; ++db) {
          tma_load_2d(Ks + s * KVBYTES + db * 8192, &tmK, &kv_full[s], h * D + db * 64, b * p.T + c * 64);
          tma_load_2d(Vs + s * KVBYTES + db * 8192, &tmV, &kv_full[s], h * D + db * 64, b * p.T + c * 64);
        }
      }
    }
  } else if (warp == 8) {
    // =============================== MMA issuer =================================================
    if (lane == 0 && n > 0) {
      constexpr uint32_t idesc_qk = idesc_bf16(128, 64, 0);
      constexpr uint32_t idesc_pv = idesc_bf16(128, D, 1);
      // descriptor words built once; inside the loops an operand is addressed by adding to the low word
      const DescWords q_d = desc_words_sw128(smem_u32(Qs), 16, 1024), k_d = desc_words_sw128(smem_u32(Ks), 16, 1024),
                      p_d = desc_words_sw128(smem_u32(Ps), 16, 1024), v_d = desc_words_sw128(smem_u32(Vs), 8192, 1024);
      auto issue_qk = [&](int st, int s) {   // st: K/V ring stage of the entry, s: its S buffer
        const uint32_t kb = k_d.lo + st * (KVBYTES >> 4);
        mma_ss_w<false>(tS + s * 64, q_d.lo, q_d.hi, kb, k_d.hi, idesc_qk);
#pragma unroll
        for (int kk = 1; kk < D / 16; ++kk)
          mma_ss_w<true>(tS + s * 64, q_d.lo + (((kk >> 2) * 16384 + (kk & 3) * 32) >> 4), q_d.hi,
                         kb + (((kk >> 2) * 8192 + (kk & 3) * 32) >> 4), k_d.hi, idesc_qk);
        mma_commit(&s_full[s]);
      };
      bool ok = mbar_wait(&kv_full[0], 0);
      if (ok) {
        tc_fence_after();
        issue_qk(0, 0);
      }
      int st = 0;                 // ring stage of entry i
      int st1 = 0, ph1 = 0;       // ring stage and phase of entry i + 1
      for (int i = 0; ok && i < n; ++i) {
        const int s = i & 1, u = i >> 1;
        if (abort_s) break;
        if (++st1 == NST) { st1 = 0; ph1 ^= 1; }
        if (i + 1 < n) {
          ok = mbar_wait(&kv_full[st1], ph1);
          if (!ok) break;
          tc_fence_after();
          issue_qk(st1, s ^ 1);
        }
        ok = mbar_wait(&p_full[s], u & 1);
        if (!ok) break;
        tc_fence_after();
        {
          const uint32_t a0 = p_d.lo + s * (16384 >> 4), b0 = v_d.lo + st * (KVBYTES >> 4);
          mma_ss_wr(tO, a0, p_d.hi, b0, v_d.hi, idesc_pv, i > 0 ? 1u : 0u);
#pragma unroll
          for (int kk = 1; kk < 4; ++kk)
            mma_ss_w<true>(tO, a0 + ((kk * 32) >> 4), p_d.hi, b0 + ((kk * 2048) >> 4), v_d.hi, idesc_pv);
        }
        mma_commit(&pv_done[s]);
        mma_commit(&kv_free[st]);
        st = st1;
      }
      if (ok) mma_commit(&all_done);  // epilogue barrier for both row warpgroups
      if (!ok) { abort_s = 1; atomicExch(&g_device_status, 102); }
    }
  } else {
    // =============================== softmax rows ===============================================
    const float scale_log2 = p.scale * kLog2e;
    const float slope = p.slope ? p.slope[hq] : 0.f;
    int ptr = 0;
    int cur = (nvalid > 0) ? __ldg(ids) : 0x7fffffff;       // next unconsumed id and its weight are held
    float cur_w = (nvalid > 0) ? to_f(wrow[0]) : 0.f;       // one step ahead, so their loads are not waited on
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    bool ok = true;
    for (int i = wg; i < n; i += 2) {
      const int s = i & 1, u = i >> 1;
      const int c = union_s[i];
      float wsum = 0.f;
      bool owner = false;
      if (!unsorted) {
        while (cur < c) {  // ids belonging to the other warpgroup's entries
          ++ptr;
          cur = (ptr < nvalid) ? __ldg(ids + ptr) : 0x7fffffff;
          cur_w = (ptr < nvalid) ? to_f(wrow[ptr]) : 0.f;
        }
        while (cur == c) {
          owner = true;
          wsum += cur_w;
          ++ptr;
          cur = (ptr < nvalid) ? __ldg(ids + ptr) : 0x7fffffff;
          cur_w = (ptr < nvalid) ? to_f(wrow[ptr]) : 0.f;
        }
      } else {
        for (int k = 0; k < nvalid; ++k)
          if (__ldg(ids + k) == c) { owner = true; wsum += to_f(wrow[k]); }
      }
      ok = mbar_wait(&s_full[s], u & 1);
      if (i >= 2) ok = mbar_wait(&pv_done[s], (u - 1) & 1) && ok;
      ok = __all_sync(0xffffffffu, ok) && !abort_s;
      if (!ok) break;
      tc_fence_after();
      float sv[64];
      tmem_ld32(tS + lane_base + s * 64, sv);
      tmem_ld32(tS + lane_base + s * 64 + 32, sv + 32);
      tmem_ld_wait();
      uint8_t* prow = Ps + s * 16384;
      if (owner) {
        if (slope != 0.f) {
#pragma unroll
          for (int j = 0; j < 62; ++j) sv[j] -= slope * (float)(62 - j);
        }
        if (p.mask_last) sv[63] = -CUDART_INF_F;
        float m4[4] = {sv[0], sv[1], sv[2], sv[3]};   // interleaved partial reductions (short chains)
#pragma unroll
        for (int j = 4; j < 64; ++j) m4[j & 3] = fmaxf(m4[j & 3], sv[j]);
        const float m = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
        const float mb = m * scale_log2;
        float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < 64; ++j) {
          sv[j] = ex2(fmaf(sv[j], scale_log2, -mb));
          s4[j & 3] += sv[j];
        }
        const float sum = (s4[0] + s4[1]) + (s4[2] + s4[3]);
        const float f = wsum / sum;
#pragma unroll
        for (int c8 = 0; c8 < 8; ++c8) {
          __nv_bfloat162 hh[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) hh[e] = __floats2bfloat162_rn(sv[c8 * 8 + 2 * e] * f, sv[c8 * 8 + 2 * e + 1] * f);
          *reinterpret_cast<uint4*>(prow + sw128_off(r, c8)) = *reinterpret_cast<uint4*>(hh);
        }
      } else {
#pragma unroll
        for (int c8 = 0; c8 < 8; ++c8) *reinterpret_cast<uint4*>(prow + sw128_off(r, c8)) = make_uint4(0u, 0u, 0u, 0u);
      }
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(&p_full[s]);
    }
    // ---- epilogue: O row -> bf16 -> global ---------------------------------------------------------
    if (ok && n > 0) {
      ok = mbar_wait(&all_done, 0);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok && lane == 0) { abort_s = 1; atomicExch(&g_device_status, 103); }
    } else if (!ok && lane == 0) {
      abort_s = 1;
      atomicExch(&g_device_status, 104);
    }
    bf16* orow = static_cast<bf16*>(p.o) + (((int64_t)b * p.L + (valid ? t : 0)) * p.h_q + hq) * D;
    if (ok) tc_fence_after();
#pragma unroll
    for (int cb = wg; cb < D / 32; cb += 2) {  // each warpgroup stores half of the columns
      float ov[32];
      if (ok && n > 0) {
        tmem_ld32(tO + lane_base + cb * 32, ov);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) ov[j] = 0.f;
      }
      if (valid) {
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) {
          __nv_bfloat162 hh[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) hh[e] = __floats2bfloat162_rn(ov[c8 * 8 + 2 * e], ov[c8 * 8 + 2 * e + 1]);
          *reinterpret_cast<uint4*>(orow + cb * 32 + c8 * 8) = *reinterpret_cast<uint4*>(hh);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 8) tmem_dealloc(tmem, 256);
}


// =================================================================================================
// Backward, two atomic-free passes over the same (128-row query block, chunk) pairs as the forward:
//   pass "dq"  (query-major, one CTA per query block): dQ accumulates in TMEM over the block's union
//              list; dW is written per (row, slot).  It also stores the block's union bitmap and its
//              "all lists ascending" flag in the workspace for the second pass.
//   pass "dkv" (chunk-major, one CTA per chunk): walks the query blocks whose bitmap holds the chunk;
//              dK and dV of the chunk accumulate in TMEM (M = 64 accumulators) and are written once.
// Per pair both passes recompute S = Q K^T and dP = dO V^T on the tensor cores; one thread per row
// forms P, dw = sum_j P_j dP_j, dS = scale w P (dP - dw) (ops/hils_fwd_bwd_head.py:651-757).
// =================================================================================================

struct BwdWs {
  uint32_t* bitmap;  // [B*h_kv][nblk][nwords]  union bitmap of each query block
  uint16_t* wtab;    // [B*h_kv][nblk][umax][128]  bf16 weight of (block, union entry, row); kNotOwner when the
                     // row did not select that chunk.  Written by the dq pass, read by the dkv pass.
  int umax;
};
constexpr uint16_t kNotOwner = 0x7FC1;  // a bf16 NaN pattern
constexpr int kMaxMaskWords = 32;       // ownership bit masks are kept for unions of up to 1024 chunks

template <int D>
__global__ void __launch_bounds__(kBwdThreads, 1) sparse_bwd_dq_tc_kernel(SparseParams p, BwdWs ws,
                                                                          const __grid_constant__ CUtensorMap tmK,
                                                                          const __grid_constant__ CUtensorMap tmV) {
  constexpr int DB = D / 64;
  constexpr int QBYTES = DB * 16384;
  constexpr int KVBYTES = DB * 8192;
  // S/dP accumulator buffers in TMEM and K/V ring depth.  With three accumulator buffers the products of
  // entry i+2 are issued as soon as entry i-1 has been consumed, one full entry ahead of the warpgroup
  // that will read them, so that warpgroup never waits on the tensor pipe; the ring then has to hold the
  // entries i-1 .. i+2 plus the loads in flight.  D = 128 has shared memory for three stages only and
  // keeps two buffers (products issued one entry ahead).
  constexpr int NSB = (D == 64) ? 3 : 2;
  constexpr int NST = (D == 64) ? 6 : 3;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* Qs = smem;
  uint8_t* dOs = Qs + QBYTES;
  uint8_t* Ks = dOs + QBYTES;            // NST stages
  uint8_t* Vs = Ks + NST * KVBYTES;      // NST stages
  uint8_t* dSs = Vs + NST * KVBYTES;       // 2 x [128 x 64] bf16
  int* union_s = reinterpret_cast<int*>(dSs + 2 * 16384);
  const int nchunk = p.T / 64;
  const int nwords = (nchunk + 31) >> 5;
  const int G = p.h_q / p.h_kv, QB = 128 / G;
  const int umax = min(nchunk, QB * p.K);
  uint32_t* bitmap_s = reinterpret_cast<uint32_t*>(union_s + umax);
  // ownership of the union entries: word w of row r (at own_s[w * 128 + r]) has bit e set when the row selected
  // entry 32 w + e; pref_s[w] = number of union entries below chunk 32 w.  Present when the shape leaves room.
  const int nmw = (umax + 31) >> 5;
  const bool have_mask = nmw <= kMaxMaskWords;
  int* pref_s = reinterpret_cast<int*>(bitmap_s + nwords);
  uint32_t* own_s = reinterpret_cast<uint32_t*>(pref_s + nwords);

  __shared__ uint64_t kv_full[6], kv_free[6], sdp_full[3], ds_full[2], dq_done[2], all_done;
  __shared__ uint32_t tmem_base_s;
  __shared__ int n_union_s, warp_tot_s[4];
  __shared__ volatile int abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nblk = gridDim.x;
  const int blk = nblk - 1 - blockIdx.x;
  const int q0 = blk * QB, h = blockIdx.y, b = blockIdx.z;

  if (tid == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&ds_full[s], 128);
      mbar_init(&dq_done[s], 1);
    }
    for (int s = 0; s < NSB; ++s) mbar_init(&sdp_full[s], 1);
    for (int st = 0; st < NST; ++st) {
      mbar_init(&kv_full[st], 1);
      mbar_init(&kv_free[st], 1);
    }
    mbar_init(&all_done, 1);
    mbar_init_fence();
    abort_s = 0;
  }
  if (warp == 8) tmem_alloc(&tmem_base_s, 512);
  for (int w = tid; w < nwords; w += kBwdThreads) bitmap_s[w] = 0u;
  __syncthreads();

  // rows: two warpgroups (threads 0..127 and 128..255) each own all 128 rows and alternate over the
  // union entries (warpgroup w takes entries w, w+2, ... and the buffers of stage w)
  const int r = tid & 127, wg = tid >> 7;
  const int ql = r / G, g = r % G, t = q0 + ql;
  const bool is_row = tid < 256, is_loader = tid < 128;
  const bool valid = is_row && t < p.L;
  const int hq = h * G + g;
  const int64_t rowi = ((int64_t)b * p.L + (valid ? t : 0)) * p.h_q + hq;
  const int32_t* ids = p.idx + (((int64_t)b * p.L + (valid ? t : 0)) * p.h_kv + h) * p.K;
  const bf16* wrow = static_cast<const bf16*>(p.w) + rowi * p.num_weights;
  bf16* dwrow = static_cast<bf16*>(p.d_w) + rowi * p.num_weights;
  int nvalid = 0, my_unsorted = 0;
  if (is_loader) {
    const bf16* qrow = static_cast<const bf16*>(p.q) + rowi * D;
    const bf16* dorow = static_cast<const bf16*>(p.d_o) + rowi * D;
#pragma unroll
    for (int c = 0; c < D / 8; ++c) {
      uint4 x = make_uint4(0u, 0u, 0u, 0u), y = make_uint4(0u, 0u, 0u, 0u);
      if (valid) {
        x = *reinterpret_cast<const uint4*>(qrow + c * 8);
        y = *reinterpret_cast<const uint4*>(dorow + c * 8);
      }
      *reinterpret_cast<uint4*>(Qs + (c >> 3) * 16384 + sw128_off(r, c & 7)) = x;
      *reinterpret_cast<uint4*>(dOs + (c >> 3) * 16384 + sw128_off(r, c & 7)) = y;
    }
    if (valid)
      for (int k = 0; k < p.num_weights; ++k) dwrow[k] = __float2bfloat16_rn(0.f);
  }
  if (valid) {
    int prev = -1;
    for (int k = 0; k < p.K; ++k) {
      const int id = __ldg(ids + k);
      if (id < 0) break;
      ++nvalid;
      if (id <= prev) my_unsorted = 1;   // descending or repeated ids: the general path below
      prev = id;
      if (is_loader && g == 0 && id < nchunk) atomicOr(&bitmap_s[id >> 5], 1u << (id & 31));
    }
  }
  const int unsorted = __syncthreads_or(my_unsorted);
  {
    const int64_t bh = (int64_t)b * p.h_kv + h;
    for (int w = tid; w < nwords; w += kBwdThreads) ws.bitmap[(bh * nblk + blk) * nwords + w] = bitmap_s[w];
    const int wpt = (nwords + 127) / 128;
    int cnt = 0;
    if (is_loader)
      for (int w = tid * wpt; w < min(nwords, (tid + 1) * wpt); ++w) cnt += __popc(bitmap_s[w]);
    int inc = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int nn = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += nn;
    }
    if (is_loader && lane == 31) warp_tot_s[warp] = inc;
    __syncthreads();
    if (is_loader) {
      int base = inc - cnt;
      for (int w = 0; w < warp; ++w) base += warp_tot_s[w];
      for (int w = tid * wpt; w < min(nwords, (tid + 1) * wpt); ++w) {
        uint32_t bits = bitmap_s[w];
        pref_s[w] = base;
        while (bits) {
          const int bpos = __ffs(bits) - 1;
          bits &= bits - 1;
          if (base < umax) union_s[base] = w * 32 + bpos;
          ++base;
        }
      }
      if (tid == 127) n_union_s = min(base, umax);
    }
  }
  const bool fast_own = have_mask && !unsorted;
  if (fast_own) {
    __syncthreads();   // pref_s complete
    if (is_loader) {
      for (int w = 0; w < nmw; ++w) own_s[w * 128 + r] = 0u;
      for (int k = 0; k < nvalid; ++k) {
        const int id = __ldg(ids + k);
        if (id < nchunk) {
          const int pos = pref_s[id >> 5] + __popc(bitmap_s[id >> 5] & ((1u << (id & 31)) - 1u));
          own_s[(pos >> 5) * 128 + r] |= 1u << (pos & 31);
        }
      }
    }
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const int n = n_union_s;
  const uint32_t tmem = tmem_base_s;
  const uint32_t tdQ = tmem + NSB * 128;

  if (warp == 9) {
    if (lane == 0) {
      for (int i = 0; i < n; ++i) {
        const int s = i % NST;
        if (abort_s) break;
        if (i >= NST && !mbar_wait(&kv_free[s], ((i / NST) - 1) & 1)) { abort_s = 1; atomicExch(&g_device_status, 201); break; }
        const int c = union_s[i];
        mbar_expect_tx(&kv_full[s], 2 * KVBYTES);
#pragma unroll
        for (int db = 0; db < DB; ++db) {
          tma_load_2d(Ks + s * KVBYTES + db * 8192, &tmK, &kv_full[s], h * D + db * 64, b * p.T + c * 64);
          tma_load_2d(Vs + s * KVBYTES + db * 8192, &tmV, &kv_full[s], h * D + db * 64, b * p.T + c * 64);
        }
      }
    }
  } else if (warp == 8) {
    if (lane == 0 && n > 0) {
      constexpr uint32_t idesc_s = idesc_bf16(128, 64, 0);
      constexpr uint32_t idesc_dq = idesc_bf16(128, D, 1);
      // descriptor words built once; inside the loops an operand is addressed by adding to the low word
      const DescWords q_d = desc_words_sw128(smem_u32(Qs), 16, 1024), do_d = desc_words_sw128(smem_u32(dOs), 16, 1024),
                      k_d = desc_words_sw128(smem_u32(Ks), 16, 1024), v_d = desc_words_sw128(smem_u32(Vs), 16, 1024),
                      ds_d = desc_words_sw128(smem_u32(dSs), 16, 1024), kmn_d = desc_words_sw128(smem_u32(Ks), 8192, 1024);
      auto issue_sdp = [&](int st, int sb) {   // st: K/V ring stage of the entry, sb: its S/dP buffer
        const uint32_t kb = k_d.lo + st * (KVBYTES >> 4), vb = v_d.lo + st * (KVBYTES >> 4);
        const uint32_t ts = tmem + sb * 128;
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
        mma_commit(&sdp_full[sb]);
      };
      // entries 0 .. NSB-2 are issued before the loop; iteration i then issues entry e = i + NSB - 1, whose
      // buffer was last read for entry i - 1 (consumed: its dS arrival was waited for in iteration i - 1)
      bool ok = true;
      int ste = 0, phe = 0, sbe = 0;   // ring stage, ring phase and accumulator buffer of the next entry to issue
      auto issue_next = [&]() {
        ok = mbar_wait(&kv_full[ste], phe);
        if (!ok) return;
        tc_fence_after();
        issue_sdp(ste, sbe);
        if (++ste == NST) { ste = 0; phe ^= 1; }
        if (++sbe == NSB) sbe = 0;
      };
      for (int e = 0; ok && e < NSB - 1 && e < n; ++e) issue_next();
      int st = 0;                      // ring stage of entry i
      for (int i = 0; ok && i < n; ++i) {
        const int s = i & 1, u = i >> 1;
        if (abort_s) break;
        if (i + NSB - 1 < n) {
          issue_next();
          if (!ok) break;
        }
        ok = mbar_wait(&ds_full[s], u & 1);
        if (!ok) break;
        tc_fence_after();
        {
          const uint32_t a0 = ds_d.lo + s * (16384 >> 4), b0 = kmn_d.lo + st * (KVBYTES >> 4);
          mma_ss_wr(tdQ, a0, ds_d.hi, b0, kmn_d.hi, idesc_dq, i > 0 ? 1u : 0u);
#pragma unroll
          for (int kk = 1; kk < 4; ++kk)
            mma_ss_w<true>(tdQ, a0 + ((kk * 32) >> 4), ds_d.hi, b0 + ((kk * 2048) >> 4), kmn_d.hi, idesc_dq);
        }
        mma_commit(&dq_done[s]);
        mma_commit(&kv_free[st]);
        if (++st == NST) st = 0;
      }
      // both row warpgroups wait on this for the epilogue: a parity wait on a stage barrier could be
      // satisfied by an older phase for the warpgroup that did not take the last entry
      if (ok) mma_commit(&all_done);
      if (!ok) { abort_s = 1; atomicExch(&g_device_status, 202); }
    }
  } else {
    const float scale_log2 = p.scale * kLog2e;
    const float slope = p.slope ? p.slope[hq] : 0.f;
    int ptr = 0;
    int cur = (nvalid > 0) ? __ldg(ids) : 0x7fffffff;       // next unconsumed id and its weight are held
    float cur_w = (nvalid > 0) ? to_f(wrow[0]) : 0.f;       // one step ahead, so their loads are not waited on
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    bool ok = true;
    int sb = wg, sph = 0;   // accumulator buffer of entry i (i % NSB) and the phase of its barrier ((i / NSB) & 1)
    int own_w = 0, own_below = 0;                       // current ownership word and the row's slots in the words below it
    uint32_t own_bits = fast_own ? own_s[r] : 0u;
    for (int i = wg; i < n; i += 2) {
      const int s = i & 1, u = i >> 1;
      const int c = union_s[i];
      float wsum = 0.f;
      bool owner = false;
      int k_first = 0, k_last = 0;
      if (fast_own) {
        // ids strictly ascending: the slot of entry i is the number of the row's entries below it
        while (own_w < (i >> 5)) {
          own_below += __popc(own_bits);
          ++own_w;
          own_bits = own_s[own_w * 128 + r];
        }
        owner = (own_bits >> (i & 31)) & 1u;
        k_first = own_below + __popc(own_bits & ((1u << (i & 31)) - 1u));
        k_last = k_first + (owner ? 1 : 0);
        if (owner) wsum = to_f(wrow[k_first]);
      } else if (!unsorted) {
        while (cur < c) {  // ids consumed by the other warpgroup's entries
          ++ptr;
          cur = (ptr < nvalid) ? __ldg(ids + ptr) : 0x7fffffff;
          cur_w = (ptr < nvalid) ? to_f(wrow[ptr]) : 0.f;
        }
        k_first = ptr;
        while (cur == c) {
          owner = true;
          wsum += cur_w;
          ++ptr;
          cur = (ptr < nvalid) ? __ldg(ids + ptr) : 0x7fffffff;
          cur_w = (ptr < nvalid) ? to_f(wrow[ptr]) : 0.f;
        }
        k_last = ptr;
      } else {
        for (int k = 0; k < nvalid; ++k)
          if (__ldg(ids + k) == c) { owner = true; wsum += to_f(wrow[k]); }
      }
      ok = mbar_wait(&sdp_full[sb], sph);
      ok = __all_sync(0xffffffffu, ok) && !abort_s;
      if (!ok) break;
      tc_fence_after();
      float sv[64], dp[64];
      const uint32_t tsd = tmem + lane_base + sb * 128;
      tmem_ld32(tsd, sv);
      tmem_ld32(tsd + 32, sv + 32);
      tmem_ld_wait();
      tmem_ld32(tsd + 64, dp);        // in flight while the S row is exponentiated
      tmem_ld32(tsd + 96, dp + 32);
      float esum = 1.f;
      if (owner) esum = bwd_row_exp(sv, scale_log2, slope, p.mask_last);
      tmem_ld_wait64(dp);
      sb += 2;
      if (sb >= NSB) { sb -= NSB; sph ^= 1; }
      {
        const __nv_bfloat16 wb = __float2bfloat16_rn(wsum);
        ws.wtab[((((int64_t)b * p.h_kv + h) * nblk + blk) * ws.umax + i) * 128 + r] =
            owner ? *reinterpret_cast<const uint16_t*>(&wb) : kNotOwner;
      }
      // the dS buffer was last read by the dQ product of entry i - 2
      if (i >= 2) {
        ok = mbar_wait(&dq_done[s], (u - 1) & 1);
        ok = __all_sync(0xffffffffu, ok) && !abort_s;
        if (!ok) break;
      }
      uint8_t* dsrow = dSs + s * 16384;
      if (owner) {
        const float dw = bwd_row_grad<false>(sv, dp, esum, wsum, p.scale);
        store_row_bf16_sw128(dsrow, r, sv);
        const bf16 dwb = __float2bfloat16_rn(dw);
        if (!unsorted) {
          for (int k = k_first; k < k_last; ++k) dwrow[k] = dwb;
        } else {
          for (int k = 0; k < nvalid; ++k)
            if (__ldg(ids + k) == c) dwrow[k] = dwb;
        }
      } else {
        store_row_zero_sw128(dsrow, r);
      }
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(&ds_full[s]);
    }
    if (ok && n > 0) {
      ok = mbar_wait(&all_done, 0);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok && lane == 0) { abort_s = 1; atomicExch(&g_device_status, 203); }
    } else if (!ok && lane == 0) {
      abort_s = 1;
      atomicExch(&g_device_status, 204);
    }
    bf16* orow = static_cast<bf16*>(p.d_q) + rowi * D;
    if (ok) tc_fence_after();
#pragma unroll
    for (int cb = wg; cb < D / 32; cb += 2) {  // each warpgroup writes half of the columns
      float ov[32];
      if (ok && n > 0) {
        tmem_ld32(tdQ + lane_base + cb * 32, ov);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) ov[j] = 0.f;
      }
      if (valid) {
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) {
          __nv_bfloat162 hh[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) hh[e] = __floats2bfloat162_rn(ov[c8 * 8 + 2 * e], ov[c8 * 8 + 2 * e + 1]);
          *reinterpret_cast<uint4*>(orow + cb * 32 + c8 * 8) = *reinterpret_cast<uint4*>(hh);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 8) tmem_dealloc(tmem, 512);
}

template <int D>
__global__ void __launch_bounds__(kBwdThreads, 1) sparse_bwd_dkv_tc_kernel(SparseParams p, BwdWs ws, int nblk,
                                                                           const __grid_constant__ CUtensorMap tmK,
                                                                           const __grid_constant__ CUtensorMap tmV,
                                                                           const __grid_constant__ CUtensorMap tmQ,
                                                                           const __grid_constant__ CUtensorMap tmdO) {
  constexpr int DB = D / 64;
  constexpr int QBYTES = DB * 16384;
  constexpr int KVBYTES = DB * 8192;
  constexpr int NDS = (D == 64) ? 2 : 1;   // buffers for the dS / wP tiles
  constexpr int NQ = (D == 64) ? 3 : 2;    // Q / dO ring depth
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* Qs = smem;                      // NQ stages
  uint8_t* dOs = Qs + NQ * QBYTES;         // NQ stages
  uint8_t* Ks = dOs + NQ * QBYTES;
  uint8_t* Vs = Ks + KVBYTES;
  uint8_t* dSs = Vs + KVBYTES;             // NDS x 16 KB
  uint8_t* Pws = dSs + NDS * 16384;        // NDS x 16 KB
  int* list_s = reinterpret_cast<int*>(Pws + NDS * 16384);   // owning query blocks
  int* pos_s = list_s + nblk;                                // position of this chunk in each block's union list

  __shared__ uint64_t kv_full, qdo_full[4], qdo_free[4], sdp_full[2], dsp_full[2], dkv_done[2], all_done;
  __shared__ uint32_t tmem_base_s;
  __shared__ int m_s, warp_tot_s[4];
  __shared__ volatile int abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int nchunk = p.T / 64, nwords = (nchunk + 31) >> 5;
  const int G = p.h_q / p.h_kv, QB = 128 / G;
  const int64_t bh = (int64_t)b * p.h_kv + h;

  if (tid == 0) {
    mbar_init(&kv_full, 1);
    mbar_init(&all_done, 1);
    for (int st = 0; st < NQ; ++st) {
      mbar_init(&qdo_full[st], 1);
      mbar_init(&qdo_free[st], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sdp_full[s], 1);
      mbar_init(&dsp_full[s], 128);
      mbar_init(&dkv_done[s], 1);
    }
    mbar_init_fence();
    abort_s = 0;
  }
  if (warp == 8) tmem_alloc(&tmem_base_s, 512);
  // ---- query blocks that selected this chunk, ascending ----------------------------------------
  {
    const int per = (nblk + 127) / 128;
    int cnt = 0;
    if (tid < 128)
      for (int j = tid * per; j < min(nblk, (tid + 1) * per); ++j)
        cnt += (ws.bitmap[(bh * nblk + j) * nwords + (c >> 5)] >> (c & 31)) & 1u;
    int inc = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int nn = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += nn;
    }
    if (tid < 128 && lane == 31) warp_tot_s[warp] = inc;
    __syncthreads();
    if (tid < 128) {
      int base = inc - cnt;
      for (int w = 0; w < warp; ++w) base += warp_tot_s[w];
      for (int j = tid * per; j < min(nblk, (tid + 1) * per); ++j)
        if ((ws.bitmap[(bh * nblk + j) * nwords + (c >> 5)] >> (c & 31)) & 1u) {
          const uint32_t* bm = ws.bitmap + (bh * nblk + j) * nwords;
          int pos = __popc(bm[c >> 5] & ((1u << (c & 31)) - 1u));
          for (int w = 0; w < (c >> 5); ++w) pos += __popc(bm[w]);
          list_s[base] = j;
          pos_s[base] = pos;
          ++base;
        }
      if (tid == 127) m_s = base;
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const int m = m_s;
  const uint32_t tmem = tmem_base_s;
  const uint32_t tdK = tmem + 256, tdV = tmem + 256 + D;

  if (warp == 9) {
    if (lane == 0 && m > 0) {
      mbar_expect_tx(&kv_full, 2 * KVBYTES);
#pragma unroll
      for (int db = 0; db < DB; ++db) {
        tma_load_2d(Ks + db * 8192, &tmK, &kv_full, h * D + db * 64, b * p.T + c * 64);
        tma_load_2d(Vs + db * 8192, &tmV, &kv_full, h * D + db * 64, b * p.T + c * 64);
      }
      for (int j = 0; j < m; ++j) {
        const int s = j % NQ;
        if (abort_s) break;
        if (j >= NQ && !mbar_wait(&qdo_free[s], ((j / NQ) - 1) & 1)) { abort_s = 1; atomicExch(&g_device_status, 301); break; }
        const int blk = list_s[j];
        mbar_expect_tx(&qdo_full[s], 2 * QBYTES);
#pragma unroll
        for (int db = 0; db < DB; ++db) {
          tma_load_3d(Qs + s * QBYTES + db * 16384, &tmQ, &qdo_full[s], db * 64, h * G, b * p.L + blk * QB);
          tma_load_3d(dOs + s * QBYTES + db * 16384, &tmdO, &qdo_full[s], db * 64, h * G, b * p.L + blk * QB);
        }
      }
    }
  } else if (warp == 8) {
    if (lane == 0 && m > 0) {
      constexpr uint32_t idesc_s = idesc_bf16(128, 64, 0);
      constexpr uint32_t idesc_dkv = idesc_bf16(64, D, 1, 1);
      // D = 64: dK and dV of a block come from ONE product of M = 128, N = 128: A = [dS^T ; (wP)^T] (the
      // two tiles are 64-row blocks of an MN-major operand, NDS * 16 KB apart), B = [Q | dO] (64-column
      // blocks NQ * 16 KB apart); the diagonal blocks of the 128 x 128 accumulator are dK (rows 0..63,
      // columns 0..63) and dV (rows 64..127, columns 64..127), the off-diagonal ones are not read.  Half
      // the MMA instructions for the same operand bytes: an instruction of this size is bound by its
      // shared-memory reads either way.
      constexpr bool kStacked = (D == 64);
      constexpr uint32_t idesc_st = idesc_bf16(128, 128, 1, 1);
      const DescWords ast_d = desc_words_sw128(smem_u32(dSs), NDS * 16384, 1024),
                      bst_d = desc_words_sw128(smem_u32(Qs), NQ * QBYTES, 1024);
      // descriptor words built once (see the dq kernel); the Q / dO tiles are read K-major for S and dP and
      // MN-major (16 query rows per step) for dK and dV
      const DescWords q_d = desc_words_sw128(smem_u32(Qs), 16, 1024), do_d = desc_words_sw128(smem_u32(dOs), 16, 1024),
                      k_d = desc_words_sw128(smem_u32(Ks), 16, 1024), v_d = desc_words_sw128(smem_u32(Vs), 16, 1024),
                      qmn_d = desc_words_sw128(smem_u32(Qs), 16384, 1024), domn_d = desc_words_sw128(smem_u32(dOs), 16384, 1024),
                      ds_d = desc_words_sw128(smem_u32(dSs), 16384, 1024), pw_d = desc_words_sw128(smem_u32(Pws), 16384, 1024);
      auto issue_sdp = [&](int sq, int s) {   // sq: Q/dO ring stage of the block, s: its S/dP buffer
        const uint32_t qb = q_d.lo + sq * (QBYTES >> 4), dob = do_d.lo + sq * (QBYTES >> 4);
        const uint32_t ts = tmem + s * 128;
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
        mma_commit(&sdp_full[s]);
      };
      bool ok = mbar_wait(&kv_full, 0) && mbar_wait(&qdo_full[0], 0);
      if (ok) { tc_fence_after(); issue_sdp(0, 0); }
      int sq = 0;                 // ring stage of block j
      int sq1 = 0, ph1 = 0;       // ring stage and phase of block j + 1
      for (int j = 0; ok && j < m; ++j) {
        const int s = j & 1, u = j >> 1, sb = (NDS == 2) ? s : 0;
        if (abort_s) break;
        if (++sq1 == NQ) { sq1 = 0; ph1 ^= 1; }
        if (j + 1 < m) {
          ok = mbar_wait(&qdo_full[sq1], ph1);
          if (!ok) break;
          tc_fence_after();
          issue_sdp(sq1, s ^ 1);
        }
        ok = mbar_wait(&dsp_full[s], u & 1);
        if (!ok) break;
        tc_fence_after();
        {
          const uint32_t dsb = ds_d.lo + sb * (16384 >> 4), pwb = pw_d.lo + sb * (16384 >> 4);
          const uint32_t qb = qmn_d.lo + sq * (QBYTES >> 4), dob = domn_d.lo + sq * (QBYTES >> 4);
          if (kStacked) {
            const uint32_t a0 = ast_d.lo + sb * (16384 >> 4), b0 = bst_d.lo + sq * (QBYTES >> 4);
            mma_ss_wr(tdK, a0, ast_d.hi, b0, bst_d.hi, idesc_st, j > 0 ? 1u : 0u);
#pragma unroll
            for (int kk = 1; kk < 8; ++kk)   // 16 query rows per step
              mma_ss_w<true>(tdK, a0 + ((kk * 2048) >> 4), ast_d.hi, b0 + ((kk * 2048) >> 4), bst_d.hi, idesc_st);
          } else {
            mma_ss_wr(tdK, dsb, ds_d.hi, qb, qmn_d.hi, idesc_dkv, j > 0 ? 1u : 0u);
            mma_ss_wr(tdV, pwb, pw_d.hi, dob, domn_d.hi, idesc_dkv, j > 0 ? 1u : 0u);
#pragma unroll
            for (int kk = 1; kk < 8; ++kk) {   // 16 query rows per step
              mma_ss_w<true>(tdK, dsb + ((kk * 2048) >> 4), ds_d.hi, qb + ((kk * 2048) >> 4), qmn_d.hi, idesc_dkv);
              mma_ss_w<true>(tdV, pwb + ((kk * 2048) >> 4), pw_d.hi, dob + ((kk * 2048) >> 4), domn_d.hi, idesc_dkv);
            }
          }
        }
        mma_commit(&dkv_done[s]);
        mma_commit(&qdo_free[sq]);
        sq = sq1;
      }
      if (ok) mma_commit(&all_done);  // epilogue barrier for both row warpgroups (see the dq kernel)
      if (!ok) { abort_s = 1; atomicExch(&g_device_status, 302); }
    }
  } else {
    // two row warpgroups alternate over the query blocks (warpgroup w takes blocks w, w+2, ...)
    const int r = tid & 127, wg = tid >> 7, ql = r / G, g = r % G, hq = h * G + g;
    const float scale_log2 = p.scale * kLog2e;
    const float slope = p.slope ? p.slope[hq] : 0.f;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    bool ok = true;
    uint16_t wnext = kNotOwner;
    if (wg < m) wnext = __ldg(ws.wtab + (((bh * nblk + list_s[wg]) * ws.umax + pos_s[wg]) * 128 + r));
    for (int j = wg; j < m; j += 2) {
      const int s = j & 1, u = j >> 1, sb = j % NDS;
      // weight of this row for the chunk, looked up in the table of the dq pass; the entry of this
      // warpgroup's next block is requested now so that its latency is hidden
      const uint16_t wraw = wnext;
      if (j + 2 < m)
        wnext = __ldg(ws.wtab + (((bh * nblk + list_s[j + 2]) * ws.umax + pos_s[j + 2]) * 128 + r));
      const bool owner = wraw != kNotOwner;
      const float wsum = owner ? __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(&wraw)) : 0.f;
      ok = mbar_wait(&sdp_full[s], u & 1);
      if (j >= NDS) ok = mbar_wait(&dkv_done[(j - NDS) & 1], ((j - NDS) >> 1) & 1) && ok;
      ok = __all_sync(0xffffffffu, ok) && !abort_s;
      if (!ok) break;
      tc_fence_after();
      float sv[64], dp[64];
      tmem_ld32(tmem + lane_base + s * 128, sv);
      tmem_ld32(tmem + lane_base + s * 128 + 32, sv + 32);
      tmem_ld_wait();
      tmem_ld32(tmem + lane_base + s * 128 + 64, dp);        // in flight while the S row is exponentiated
      tmem_ld32(tmem + lane_base + s * 128 + 96, dp + 32);
      float esum = 1.f;
      if (owner) esum = bwd_row_exp(sv, scale_log2, slope, p.mask_last);
      tmem_ld_wait64(dp);
      if (owner) {
        bwd_row_grad<true>(sv, dp, esum, wsum, p.scale);
        store_row_bf16_sw128(dSs + sb * 16384, r, sv);
        store_row_bf16_sw128(Pws + sb * 16384, r, dp);
      } else {
        store_row_zero_sw128(dSs + sb * 16384, r);
        store_row_zero_sw128(Pws + sb * 16384, r);
      }
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(&dsp_full[s]);
    }
    if (ok && m > 0) {
      ok = mbar_wait(&all_done, 0);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok && lane == 0) { abort_s = 1; atomicExch(&g_device_status, 303); }
    } else if (!ok && lane == 0) {
      abort_s = 1;
      atomicExch(&g_device_status, 304);
    }
    // M = 64 accumulators: key row 16*warp + lane lives in TMEM lane 32*warp + lane, lanes 0..15 of each warp
    const int krow = 16 * (warp & 3) + lane;
    const int64_t tok = (int64_t)b * p.T + (int64_t)c * 64 + krow;
    bf16* dkrow = static_cast<bf16*>(p.d_k_out) + (tok * p.h_kv + h) * D;
    bf16* dvrow = static_cast<bf16*>(p.d_v_out) + (tok * p.h_kv + h) * D;
    if (ok) tc_fence_after();
    if (D == 64) {
      // stacked accumulator (M = 128): TMEM lane = row; rows 0..63 hold dK in columns 0..63, rows 64..127 hold
      // dV in columns 64..127.  Warps 0, 1 of a warpgroup write dK rows, warps 2, 3 dV rows; warpgroup w
      // takes the 32-column half w.
      const int wq = warp & 3;
      const bool is_v = wq >= 2;
      const int64_t tokr = (int64_t)b * p.T + (int64_t)c * 64 + 32 * (wq & 1) + lane;
      float ov[32];
      if (ok && m > 0) {
        tmem_ld32(tdK + lane_base + (is_v ? 64 : 0) + wg * 32, ov);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) ov[jj] = 0.f;
      }
      bf16* dst = static_cast<bf16*>(is_v ? p.d_v_out : p.d_k_out) + (tokr * p.h_kv + h) * D + wg * 32;
#pragma unroll
      for (int c8 = 0; c8 < 4; ++c8) {
        __nv_bfloat162 hh[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) hh[e] = __floats2bfloat162_rn(ov[c8 * 8 + 2 * e], ov[c8 * 8 + 2 * e + 1]);
        *reinterpret_cast<uint4*>(dst + c8 * 8) = *reinterpret_cast<uint4*>(hh);
      }
    } else {
      const int which = wg;  // warpgroup 0 writes dK, warpgroup 1 writes dV
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
        if (lane < 16) {
          bf16* dst = (which ? dvrow : dkrow) + cb * 32;
#pragma unroll
          for (int c8 = 0; c8 < 4; ++c8) {
            __nv_bfloat162 hh[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) hh[e] = __floats2bfloat162_rn(ov[c8 * 8 + 2 * e], ov[c8 * 8 + 2 * e + 1]);
            *reinterpret_cast<uint4*>(dst + c8 * 8) = *reinterpret_cast<uint4*>(hh);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 8) tmem_dealloc(tmem, 512);
}

static bool tc_shape_ok(const SparseParams& p) {
  const int D = p.D;
  if (p.S != 64 || p.D != p.Dv || (D != 64 && D != 128)) return false;
  const int G = p.h_q / p.h_kv;
  if (G > 128 || (128 % G) != 0) return false;
  if (p.T < 64 || p.K > 1024) return false;
  if ((int64_t)p.B * p.T >= (1ll << 31) || (int64_t)p.B * p.L >= (1ll << 31)) return false;
  return true;
}

static size_t tc_bwd_smem_dq(const SparseParams& p) {
  const int D = p.D, G = p.h_q / p.h_kv, QB = 128 / G, nchunk = p.T / 64;
  const int umax = min(nchunk, QB * p.K);
  const int NST = (D == 64) ? 6 : 3;
  const size_t nmw = (size_t)(umax + 31) / 32;
  return 1024 + 2 * (size_t)(D / 64) * 16384 + 2 * (size_t)NST * (D / 64) * 8192 + 2 * 16384 + (size_t)umax * 4 +
         (size_t)((nchunk + 31) / 32) * 8 + (nmw <= (size_t)kMaxMaskWords ? nmw * 512 : 0) + 16;
}
static size_t tc_bwd_smem_dkv(const SparseParams& p, int nblk) {
  const int D = p.D, NDS = (D == 64) ? 2 : 1, NQ = (D == 64) ? 3 : 2;
  return 1024 + 2 * (size_t)NQ * (D / 64) * 16384 + 2 * (size_t)(D / 64) * 8192 + 2 * (size_t)NDS * 16384 + (size_t)nblk * 8 + 16;
}

// workspace of the tensor-core backward (0 when the shape is outside this path)
size_t sparse_bwd_tc_workspace(const SparseParams& p) {
  if (!tc_shape_ok(p)) return 0;
  const int G = p.h_q / p.h_kv, QB = 128 / G, nblk = ceil_div(p.L, QB), nchunk = p.T / 64;
  if (tc_bwd_smem_dq(p) > 220 * 1024 || tc_bwd_smem_dkv(p, nblk) > 220 * 1024) return 0;
  const size_t nw = (size_t)((nchunk + 31) / 32);
  const size_t umax = (size_t)min(nchunk, QB * p.K);
  const size_t tab = (size_t)p.B * p.h_kv * nblk * umax * 128 * sizeof(uint16_t);
  if (tab > ((size_t)16 << 30)) return 0;   // ownership table beyond 16 GiB: shape left to the generic path
  return (size_t)p.B * p.h_kv * nblk * nw * 4 + 256 + tab;
}

int sparse_bwd_tc_launch(const SparseParams& p, void* d_k, void* d_v, void* workspace, cudaStream_t st) {
  if (sparse_bwd_tc_workspace(p) == 0) return HILS_ERR_UNSUPPORTED;
  if (((uintptr_t)p.q | (uintptr_t)p.k | (uintptr_t)p.v | (uintptr_t)p.d_o | (uintptr_t)p.d_q | (uintptr_t)d_k |
       (uintptr_t)d_v) & 15)
    return HILS_ERR_UNSUPPORTED;
  const int D = p.D, G = p.h_q / p.h_kv, QB = 128 / G, nblk = ceil_div(p.L, QB), nchunk = p.T / 64;
  const size_t nw = (size_t)((nchunk + 31) / 32);
  BwdWs ws;
  ws.bitmap = static_cast<uint32_t*>(workspace);
  ws.wtab = reinterpret_cast<uint16_t*>(reinterpret_cast<uint8_t*>(workspace) +
                                        (((size_t)p.B * p.h_kv * nblk * nw * 4 + 255) & ~(size_t)255));
  ws.umax = min(nchunk, QB * p.K);
  SparseParams pp = p;
  pp.d_k_out = d_k;
  pp.d_v_out = d_v;
  CUtensorMap tmK, tmV, tmQ, tmdO;
  if (int rc = make_tmap_bf16_rows(&tmK, p.k, (uint64_t)p.B * p.T, (uint64_t)p.h_kv * D, (uint64_t)p.h_kv * D, 64)) return rc;
  if (int rc = make_tmap_bf16_rows(&tmV, p.v, (uint64_t)p.B * p.T, (uint64_t)p.h_kv * D, (uint64_t)p.h_kv * D, 64)) return rc;
  if (int rc = make_tmap_bf16_thd(&tmQ, p.q, (uint64_t)p.B * p.L, p.h_q, D, G, QB)) return rc;
  if (int rc = make_tmap_bf16_thd(&tmdO, p.d_o, (uint64_t)p.B * p.L, p.h_q, D, G, QB)) return rc;
  if (p.T % 64 != 0) {  // tokens after the last full chunk belong to no chunk: their gradients are zero
    cudaMemsetAsync(d_k, 0, (size_t)p.B * p.T * p.h_kv * D * 2, st);
    cudaMemsetAsync(d_v, 0, (size_t)p.B * p.T * p.h_kv * D * 2, st);
  }
  const size_t smem_dq = tc_bwd_smem_dq(p), smem_dkv = tc_bwd_smem_dkv(p, nblk);
  dim3 grid_q(nblk, p.h_kv, p.B), grid_c(nchunk, p.h_kv, p.B);
  if (D == 64) {
    cudaFuncSetAttribute(sparse_bwd_dq_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_dq);
    cudaFuncSetAttribute(sparse_bwd_dkv_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_dkv);
    sparse_bwd_dq_tc_kernel<64><<<grid_q, kBwdThreads, smem_dq, st>>>(pp, ws, tmK, tmV);
    sparse_bwd_dkv_tc_kernel<64><<<grid_c, kBwdThreads, smem_dkv, st>>>(pp, ws, nblk, tmK, tmV, tmQ, tmdO);
  } else {
    cudaFuncSetAttribute(sparse_bwd_dq_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_dq);
    cudaFuncSetAttribute(sparse_bwd_dkv_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_dkv);
    sparse_bwd_dq_tc_kernel<128><<<grid_q, kBwdThreads, smem_dq, st>>>(pp, ws, tmK, tmV);
    sparse_bwd_dkv_tc_kernel<128><<<grid_c, kBwdThreads, smem_dkv, st>>>(pp, ws, nblk, tmK, tmV, tmQ, tmdO);
  }
  HILS_LAUNCH_CHECK("sparse_attn_bwd (tensor-core path)");
  return HILS_OK;
}

// Returns HILS_ERR_UNSUPPORTED (without setting an error text) when the shape is outside this path.
int sparse_fwd_tc_launch(const SparseParams& p, cudaStream_t st) {
  const int D = p.D;
  if (p.S != 64 || p.D != p.Dv || (D != 64 && D != 128)) return HILS_ERR_UNSUPPORTED;
  const int G = p.h_q / p.h_kv;
  if (G > 128 || (128 % G) != 0) return HILS_ERR_UNSUPPORTED;
  if (p.T < 64 || p.K > 1024) return HILS_ERR_UNSUPPORTED;
  if (((uintptr_t)p.q | (uintptr_t)p.k | (uintptr_t)p.v | (uintptr_t)p.o) & 15) return HILS_ERR_UNSUPPORTED;
  if ((int64_t)p.B * p.T >= (1ll << 31)) return HILS_ERR_UNSUPPORTED;
  const int QB = 128 / G, nchunk = p.T / 64;
  const int umax = min(nchunk, QB * p.K);
  const size_t smem = 1024 + (size_t)(D / 64) * 16384 + 2 * (size_t)kFwdStages * (D / 64) * 8192 + 2 * 16384 + (size_t)umax * 4 +
                      (size_t)((nchunk + 31) / 32) * 4 + 16;
  if (smem > 220 * 1024) return HILS_ERR_UNSUPPORTED;
  CUtensorMap tmK, tmV;
  if (int rc = make_tmap_bf16_rows(&tmK, p.k, (uint64_t)p.B * p.T, (uint64_t)p.h_kv * D, (uint64_t)p.h_kv * D, 64)) return rc;
  if (int rc = make_tmap_bf16_rows(&tmV, p.v, (uint64_t)p.B * p.T, (uint64_t)p.h_kv * D, (uint64_t)p.h_kv * D, 64)) return rc;
  dim3 grid(ceil_div(p.L, QB), p.h_kv, p.B);
  if (D == 64) {
    cudaFuncSetAttribute(sparse_fwd_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sparse_fwd_tc_kernel<64><<<grid, kBwdThreads, smem, st>>>(p, tmK, tmV);
  } else {
    cudaFuncSetAttribute(sparse_fwd_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sparse_fwd_tc_kernel<128><<<grid, kBwdThreads, smem, st>>>(p, tmK, tmV);
  }
  HILS_LAUNCH_CHECK("sparse_attn_fwd (tensor-core path)");
  return HILS_OK;
}

}  // namespace hils

namespace hils {
// device-side error word of this file's kernels (0 = none); synchronises and clears
int take_status_sparse_tc() {
  int v = 0, zero = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  if (cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));
  return v;
}
}  // namespace hils
