// Sparse chunk attention forward, query-block-major, on the 5th-generation tensor cores (tcgen05 + TMEM + TMA), bf16.
// The kernel for DENSE selections (a token selects a large share of its candidate chunks); sparse selections and the
// backward pass run chunk-major over gathered owner rows (sparse_attn_cm.cu).
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

constexpr int kFwdThreads = 320;  // 2 row warpgroups + MMA warp + TMA warp
constexpr int kFwdStages = 3;     // K/V ring depth of the forward kernel

template <int D>
__global__ void __launch_bounds__(kFwdThreads, 2) sparse_fwd_tc_kernel(SparseParams p, const __grid_constant__ CUtensorMap tmK,
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
  for (int w = tid; w < nwords; w += kFwdThreads) bitmap_s[w] = 0u;
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
    sparse_fwd_tc_kernel<64><<<grid, kFwdThreads, smem, st>>>(p, tmK, tmV);
  } else {
    cudaFuncSetAttribute(sparse_fwd_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sparse_fwd_tc_kernel<128><<<grid, kFwdThreads, smem, st>>>(p, tmK, tmV);
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
