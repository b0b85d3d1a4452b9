// Backward of the selection scores, bf16, on the warp-level tensor cores.
//
// scores[i,g,k] = scale * q[i,g] . k'[id(i,k)]  (ops/topk_head_softmax.py:1040-1092 scatters the score
// gradient into a dense (rows x N) matrix and runs two batched matrix products).  Here the dense matrix
// exists only as a 64 x 128 tile in shared memory: a CTA walks blocks of 64 (token, member) rows of one
// (batch, key head), scatters their K score gradients into the tile and multiplies
//     dq  [64 x D]  = tile     [64 x 128] . k' [128 x D]
//     dk' [128 x D] += tile^T  [128 x 64] . q  [64 x D]
// with mma.sync m16n8k16.  With a single 128-candidate tile (N <= 128) the dk' accumulators stay in
// registers over all row blocks of the CTA and leave as one fp32 vector atomic per element pair.
#include "common.cuh"

namespace hils {

struct TopkBwdMmaParams {
  const bf16* ds; const int32_t* ids; const bf16* q; const bf16* lmks;
  bf16* dq; float* dl;
  int L, N, h_kv, G, K, per_qhead;
  float scale;
};

constexpr int kBwdRows = 64;       // rows per block
constexpr int kBwdBlocks = 8;      // row blocks per CTA
constexpr int kBwdTile = 128;      // candidates per tile
constexpr int kDsStride = kBwdTile + 8;

__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int NK>   // NK = D / 16
__global__ void __launch_bounds__(256) topk_bwd_mma_kernel(TopkBwdMmaParams p) {
  constexpr int D = NK * 16, RS = D + 8, NB = D / 8, CPR = D / 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* ds_s = reinterpret_cast<bf16*>(smem_raw);                // [64][136] score gradients, dense over one tile
  bf16* k_s = ds_s + kBwdRows * kDsStride;                       // [128][RS] chunk keys of the tile
  bf16* q_s = k_s + kBwdTile * RS;                               // [64][RS] query rows of the block
  __shared__ int max_id_s;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int members = p.per_qhead ? 1 : p.G;                     // rows per token in this CTA
  const int hl = blockIdx.y;                                     // key head
  const int h = p.per_qhead ? hl / p.G : hl, g_fixed = p.per_qhead ? hl % p.G : 0;
  const int HL = p.per_qhead ? p.h_kv * p.G : p.h_kv;
  const int64_t b = blockIdx.z;
  const int n_rows = p.L * members;                              // rows of this (batch, key head)
  const int cta_row0 = blockIdx.x * kBwdRows * kBwdBlocks;
  const int ntile_all = (p.N + kBwdTile - 1) / kBwdTile;
  const bool keep_dk = ntile_all == 1;                           // dk' accumulators live across the row blocks
  const uint32_t ds32 = (uint32_t)__cvta_generic_to_shared(ds_s);
  const uint32_t k32 = (uint32_t)__cvta_generic_to_shared(k_s);
  const uint32_t q32 = (uint32_t)__cvta_generic_to_shared(q_s);

  auto row_ptrs = [&](int r, int64_t& row_index, int64_t& tok_head) {   // r: row inside this (b, head)
    const int l = r / members, gi = p.per_qhead ? g_fixed : r - l * members;
    tok_head = (b * p.L + l) * p.h_kv + h;
    row_index = tok_head * p.G + gi;
  };
  auto load_keys = [&](int c0) {
    for (int i = tid; i < kBwdTile * CPR; i += 256) {
      const int row = i / CPR, col = (i - row * CPR) * 8;
      uint4 x = make_uint4(0u, 0u, 0u, 0u);
      if (c0 + row < p.N) x = *reinterpret_cast<const uint4*>(p.lmks + ((b * p.N + c0 + row) * HL + hl) * D + col);
      *reinterpret_cast<uint4*>(k_s + row * RS + col) = x;
    }
  };
  float dk[NB][4];                                               // warp w: candidates 16w..16w+15 of the tile
#pragma unroll
  for (int nb = 0; nb < NB; ++nb)
#pragma unroll
    for (int e = 0; e < 4; ++e) dk[nb][e] = 0.f;
  auto flush_dk = [&](int c0) {
#pragma unroll
    for (int hr = 0; hr < 2; ++hr) {
      const int c = c0 + warp * 16 + (lane >> 2) + hr * 8;
      if (c < p.N) {
        float* dst = p.dl + ((b * p.N + c) * HL + hl) * D + (lane & 3) * 2;
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          const float2 v = make_float2(dk[nb][2 * hr] * p.scale, dk[nb][2 * hr + 1] * p.scale);
          if (v.x != 0.f || v.y != 0.f) atomicAdd(reinterpret_cast<float2*>(dst + nb * 8), v);
        }
      }
    }
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
      for (int e = 0; e < 4; ++e) dk[nb][e] = 0.f;
  };
  auto load_q = [&](int r0) {
    for (int i = tid; i < kBwdRows * CPR; i += 256) {
      const int row = i / CPR, col = (i - row * CPR) * 8;
      uint4 x = make_uint4(0u, 0u, 0u, 0u);
      if (r0 + row < n_rows) {
        int64_t ri, th;
        row_ptrs(r0 + row, ri, th);
        x = *reinterpret_cast<const uint4*>(p.q + ri * D + col);
      }
      *reinterpret_cast<uint4*>(q_s + row * RS + col) = x;
    }
  };
  // number of candidate tiles the block's rows reach (from its largest selected id); all threads call it
  auto block_ntile = [&](int r0) -> int {
    if (tid == 0) max_id_s = -1;
    __syncthreads();
    const int row = tid >> 2;
    int mx = -1;
    if (r0 + row < n_rows) {
      int64_t ri, th;
      row_ptrs(r0 + row, ri, th);
      for (int k = tid & 3; k < p.K; k += 4) mx = max(mx, p.ids[th * p.K + k]);
    }
    mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    if ((tid & 3) == 0 && mx >= 0) atomicMax(&max_id_s, mx);
    __syncthreads();
    const int max_id = max_id_s;
    __syncthreads();                                             // everyone has read it before the next reset
    return max_id < 0 ? 0 : min(ntile_all, max_id / kBwdTile + 1);
  };
  // dense [64 x 128] tile of the block's score gradients that fall into candidates c0..c0+127 (ends with a barrier)
  auto build_tile = [&](int r0, int c0) {
    for (int i = tid; i < kBwdRows * kDsStride / 8; i += 256) reinterpret_cast<uint4*>(ds_s)[i] = make_uint4(0u, 0u, 0u, 0u);
    __syncthreads();
    const int row = tid >> 2;                                    // scatter: four threads per row
    if (r0 + row < n_rows) {
      int64_t ri, th;
      row_ptrs(r0 + row, ri, th);
      for (int k = tid & 3; k < p.K; k += 4) {
        const int id = p.ids[th * p.K + k];
        if (id >= c0 && id < c0 + kBwdTile && id < p.N) ds_s[row * kDsStride + id - c0] = p.ds[ri * p.K + k];
      }
    }
    __syncthreads();
  };
  // dq += tile . k'     (warp w: rows 16(w&3).., d-half (w>>2))
  auto mma_dq = [&](float (&dq)[NB / 2][4]) {
    const int mrow = (warp & 3) * 16, nhalf = (warp >> 2) * (D / 2);
    const uint32_t a_addr = ds32 + (uint32_t)((mrow + (lane & 7) + ((lane >> 3) & 1) * 8) * kDsStride + (lane >> 4) * 8) * 2u;
    const uint32_t b_addr = k32 + (uint32_t)(((lane & 7) + ((lane >> 3) & 1) * 8) * RS + nhalf + ((lane >> 4) & 1) * 8) * 2u;
#pragma unroll
    for (int kk = 0; kk < kBwdTile / 16; ++kk) {
      uint32_t a[4];
      ldsm4(a, a_addr + kk * 32);
#pragma unroll
      for (int np = 0; np < NB / 4; ++np) {
        uint32_t bb[4];
        ldsm4_t(bb, b_addr + (uint32_t)(kk * 16 * RS + np * 16) * 2u);
        mma16816(dq[2 * np], a, bb[0], bb[1]);
        mma16816(dq[2 * np + 1], a, bb[2], bb[3]);
      }
    }
  };
  // dk' += tile^T . q   (warp w: candidates 16w..16w+15 of the tile)
  auto mma_dk = [&]() {
    const int mcol = warp * 16;
    const uint32_t a_addr = ds32 + (uint32_t)(((lane & 7) + ((lane >> 4) & 1) * 8) * kDsStride + mcol + ((lane >> 3) & 1) * 8) * 2u;
    const uint32_t b_addr = q32 + (uint32_t)(((lane & 7) + ((lane >> 3) & 1) * 8) * RS + ((lane >> 4) & 1) * 8) * 2u;
#pragma unroll
    for (int kk = 0; kk < kBwdRows / 16; ++kk) {
      uint32_t a[4];
      ldsm4_t(a, a_addr + (uint32_t)(kk * 16 * kDsStride) * 2u);
#pragma unroll
      for (int np = 0; np < NB / 2; ++np) {
        uint32_t bb[4];
        ldsm4_t(bb, b_addr + (uint32_t)(kk * 16 * RS + np * 16) * 2u);
        mma16816(dk[2 * np], a, bb[0], bb[1]);
        mma16816(dk[2 * np + 1], a, bb[2], bb[3]);
      }
    }
  };
  auto store_dq = [&](int r0, float (&dq)[NB / 2][4]) {
    const int mrow = (warp & 3) * 16, nhalf = (warp >> 2) * (D / 2);
#pragma unroll
    for (int hr = 0; hr < 2; ++hr) {
      const int r = r0 + mrow + (lane >> 2) + hr * 8;
      if (r < n_rows) {
        int64_t ri, th;
        row_ptrs(r, ri, th);
        bf16* dst = p.dq + ri * D + nhalf + (lane & 3) * 2;
#pragma unroll
        for (int nb = 0; nb < NB / 2; ++nb)
          *reinterpret_cast<__nv_bfloat162*>(dst + nb * 8) =
              __floats2bfloat162_rn(dq[nb][2 * hr] * p.scale, dq[nb][2 * hr + 1] * p.scale);
      }
    }
  };

  if (keep_dk) {
    // one candidate tile: its keys stay in shared memory and the dk' accumulators in registers over all row blocks
    load_keys(0);
    for (int blk = 0; blk < kBwdBlocks; ++blk) {
      const int r0 = cta_row0 + blk * kBwdRows;
      if (r0 >= n_rows) break;
      __syncthreads();                                           // previous block's tiles are consumed
      load_q(r0);
      const int ntile = block_ntile(r0);
      float dq[NB / 2][4];
#pragma unroll
      for (int nb = 0; nb < NB / 2; ++nb)
#pragma unroll
        for (int e = 0; e < 4; ++e) dq[nb][e] = 0.f;
      if (ntile > 0) {
        build_tile(r0, 0);
        mma_dq(dq);
        mma_dk();
      }
      store_dq(r0, dq);
    }
    flush_dk(0);
    return;
  }

  // Several candidate tiles.  Phase 1, row block outer: dq of a block over the tiles its rows reach.  Phase 2, tile
  // outer: dk' of a tile accumulates in registers over ALL row blocks of the CTA and leaves as atomics once per
  // (CTA, tile) - an eighth of the atomic traffic of flushing per (row block, tile).
  __shared__ int nt_s[kBwdBlocks];
  int nt_max = 0;
  for (int blk = 0; blk < kBwdBlocks; ++blk) {
    const int r0 = cta_row0 + blk * kBwdRows;
    int ntile = 0;
    if (r0 < n_rows) ntile = block_ntile(r0);
    if (tid == 0) nt_s[blk] = ntile;
    nt_max = max(nt_max, ntile);
    if (r0 >= n_rows) continue;
    float dq[NB / 2][4];
#pragma unroll
    for (int nb = 0; nb < NB / 2; ++nb)
#pragma unroll
      for (int e = 0; e < 4; ++e) dq[nb][e] = 0.f;
    for (int t = 0; t < ntile; ++t) {
      __syncthreads();                                           // the previous tile is consumed
      load_keys(t * kBwdTile);
      build_tile(r0, t * kBwdTile);
      mma_dq(dq);
    }
    store_dq(r0, dq);
  }
  __syncthreads();
  for (int t = 0; t < nt_max; ++t) {
    for (int blk = 0; blk < kBwdBlocks; ++blk) {
      const int r0 = cta_row0 + blk * kBwdRows;
      if (r0 >= n_rows || nt_s[blk] <= t) continue;
      __syncthreads();                                           // the previous block's tiles are consumed
      load_q(r0);
      build_tile(r0, t * kBwdTile);
      mma_dk();
    }
    flush_dk(t * kBwdTile);
  }
}

// -------------------------------------------------------------------------------------------------
// The same two products for several candidate tiles (N > 128) and up to 32 slots per token, software-pipelined.
// In the kernel above every (row block, tile) pair waits in turn for its key tile, for the ids and for the score
// gradients (global loads issued when they are needed) and clears the whole dense tile between block-wide barriers.
// Here a thread keeps the K/4 (id, gradient) pairs of its row in registers for as long as the block is worked on,
// the key tiles (phase 1) and the query blocks (phase 2) arrive through cp.async in two buffers one step ahead, the
// ids of the next block are loaded while the current one multiplies, and only the cells a thread scattered are cleared
// again afterwards.
// -------------------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait1() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait0() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

constexpr int kPipeSlots = 8;      // (id, gradient) pairs per thread: four threads per row, K <= 32

template <int NK>   // NK = D / 16
__global__ void __launch_bounds__(256, 2) topk_bwd_pipe_kernel(TopkBwdMmaParams p) {
  constexpr int D = NK * 16, RS = D + 8, NB = D / 8, CPR = D / 8;
  constexpr uint32_t kKeyBuf = kBwdTile * RS * 2, kQBuf = kBwdRows * RS * 2;   // bytes
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* ds_s = reinterpret_cast<bf16*>(smem_raw);                // [64][136] score gradients, dense over one tile
  unsigned char* buf = smem_raw + kBwdRows * kDsStride * 2;      // phase 1: two key tiles; phase 2: two query blocks
  __shared__ int max_id_s;
  __shared__ int nt_s[kBwdBlocks];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int members = p.per_qhead ? 1 : p.G;
  const int hl = blockIdx.y;
  const int h = p.per_qhead ? hl / p.G : hl, g_fixed = p.per_qhead ? hl % p.G : 0;
  const int HL = p.per_qhead ? p.h_kv * p.G : p.h_kv;
  const int64_t b = blockIdx.z;
  const int n_rows = p.L * members;
  const int cta_row0 = blockIdx.x * kBwdRows * kBwdBlocks;
  const int ntile_all = (p.N + kBwdTile - 1) / kBwdTile;
  const uint32_t ds32 = (uint32_t)__cvta_generic_to_shared(ds_s);
  const uint32_t buf32 = (uint32_t)__cvta_generic_to_shared(buf);
  const int KPT = p.K >> 2, srow = tid >> 2, k0 = (tid & 3) * KPT;   // this thread's slots of row srow: k0 .. k0+KPT-1

  auto row_ptrs = [&](int r, int64_t& row_index, int64_t& tok_head) {
    const int l = r / members, gi = p.per_qhead ? g_fixed : r - l * members;
    tok_head = (b * p.L + l) * p.h_kv + h;
    row_index = tok_head * p.G + gi;
  };
  auto issue_keys = [&](int c0, int which) {
    const uint32_t base = buf32 + (uint32_t)which * kKeyBuf;
    for (int i = tid; i < kBwdTile * CPR; i += 256) {
      const int row = i / CPR, col = (i - row * CPR) * 8;
      const uint32_t dst = base + (uint32_t)(row * RS + col) * 2u;
      if (c0 + row < p.N) cp_async16(dst, p.lmks + ((b * p.N + c0 + row) * HL + hl) * D + col);
      else *reinterpret_cast<uint4*>(buf + (size_t)which * kKeyBuf + (size_t)(row * RS + col) * 2) = make_uint4(0u, 0u, 0u, 0u);
    }
  };
  auto issue_q = [&](int r0, int which) {
    const uint32_t base = buf32 + (uint32_t)which * kQBuf;
    for (int i = tid; i < kBwdRows * CPR; i += 256) {
      const int row = i / CPR, col = (i - row * CPR) * 8;
      const uint32_t dst = base + (uint32_t)(row * RS + col) * 2u;
      if (r0 + row < n_rows) {
        int64_t ri, th;
        row_ptrs(r0 + row, ri, th);
        cp_async16(dst, p.q + ri * D + col);
      } else {
        *reinterpret_cast<uint4*>(buf + (size_t)which * kQBuf + (size_t)(row * RS + col) * 2) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
  };
  // the thread's (id, gradient) pairs of row r0 + srow; ids outside [0, N) become -1
  auto load_pairs = [&](int r0, int (&id)[kPipeSlots], bf16 (&g)[kPipeSlots]) {
#pragma unroll
    for (int j = 0; j < kPipeSlots; ++j) { id[j] = -1; g[j] = __float2bfloat16_rn(0.f); }
    if (r0 + srow < n_rows) {
      int64_t ri, th;
      row_ptrs(r0 + srow, ri, th);
      const int32_t* ip = p.ids + th * p.K + k0;
      const bf16* gp = p.ds + ri * p.K + k0;
#pragma unroll
      for (int j = 0; j < kPipeSlots; ++j)
        if (j < KPT) {
          const int v = ip[j];
          id[j] = (v >= 0 && v < p.N) ? v : -1;
          g[j] = gp[j];
        }
    }
  };
  auto scatter = [&](int c0, const int (&id)[kPipeSlots], const bf16 (&g)[kPipeSlots]) {
#pragma unroll
    for (int j = 0; j < kPipeSlots; ++j)
      if (id[j] >= c0 && id[j] < c0 + kBwdTile) ds_s[srow * kDsStride + id[j] - c0] = g[j];
  };
  auto unscatter = [&](int c0, const int (&id)[kPipeSlots]) {
#pragma unroll
    for (int j = 0; j < kPipeSlots; ++j)
      if (id[j] >= c0 && id[j] < c0 + kBwdTile) ds_s[srow * kDsStride + id[j] - c0] = __float2bfloat16_rn(0.f);
  };
  float dk[NB][4];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb)
#pragma unroll
    for (int e = 0; e < 4; ++e) dk[nb][e] = 0.f;
  auto flush_dk = [&](int c0) {
#pragma unroll
    for (int hr = 0; hr < 2; ++hr) {
      const int c = c0 + warp * 16 + (lane >> 2) + hr * 8;
      if (c < p.N) {
        float* dst = p.dl + ((b * p.N + c) * HL + hl) * D + (lane & 3) * 2;
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          const float2 v = make_float2(dk[nb][2 * hr] * p.scale, dk[nb][2 * hr + 1] * p.scale);
          if (v.x != 0.f || v.y != 0.f) atomicAdd(reinterpret_cast<float2*>(dst + nb * 8), v);
        }
      }
    }
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
      for (int e = 0; e < 4; ++e) dk[nb][e] = 0.f;
  };
  auto block_ntile = [&](int r0) -> int {
    if (tid == 0) max_id_s = -1;
    __syncthreads();
    int mx = -1;
    if (r0 + srow < n_rows) {
      int64_t ri, th;
      row_ptrs(r0 + srow, ri, th);
      for (int k = tid & 3; k < p.K; k += 4) mx = max(mx, p.ids[th * p.K + k]);
    }
    mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    if ((tid & 3) == 0 && mx >= 0) atomicMax(&max_id_s, mx);
    __syncthreads();
    const int max_id = max_id_s;
    __syncthreads();
    return max_id < 0 ? 0 : min(ntile_all, max_id / kBwdTile + 1);
  };
  auto mma_dq = [&](float (&dq)[NB / 2][4], int which) {
    const int mrow = (warp & 3) * 16, nhalf = (warp >> 2) * (D / 2);
    const uint32_t k32 = buf32 + (uint32_t)which * kKeyBuf;
    const uint32_t a_addr = ds32 + (uint32_t)((mrow + (lane & 7) + ((lane >> 3) & 1) * 8) * kDsStride + (lane >> 4) * 8) * 2u;
    const uint32_t b_addr = k32 + (uint32_t)(((lane & 7) + ((lane >> 3) & 1) * 8) * RS + nhalf + ((lane >> 4) & 1) * 8) * 2u;
#pragma unroll
    for (int kk = 0; kk < kBwdTile / 16; ++kk) {
      uint32_t a[4];
      ldsm4(a, a_addr + kk * 32);
#pragma unroll
      for (int np = 0; np < NB / 4; ++np) {
        uint32_t bb[4];
        ldsm4_t(bb, b_addr + (uint32_t)(kk * 16 * RS + np * 16) * 2u);
        mma16816(dq[2 * np], a, bb[0], bb[1]);
        mma16816(dq[2 * np + 1], a, bb[2], bb[3]);
      }
    }
  };
  auto mma_dk = [&](int which) {
    const int mcol = warp * 16;
    const uint32_t q32 = buf32 + (uint32_t)which * kQBuf;
    const uint32_t a_addr = ds32 + (uint32_t)(((lane & 7) + ((lane >> 4) & 1) * 8) * kDsStride + mcol + ((lane >> 3) & 1) * 8) * 2u;
    const uint32_t b_addr = q32 + (uint32_t)(((lane & 7) + ((lane >> 3) & 1) * 8) * RS + ((lane >> 4) & 1) * 8) * 2u;
#pragma unroll
    for (int kk = 0; kk < kBwdRows / 16; ++kk) {
      uint32_t a[4];
      ldsm4_t(a, a_addr + (uint32_t)(kk * 16 * kDsStride) * 2u);
#pragma unroll
      for (int np = 0; np < NB / 2; ++np) {
        uint32_t bb[4];
        ldsm4_t(bb, b_addr + (uint32_t)(kk * 16 * RS + np * 16) * 2u);
        mma16816(dk[2 * np], a, bb[0], bb[1]);
        mma16816(dk[2 * np + 1], a, bb[2], bb[3]);
      }
    }
  };
  auto store_dq = [&](int r0, float (&dq)[NB / 2][4]) {
    const int mrow = (warp & 3) * 16, nhalf = (warp >> 2) * (D / 2);
#pragma unroll
    for (int hr = 0; hr < 2; ++hr) {
      const int r = r0 + mrow + (lane >> 2) + hr * 8;
      if (r < n_rows) {
        int64_t ri, th;
        row_ptrs(r, ri, th);
        bf16* dst = p.dq + ri * D + nhalf + (lane & 3) * 2;
#pragma unroll
        for (int nb = 0; nb < NB / 2; ++nb)
          *reinterpret_cast<__nv_bfloat162*>(dst + nb * 8) =
              __floats2bfloat162_rn(dq[nb][2 * hr] * p.scale, dq[nb][2 * hr + 1] * p.scale);
      }
    }
  };

  for (int i = tid; i < kBwdRows * kDsStride / 8; i += 256) reinterpret_cast<uint4*>(ds_s)[i] = make_uint4(0u, 0u, 0u, 0u);
  // Phase 1, row block outer: dq of a block over the tiles its rows reach; key tile t + 1 arrives while tile t multiplies.
  int nt_max = 0;
  int id[kPipeSlots];
  bf16 g[kPipeSlots];
  for (int blk = 0; blk < kBwdBlocks; ++blk) {
    const int r0 = cta_row0 + blk * kBwdRows;
    int ntile = 0;
    if (r0 < n_rows) ntile = block_ntile(r0);                    // (barriers: the previous block is finished with everything)
    if (tid == 0) nt_s[blk] = ntile;
    nt_max = max(nt_max, ntile);
    if (r0 >= n_rows || ntile == 0) {
      if (r0 < n_rows) {                                         // rows without a selected chunk: dq = 0
        float dq0[NB / 2][4];
#pragma unroll
        for (int nb = 0; nb < NB / 2; ++nb)
#pragma unroll
          for (int e = 0; e < 4; ++e) dq0[nb][e] = 0.f;
        store_dq(r0, dq0);
      }
      continue;
    }
    issue_keys(0, 0);
    cp_async_commit();
    load_pairs(r0, id, g);
    float dq[NB / 2][4];
#pragma unroll
    for (int nb = 0; nb < NB / 2; ++nb)
#pragma unroll
      for (int e = 0; e < 4; ++e) dq[nb][e] = 0.f;
    for (int t = 0; t < ntile; ++t) {
      if (t + 1 < ntile) issue_keys((t + 1) * kBwdTile, (t + 1) & 1);   // its buffer was last read two tiles ago
      cp_async_commit();
      cp_async_wait1();                                          // this thread's pieces of key tile t have landed
      __syncwarp();                                              // the row's four threads are done clearing the last tile
      scatter(t * kBwdTile, id, g);
      __syncthreads();                                           // tile built, key tile t complete
      mma_dq(dq, t & 1);
      __syncthreads();                                           // everyone has read the tile and the keys
      unscatter(t * kBwdTile, id);
    }
    store_dq(r0, dq);
  }
  cp_async_wait0();
  __syncthreads();
  // Phase 2, tile outer: dk' of a tile accumulates in registers over ALL row blocks of the CTA and leaves as atomics once
  // per (CTA, tile); the next block's queries and (id, gradient) pairs arrive while the current block multiplies.
  auto next_block = [&](int after, int t) -> int {
    for (int blk = after + 1; blk < kBwdBlocks; ++blk)
      if (cta_row0 + blk * kBwdRows < n_rows && nt_s[blk] > t) return blk;
    return -1;
  };
  for (int t = 0; t < nt_max; ++t) {
    int cur = next_block(-1, t);
    if (cur < 0) continue;
    issue_q(cta_row0 + cur * kBwdRows, 0);
    cp_async_commit();
    load_pairs(cta_row0 + cur * kBwdRows, id, g);
    for (int i = 0; cur >= 0; ++i) {
      const int nxt = next_block(cur, t);
      int nid[kPipeSlots];
      bf16 ng[kPipeSlots];
      if (nxt >= 0) {
        issue_q(cta_row0 + nxt * kBwdRows, (i + 1) & 1);         // its buffer was last read two blocks ago
        load_pairs(cta_row0 + nxt * kBwdRows, nid, ng);
      }
      cp_async_commit();
      cp_async_wait1();
      __syncwarp();
      scatter(t * kBwdTile, id, g);
      __syncthreads();
      mma_dk(i & 1);
      __syncthreads();
      unscatter(t * kBwdTile, id);
      if (nxt >= 0) {
#pragma unroll
        for (int j = 0; j < kPipeSlots; ++j) { id[j] = nid[j]; g[j] = ng[j]; }
      }
      cur = nxt;
    }
    cp_async_wait0();
    flush_dk(t * kBwdTile);
  }
}

// d_q in bf16; dl: fp32 accumulator of the chunk-key gradient, zeroed by the caller.
int topk_bwd_mma_launch(const void* d_scores, const int32_t* indices, const void* q, const void* lmks, void* d_q,
                        float* dl, int B, int L, int N, int h_kv, int G, int D, int topk, int per_qhead, float scale,
                        cudaStream_t st) {
  if (D != 64 && D != 128) return HILS_ERR_UNSUPPORTED;
  const int HL = per_qhead ? h_kv * G : h_kv;
  if (HL > 65535 || B > 65535) return HILS_ERR_UNSUPPORTED;
  TopkBwdMmaParams p;
  p.ds = (const bf16*)d_scores; p.ids = indices; p.q = (const bf16*)q; p.lmks = (const bf16*)lmks;
  p.dq = (bf16*)d_q; p.dl = dl;
  p.L = L; p.N = N; p.h_kv = h_kv; p.G = G; p.K = topk; p.per_qhead = per_qhead; p.scale = scale;
  const int n_rows = L * (per_qhead ? 1 : G);
  dim3 grid((n_rows + kBwdRows * kBwdBlocks - 1) / (kBwdRows * kBwdBlocks), HL, B);
  if (N > kBwdTile && topk <= 4 * kPipeSlots && topk % 4 == 0) {   // several tiles: the pipelined kernel
    const size_t smem_p = (size_t)(kBwdRows * kDsStride + 2 * kBwdTile * (D + 8)) * sizeof(bf16);
    if (D == 64) {
      cudaFuncSetAttribute(topk_bwd_pipe_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_p);
      topk_bwd_pipe_kernel<4><<<grid, 256, smem_p, st>>>(p);
    } else {
      cudaFuncSetAttribute(topk_bwd_pipe_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_p);
      topk_bwd_pipe_kernel<8><<<grid, 256, smem_p, st>>>(p);
    }
    HILS_LAUNCH_CHECK("topk_bwd (tensor-core, pipelined)");
    return HILS_OK;
  }
  const size_t smem = (size_t)(kBwdRows * kDsStride + (kBwdTile + kBwdRows) * (D + 8)) * sizeof(bf16);
  if (D == 64) {
    cudaFuncSetAttribute(topk_bwd_mma_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    topk_bwd_mma_kernel<4><<<grid, 256, smem, st>>>(p);
  } else {
    cudaFuncSetAttribute(topk_bwd_mma_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    topk_bwd_mma_kernel<8><<<grid, 256, smem, st>>>(p);
  }
  HILS_LAUNCH_CHECK("topk_bwd (tensor-core)");
  return HILS_OK;
}

}  // namespace hils
