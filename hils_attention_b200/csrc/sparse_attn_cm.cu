// Sparse chunk attention, chunk-major over gathered owner rows (tcgen05 + TMEM + TMA), bf16.
//
// Every selected chunk has its own softmax (ops/hils_fwd_bwd_head.py:404-485), so the (token, slot) pairs of
// one chunk can be processed together wherever their tokens sit in the sequence.  An inverse index lists, per
// (batch, kv head, chunk), the pairs that selected the chunk.  One CTA owns one chunk: its K and V tiles
// [64 x D] are loaded once by TMA, and the chunk's owner rows are walked in tiles of 128 rows
// (128/G pairs x the G query heads of the group):
//   producer warps : gather the 128 query rows of the tile with 16-byte cp.async into a swizzled A tile
//   MMA warp       : S = Q K^T (tcgen05.mma, accumulator in TMEM), later O = P V
//   row warpgroups : one thread per row: P = w * softmax(scale S) -> shared memory (A operand of P V);
//                    then the O tile is read from TMEM and added to the fp32 output accumulator of each
//                    row's token with red.global.add (no two rows of a tile share a token)
// Every MMA row is a real (token, slot) pair: nothing is masked, whatever the overlap between neighbouring
// tokens' selections.  The price is the scatter: the partial outputs of a token's K slots meet in an fp32
// accumulator in global memory (L2-resident per head), which a last pass rounds to bf16.
// All mbarrier waits are bounded; on expiry a status word is set, every role leaves its loop and the CTA
// releases its TMEM and returns.
#include "sparse_attn_generic.cuh"
#include "umma.cuh"
#include "tc_rows.cuh"

namespace hils {

using namespace umma;

static __device__ int g_cm_status = 0;

// Bounded wait of this file's kernels: 2^20 polls (tens of milliseconds; a healthy wait lasts microseconds).
// After the first expiry anywhere on the device the status word is set and every CTA that starts later returns
// at once, so a fault costs one wait, not one per CTA.
__device__ __forceinline__ bool cm_wait(uint64_t* b, uint32_t parity) {
  const uint32_t addr = umma::smem_u32(b);
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
// contiguous bulk copy global -> shared (both 16-byte aligned, size a multiple of 16), completion counted in bytes on `bar`
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(umma::smem_u32(dst)), "l"(src), "r"(bytes), "r"(umma::smem_u32(bar))
               : "memory");
}
// TMA gather of four rows of a 2-D tensor (box = 64 columns x 1 row, 128-byte swizzle): the rows land as four
// consecutive 128-byte rows at `dst`, swizzled by their shared-memory address like a tiled load of the same place.
__device__ __forceinline__ void tma_gather4(void* dst, const CUtensorMap* map, uint64_t* bar, int col, int r0, int r1, int r2, int r3) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(umma::smem_u32(dst)), "l"(map), "r"(umma::smem_u32(bar)), "r"(col), "r"(r0), "r"(r1), "r"(r2), "r"(r3)
      : "memory");
}
// ---- scatter of accumulator tiles -------------------------------------------------------------------------------
// A tile's rows belong to different tokens, so its fp32 result is ADDED to global accumulator rows.  What bounds these
// adds is the number of requests the L2 atomic units see, not their bytes: 16-byte adds in which neighbouring lanes
// cover whole rows run about three times faster than 8-byte adds issued straight from the accumulator-fragment
// layout, and one reduce per row through the bulk-copy unit is slower again because that unit also carries the row
// gathers.  A single warp cannot issue the adds fast enough either.  Hence every row warp scatters its own 32 rows:
// each lane copies SLW columns of its row from TMEM into the warp's staging rows in shared memory, then the warp reads
// them back row by row (SLW/4 lanes per row) and issues red.global.add.v4.f32.  No barrier beyond __syncwarp.
__device__ __forceinline__ void red_add_v4(float* p, float4 v) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
template <int SLW>
struct StgGeom {
  static constexpr int kStride = SLW * 4 + 16;      // bytes per staged row (+16 keeps the 16-byte accesses conflict-free)
  static constexpr int kWarpBytes = 32 * kStride;   // staging rows of one warp
};
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {   // 16 fp32 columns of this thread's TMEM lane
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                 "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr));
}
// One warp: columns col0 .. col0 + SLW - 1 of its 32 TMEM lanes (`taddr` = this lane's address of column col0) are
// added to the accumulator rows `rowt` of the lanes (-1: no row).  `stg` = the warp's staging rows.
template <int SLW>
__device__ __forceinline__ void scatter_slice(uint8_t* stg, uint32_t taddr, int rowt, float* acc, int D, int col0, int lane) {
  constexpr int LPR = SLW / 4, RPI = 32 / LPR;      // lanes per row, rows per instruction
  float ov[SLW];
  if (SLW == 16) {
    tmem_ld16(taddr, ov);
  } else {
#pragma unroll
    for (int cb = 0; cb < SLW / 32; ++cb) umma::tmem_ld32(taddr + cb * 32, ov + cb * 32);
  }
  umma::tmem_ld_wait();
  __syncwarp();                                      // the previous slice has been read back by every lane
  uint8_t* mine = stg + lane * StgGeom<SLW>::kStride;
#pragma unroll
  for (int i = 0; i < SLW / 4; ++i)
    *reinterpret_cast<float4*>(mine + i * 16) = make_float4(ov[4 * i], ov[4 * i + 1], ov[4 * i + 2], ov[4 * i + 3]);
  __syncwarp();
  const int sub = lane / LPR, piece = lane % LPR;
#pragma unroll
  for (int it = 0; it < 32 / RPI; ++it) {
    const int row = it * RPI + sub;
    const int t = __shfl_sync(0xffffffffu, rowt, row);
    const float4 v = *reinterpret_cast<const float4*>(stg + row * StgGeom<SLW>::kStride + piece * 16);
    if (t >= 0) red_add_v4(acc + (int64_t)t * D + col0 + piece * 4, v);
  }
}
// keeps the first failure: code = 1000 * (wait site) + tile
__device__ __forceinline__ void cm_fail(int code) { atomicCAS(&g_cm_status, 0, code); }
// one poll: has the phase with this parity completed?
__device__ __forceinline__ bool cm_try(uint64_t* b, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.b32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(umma::smem_u32(b)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool cm_failed_before() { return *reinterpret_cast<volatile int*>(&g_cm_status) != 0; }

constexpr int kEntShift = 10;                 // entry = token << 10 | slot
constexpr int kEntSlotMask = (1 << kEntShift) - 1;

// =================================================================================================
// inverse index: pairs (token, slot) grouped by (batch, kv head, chunk), with their weights
// =================================================================================================
// Order inside a chunk's list: token tiles ascending; inside a tile tokens ascending, slots ascending.
// It is fixed by the index alone (no atomics decide it), so everything summed in list order is deterministic.
// The pairs' weights (one per query head of the group) are copied into a list of the same order, so the
// attention kernels stream entries and weights from contiguous memory instead of chasing token -> weight.
constexpr int kListAlign = 8;    // chunk lists start at multiples of 8 entries (16-byte aligned bulk copies)
constexpr int kTB = 4;           // tiles per metadata block
constexpr int kMS = 4;           // metadata slots in shared memory

struct InvIndex {
  const int32_t* list;    // [B*h_kv][cap]      entries (token << 10 | slot)
  const bf16* wlist;      // [B*h_kv][cap * G]  weights of the entries' G rows
  const uint32_t* coff;   // [B*h_kv][nchunk + 1] start of each chunk's list inside the (b, h) segment
  const uint32_t* tot;    // [B*h_kv][nchunk]   entries of each chunk
  size_t cap;             // entries per (b, h) segment
};

struct InvLayout {
  size_t cnt_off, tot_off, coff_off, list_off, wlist_off, total, cap;
  int TT, ntile;
};

// The staged build (inv_tile_kernel): a CTA of 8 warps owns a tile of 256 tokens and sorts the tile's entries by chunk
// in shared memory before they leave, so that a chunk's entries of the tile go out as one contiguous run.  It covers
// one query head per kv head, up to 32 slots per token and chunk counts whose histograms fit shared memory.
constexpr int kStageWarps = 8, kStageTW = 32, kStageTT = kStageWarps * kStageTW;
static bool inv_staged(int G, int K, int nchunk) { return G == 1 && K <= 32 && nchunk <= 2048; }
static size_t inv_staged_smem(int K, int nchunk, bool fill) {
  // per-warp histograms, tile totals, run offsets (+ the staged entries and weights)
  return (size_t)(kStageWarps + 2) * nchunk * 4 + 64 + (fill ? (size_t)kStageTT * K * 6 : 0);
}

static InvLayout inv_layout(int B, int L, int h_kv, int G, int K, int nchunk) {
  InvLayout l;
  int tt = (nchunk + K - 1) / K;              // keeps the per-tile histograms no larger than the list
  l.TT = inv_staged(G, K, nchunk) ? kStageTT : max(128, (tt + 31) / 32 * 32);
  l.ntile = (L + l.TT - 1) / l.TT;
  const size_t bh = (size_t)B * h_kv;
  auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
  l.cap = ((size_t)L * K + (size_t)kListAlign * nchunk + 63) & ~(size_t)63;
  l.cnt_off = 0;
  l.tot_off = up(l.cnt_off + bh * l.ntile * nchunk * 4);
  l.coff_off = up(l.tot_off + bh * nchunk * 4);
  l.list_off = up(l.coff_off + bh * (nchunk + 1) * 4);
  l.wlist_off = up(l.list_off + bh * l.cap * 4 + 256);            // + slack: block copies round their size up to 16 bytes
  l.total = up(l.wlist_off + bh * l.cap * G * 2 + 256);
  return l;
}

struct InvFill {
  int32_t* list;
  bf16* wlist;
  const bf16* w;        // (B, L, h_q, num_weights)
  int G, num_weights;
};

// ids of one token's slots k0 + lane; a row's list ends at its first negative id.  wrow: weights of (token, first
// query head of the group); w0: its entry for slot k, loaded ahead by the caller.
template <bool kFill>
__device__ __forceinline__ bool inv_step(int id, bool in_k, int t, int k, int nchunk, uint32_t* hist, const InvFill& f,
                                         const bf16* wrow, bf16 w0, int lane) {
  const unsigned neg = __ballot_sync(0xffffffffu, !in_k || id < 0);
  const bool live = neg == 0u || lane < (__ffs(neg) - 1);
  const bool take = live && id < nchunk;
  if (!kFill) {
    if (take) atomicAdd(&hist[id], 1u);
  } else {
    // equal ids inside one token (repeated slots) take consecutive positions in slot order
    const unsigned peers = __match_any_sync(0xffffffffu, take ? id : -1 - lane);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    uint32_t pos = 0;
    if (take) pos = hist[id] + rank;
    __syncwarp();
    if (take) {
      f.list[pos] = (t << kEntShift) | k;
      bf16* wl = f.wlist + (size_t)pos * f.G;
      wl[0] = w0;
      for (int g = 1; g < f.G; ++g) wl[g] = wrow[(size_t)g * f.num_weights + k];
      if (rank == __popc(peers) - 1) hist[id] = pos + 1;
    }
    __syncwarp();
  }
  return neg != 0u;
}

// one warp per (token tile, kv head, batch).  kFill = false: histogram of the tile's chunk ids.
// kFill = true: the same walk with the histogram started at each chunk's write position.
template <bool kFill>
__global__ void __launch_bounds__(32) inv_walk_kernel(const int32_t* __restrict__ idx, uint32_t* __restrict__ cnt,
                                                      const uint32_t* __restrict__ coff, InvFill f, size_t cap, int L,
                                                      int h_kv, int K, int nchunk, int TT, int ntile) {
  extern __shared__ uint32_t hist[];
  const int tile = blockIdx.x, h = blockIdx.y, b = blockIdx.z, lane = threadIdx.x;
  const size_t bh = (size_t)b * h_kv + h;
  uint32_t* my_cnt = cnt + (bh * ntile + tile) * nchunk;
  for (int c = lane; c < nchunk; c += 32) hist[c] = kFill ? coff[bh * (nchunk + 1) + c] + my_cnt[c] : 0u;
  __syncwarp();
  if (kFill) {
    f.list += bh * cap;
    f.wlist += bh * cap * f.G;
  }
  const int t0 = tile * TT, t1 = min(L, t0 + TT);
  const int32_t* base = idx + (((size_t)b * L) * h_kv + h) * K;
  const size_t tstride = (size_t)h_kv * K;
  const int h_q = h_kv * f.G;
  const bf16* wbase = kFill ? f.w + (((size_t)b * L) * h_q + (size_t)h * f.G) * f.num_weights : nullptr;
  const size_t wstride = (size_t)h_q * f.num_weights;
  const bf16 zero = __float2bfloat16_rn(0.f);
  if (K <= 32) {
    for (int t = t0; t < t1; t += 4) {   // four tokens' ids (and weights) in flight
      int v[4];
      bf16 wv[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const bool in = t + u < t1 && lane < K;
        v[u] = in ? __ldg(base + (size_t)(t + u) * tstride + lane) : -1;
        wv[u] = (kFill && in) ? wbase[(size_t)(t + u) * wstride + lane] : zero;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (t + u < t1)
          inv_step<kFill>(v[u], lane < K, t + u, lane, nchunk, hist, f, kFill ? wbase + (size_t)(t + u) * wstride : nullptr, wv[u], lane);
    }
  } else {
    for (int t = t0; t < t1; ++t)
      for (int k0 = 0; k0 < K; k0 += 32) {
        const int k = k0 + lane;
        const int id = k < K ? __ldg(base + (size_t)t * tstride + k) : -1;
        const bf16* wrow = kFill ? wbase + (size_t)t * wstride : nullptr;
        const bf16 w0 = (kFill && k < K) ? wrow[k] : zero;
        if (inv_step<kFill>(id, k < K, t, k, nchunk, hist, f, wrow, w0, lane)) break;
      }
  }
  if (!kFill) {
    __syncwarp();
    for (int c = lane; c < nchunk; c += 32) my_cnt[c] = hist[c];
  }
}

// Staged form of the walk for G = 1, K <= 32: one CTA per (token tile of 256, kv head, batch), warp w owns tokens
// 32w .. 32w+31 of the tile and holds their ids in registers (one token per lane-wide load, lane = slot).
// kFill = false: the tile's histogram.  kFill = true: per-warp histograms -> each warp's start inside every chunk's run
// of the tile (warps in token order) -> entries and weights placed in shared memory sorted by chunk, in the order of the
// plain walk (tokens ascending, slots ascending) -> every chunk's run copied out contiguously.  The plain walk writes
// every entry and weight to its own address: 4- and 2-byte stores scattered over the (b, h) segment, each a partial
// 32-byte sector that the memory system has to read, merge and write back.
template <bool kFill>
__global__ void __launch_bounds__(32 * kStageWarps) inv_tile_kernel(const int32_t* __restrict__ idx, uint32_t* __restrict__ cnt,
                                                                   const uint32_t* __restrict__ coff, InvFill f, size_t cap,
                                                                   int L, int h_kv, int K, int nchunk, int ntile) {
  extern __shared__ __align__(16) uint8_t inv_smem[];
  uint32_t* wcnt = reinterpret_cast<uint32_t*>(inv_smem);               // [warps][nchunk]
  uint32_t* tot_s = wcnt + (size_t)kStageWarps * nchunk;                // [nchunk] entries of the tile per chunk
  uint32_t* run_s = tot_s + nchunk;                                     // [nchunk] start of the chunk's run in the stage
  uint32_t* wsum = run_s + nchunk;                                      // [8] + carry
  int32_t* stage_l = reinterpret_cast<int32_t*>(wsum + 16);             // [256 * K]
  bf16* stage_w = reinterpret_cast<bf16*>(stage_l + (size_t)kStageTT * K);
  const int tile = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const size_t bh = (size_t)b * h_kv + h;
  for (int i = tid; i < (kFill ? kStageWarps : 1) * nchunk; i += 32 * kStageWarps) wcnt[i] = 0u;
  __syncthreads();
  const int t0 = tile * kStageTT + warp * kStageTW, t1 = min(L, t0 + kStageTW);
  const int32_t* base = idx + (((size_t)b * L) * h_kv + h) * K;
  const size_t tstride = (size_t)h_kv * K;
  // ids of the warp's 32 tokens; `take` bit u of lane k: slot k of token t0 + u is an entry
  int v[kStageTW];
#pragma unroll
  for (int u = 0; u < kStageTW; ++u) v[u] = (t0 + u < t1 && lane < K) ? __ldg(base + (size_t)(t0 + u) * tstride + lane) : -1;
  uint32_t take = 0u;
  uint32_t* my = kFill ? wcnt + (size_t)warp * nchunk : wcnt;
#pragma unroll
  for (int u = 0; u < kStageTW; ++u) {
    const unsigned neg = __ballot_sync(0xffffffffu, v[u] < 0);          // a row's list ends at its first negative id
    const bool live = neg == 0u || lane < (__ffs(neg) - 1);
    if (live && v[u] < nchunk) {
      take |= 1u << u;
      atomicAdd(&my[v[u]], 1u);
    }
  }
  __syncthreads();
  if constexpr (!kFill) {
    uint32_t* out = cnt + (bh * ntile + tile) * nchunk;
    for (int c = tid; c < nchunk; c += 32 * kStageWarps) out[c] = wcnt[c];
  } else {
  // each warp's start inside the chunk's run, the tile's total per chunk
  for (int c = tid; c < nchunk; c += 32 * kStageWarps) {
    uint32_t run = 0u;
#pragma unroll
    for (int w = 0; w < kStageWarps; ++w) {
      const uint32_t x = wcnt[(size_t)w * nchunk + c];
      wcnt[(size_t)w * nchunk + c] = run;
      run += x;
    }
    tot_s[c] = run;
  }
  __syncthreads();
  // exclusive scan of the totals over the chunks: thread i owns `per` consecutive chunks
  {
    const int per = (nchunk + 32 * kStageWarps - 1) / (32 * kStageWarps), c0 = tid * per, c1 = min(nchunk, c0 + per);
    uint32_t mine = 0u;
    for (int c = c0; c < c1; ++c) mine += tot_s[c];
    uint32_t inc = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t x = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += x;
    }
    if (lane == 31) wsum[warp] = inc;
    __syncthreads();
    uint32_t run = inc - mine;
    for (int w = 0; w < warp; ++w) run += wsum[w];
    for (int c = c0; c < c1; ++c) {
      run_s[c] = run;
      run += tot_s[c];
    }
  }
  __syncthreads();
  // placement in the order of the plain walk
  const bf16* wbase = f.w + (((size_t)b * L) * h_kv + h) * f.num_weights;       // G = 1: h_q = h_kv
  const size_t wstride = (size_t)h_kv * f.num_weights;
  uint32_t* mine_cnt = wcnt + (size_t)warp * nchunk;
#pragma unroll
  for (int u0 = 0; u0 < kStageTW; u0 += 8) {
    bf16 wv[8];
#pragma unroll
    for (int u = 0; u < 8; ++u)
      wv[u] = ((take >> (u0 + u)) & 1u) ? wbase[(size_t)(t0 + u0 + u) * wstride + lane] : __float2bfloat16_rn(0.f);
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const bool tk = (take >> (u0 + u)) & 1u;
      const int id = v[u0 + u];
      // equal ids inside one token (repeated slots) take consecutive positions in slot order
      const unsigned peers = __match_any_sync(0xffffffffu, tk ? id : -1 - lane);
      const int rank = __popc(peers & ((1u << lane) - 1u));
      uint32_t pos = 0u;
      if (tk) pos = run_s[id] + mine_cnt[id] + rank;
      __syncwarp();
      if (tk) {
        stage_l[pos] = ((t0 + u0 + u) << kEntShift) | lane;
        stage_w[pos] = wv[u];
        if (rank == __popc(peers) - 1) mine_cnt[id] += (uint32_t)__popc(peers);
      }
      __syncwarp();
    }
  }
  __syncthreads();
  // copy-out: 32 chunks per warp step, one chunk's run at a time
  int32_t* list = f.list + bh * cap;
  bf16* wlist = f.wlist + bh * cap;
  const uint32_t* tile_pre = cnt + (bh * ntile + tile) * nchunk;        // entries of the chunk in the tiles before this one
  for (int c0 = warp * 32; c0 < nchunk; c0 += 32 * kStageWarps) {
    const int c = c0 + lane;
    const uint32_t n_l = c < nchunk ? tot_s[c] : 0u;
    const uint32_t src_l = c < nchunk ? run_s[c] : 0u;
    const uint32_t dst_l = (c < nchunk && n_l) ? coff[bh * (nchunk + 1) + c] + tile_pre[c] : 0u;
    unsigned any = __ballot_sync(0xffffffffu, n_l != 0u);
    while (any) {
      const int j = __ffs(any) - 1;
      any &= any - 1;
      const uint32_t n = __shfl_sync(0xffffffffu, n_l, j), src = __shfl_sync(0xffffffffu, src_l, j);
      const uint32_t dst = __shfl_sync(0xffffffffu, dst_l, j);
      for (uint32_t e = lane; e < n; e += 32) {
        list[dst + e] = stage_l[src + e];
        wlist[dst + e] = stage_w[src + e];
      }
    }
  }
  }
}

// per (b, h, chunk): exclusive prefix of the tile histograms over the tiles (in place) and the chunk's total.
// A CTA takes 64 chunks; the tiles are cut into four segments walked by four groups of threads (segment sums first,
// then the prefixes: the second read of a segment comes from L2), so four times as many loads are in flight as with
// one thread per chunk.
constexpr int kScanChunks = 64, kScanSegs = 4;
__global__ void __launch_bounds__(kScanChunks * kScanSegs) inv_scan_kernel(uint32_t* __restrict__ cnt, uint32_t* __restrict__ tot,
                                                                         int nchunk, int ntile) {
  __shared__ uint32_t seg_sum[kScanSegs][kScanChunks];
  const int cl = threadIdx.x % kScanChunks, seg = threadIdx.x / kScanChunks;
  const int c = blockIdx.x * kScanChunks + cl;
  const size_t bh = blockIdx.y;
  const int per = (ntile + kScanSegs - 1) / kScanSegs, ta = min(ntile, seg * per), tb = min(ntile, ta + per);
  uint32_t* p = cnt + bh * ntile * nchunk + min(c, nchunk - 1);
  uint32_t s = 0;
  if (c < nchunk) {
#pragma unroll 8
    for (int t = ta; t < tb; ++t) s += p[(size_t)t * nchunk];
  }
  seg_sum[seg][cl] = s;
  __syncthreads();
  if (c >= nchunk) return;
  uint32_t run = 0;
  for (int i = 0; i < seg; ++i) run += seg_sum[i][cl];
#pragma unroll 8
  for (int t = ta; t < tb; ++t) {
    const uint32_t v = p[(size_t)t * nchunk];
    p[(size_t)t * nchunk] = run;
    run += v;
  }
  if (seg == kScanSegs - 1) tot[bh * nchunk + c] = run;
}

// per (b, h): exclusive prefix of the chunk totals, each rounded up to the list alignment
__global__ void __launch_bounds__(256) inv_offsets_kernel(const uint32_t* __restrict__ tot, uint32_t* __restrict__ coff, int nchunk) {
  __shared__ uint32_t wsum[8];
  __shared__ uint32_t carry_s;
  const size_t bh = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) carry_s = 0;
  __syncthreads();
  for (int c0 = 0; c0 < nchunk; c0 += 256) {
    const int c = c0 + tid;
    const uint32_t v = c < nchunk ? ((tot[bh * nchunk + c] + kListAlign - 1) / kListAlign) * kListAlign : 0u;
    uint32_t inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t n = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += n;
    }
    if (lane == 31) wsum[warp] = inc;
    __syncthreads();
    uint32_t pre = carry_s;
    for (int w = 0; w < warp; ++w) pre += wsum[w];
    if (c < nchunk) coff[bh * (nchunk + 1) + c] = pre + inc - v;
    __syncthreads();
    if (tid == 255) carry_s = pre + inc;
    __syncthreads();
  }
  if (tid == 0) coff[bh * (nchunk + 1) + nchunk] = carry_s;
}

// the index as a finished forward call left it at the start of its workspace (`built` holds inv_layout().total bytes)
static void adopt_inverse_index(const SparseParams& p, const void* built, InvIndex* ix) {
  const InvLayout l = inv_layout(p.B, p.L, p.h_kv, p.h_q / p.h_kv, p.K, p.T / 64);
  const uint8_t* ws = static_cast<const uint8_t*>(built);
  ix->list = reinterpret_cast<const int32_t*>(ws + l.list_off);
  ix->wlist = reinterpret_cast<const bf16*>(ws + l.wlist_off);
  ix->coff = reinterpret_cast<const uint32_t*>(ws + l.coff_off);
  ix->tot = reinterpret_cast<const uint32_t*>(ws + l.tot_off);
  ix->cap = l.cap;
}

static int build_inverse_index(const SparseParams& p, void* workspace, InvIndex* ix, cudaStream_t st) {
  const int nchunk = p.T / 64, G = p.h_q / p.h_kv;
  const InvLayout l = inv_layout(p.B, p.L, p.h_kv, G, p.K, nchunk);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  uint32_t* cnt = reinterpret_cast<uint32_t*>(ws + l.cnt_off);
  uint32_t* tot = reinterpret_cast<uint32_t*>(ws + l.tot_off);
  uint32_t* coff = reinterpret_cast<uint32_t*>(ws + l.coff_off);
  InvFill f;
  f.list = reinterpret_cast<int32_t*>(ws + l.list_off);
  f.wlist = reinterpret_cast<bf16*>(ws + l.wlist_off);
  f.w = static_cast<const bf16*>(p.w);
  f.G = G;
  f.num_weights = p.num_weights;
  dim3 gw(l.ntile, p.h_kv, p.B);
  if (inv_staged(G, p.K, nchunk)) {
    const size_t smem_c = inv_staged_smem(p.K, nchunk, false), smem_f = inv_staged_smem(p.K, nchunk, true);
    cudaFuncSetAttribute(inv_tile_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_c);
    cudaFuncSetAttribute(inv_tile_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_f);
    inv_tile_kernel<false><<<gw, 32 * kStageWarps, smem_c, st>>>(p.idx, cnt, nullptr, f, l.cap, p.L, p.h_kv, p.K, nchunk, l.ntile);
    inv_scan_kernel<<<dim3((nchunk + kScanChunks - 1) / kScanChunks, p.B * p.h_kv), kScanChunks * kScanSegs, 0, st>>>(cnt, tot, nchunk, l.ntile);
    inv_offsets_kernel<<<p.B * p.h_kv, 256, 0, st>>>(tot, coff, nchunk);
    inv_tile_kernel<true><<<gw, 32 * kStageWarps, smem_f, st>>>(p.idx, cnt, coff, f, l.cap, p.L, p.h_kv, p.K, nchunk, l.ntile);
    HILS_LAUNCH_CHECK("sparse_attn inverse index (staged)");
  } else {
    const size_t smem = (size_t)nchunk * 4;
    if (smem > 48 * 1024) {
      cudaFuncSetAttribute(inv_walk_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      cudaFuncSetAttribute(inv_walk_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    }
    inv_walk_kernel<false><<<gw, 32, smem, st>>>(p.idx, cnt, nullptr, f, l.cap, p.L, p.h_kv, p.K, nchunk, l.TT, l.ntile);
    inv_scan_kernel<<<dim3((nchunk + kScanChunks - 1) / kScanChunks, p.B * p.h_kv), kScanChunks * kScanSegs, 0, st>>>(cnt, tot, nchunk, l.ntile);
    inv_offsets_kernel<<<p.B * p.h_kv, 256, 0, st>>>(tot, coff, nchunk);
    inv_walk_kernel<true><<<gw, 32, smem, st>>>(p.idx, cnt, coff, f, l.cap, p.L, p.h_kv, p.K, nchunk, l.TT, l.ntile);
    HILS_LAUNCH_CHECK("sparse_attn inverse index");
  }
  ix->list = f.list;
  ix->wlist = f.wlist;
  ix->coff = coff;
  ix->tot = tot;
  ix->cap = l.cap;
  return HILS_OK;
}

// =================================================================================================
// forward
// =================================================================================================
// 2 row warpgroups + MMA/TMA warp + gather warp: 10 warps, at most 3 per scheduler, which leaves the row threads 168
// registers (a 13-warp CTA would cap every thread at 128)
constexpr int kCmThreads = 320;

template <int D>
__global__ void __launch_bounds__(kCmThreads, 1) sparse_fwd_cm_kernel(SparseParams p, InvIndex ix, float* __restrict__ o_acc,
                                                                      const __grid_constant__ CUtensorMap tmK,
                                                                      const __grid_constant__ CUtensorMap tmV,
                                                                      const __grid_constant__ CUtensorMap tmQ) {
  constexpr int DB = D / 64;
  constexpr int QBYTES = DB * 16384;     // gathered Q tile, 128 x D
  constexpr int KVBYTES = DB * 8192;     // K or V tile, 64 x D
  constexpr int NQ = (D == 64) ? 4 : 2;  // Q tile ring (gathers of several tiles in flight)
  constexpr int TM_COLS = (D == 64) ? 256 : 512;   // S: 2 x 64 columns, O: 2 x D columns
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* Ks = smem;
  uint8_t* Vs = Ks + KVBYTES;
  uint8_t* Qs = Vs + KVBYTES;            // NQ stages
  uint8_t* Ps = Qs + NQ * QBYTES;        // 2 x [128 x 64] bf16
  uint8_t* Stg = Ps + 2 * 16384;         // staging rows of the 8 row warps (32 rows x 64 fp32 columns each)

  __shared__ uint64_t kv_full, q_full[4], q_free[4], s_full[2], p_full[2], o_full[2], o_free[2];
  __shared__ uint32_t tmem_base_s;
  // metadata of the chunk's owner rows, streamed in blocks of kTB tiles by bulk copies: list entries and weights
  __shared__ __align__(16) int ent_ring[kMS][kTB * 128];
  __shared__ __align__(16) bf16 w_ring[kMS][kTB * 128];
  __shared__ uint64_t meta_full[kMS];
  __shared__ volatile int abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nchunk = p.T / 64;
  const int c = blockIdx.x;              // early chunks carry the longest lists and start first
  const int h = blockIdx.y, b = blockIdx.z;
  const size_t bh = (size_t)b * p.h_kv + h;
  const uint32_t beg = ix.coff[bh * (nchunk + 1) + c];
  const int n_ent = (int)ix.tot[bh * nchunk + c];
  if (n_ent == 0 || cm_failed_before()) return;   // nobody selected this chunk, or an earlier CTA's wait expired
  // G divides 128, so it is a power of two: rows map to (pair, group member) by shift and mask (a division by a
  // run-time G in the gather loop cost more than the copies themselves)
  const int G = p.h_q / p.h_kv, gs = 31 - __clz(G), QB = 128 >> gs;
  const int ntile = (n_ent + QB - 1) / QB;
  const int32_t* lst = ix.list + bh * ix.cap + beg;
  const bf16* wl = ix.wlist + (bh * ix.cap + beg) * G;

  if (tid == 0) {
    mbar_init(&kv_full, 1);
    for (int s = 0; s < kMS; ++s) mbar_init(&meta_full[s], 1);
    for (int s = 0; s < NQ; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_free[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&p_full[s], 128);
      mbar_init(&o_full[s], 1);
      mbar_init(&o_free[s], 128);
    }
    mbar_init_fence();
    abort_s = 0;
  }
  if (warp == 8) tmem_alloc(&tmem_base_s, TM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  const uint32_t tS = tmem, tO = tmem + 128;

  if (warp == 9) {
    // =============================== gather producer (one warp) =================================
    // The rows of a tile are fetched by TMA gather instructions, four rows each: lane l issues the gathers of rows
    // 4 l .. 4 l + 3 (one per 64-column block).  The TMA unit keeps the requests of several tiles in flight; this
    // warp only reads the tile's list entries and waits for a free ring stage.
    // Metadata block m = tiles kTB m .. kTB m + kTB - 1, slot m % kMS, fetched by bulk copies.  Block m + 1 is requested
    // when block m starts: its slot was last used by block m - 3, i.e. by tiles up to kTB (m - 2) - 1.  The ring wait of
    // tile kTB m has passed by then, which puts the row threads past tile kTB m - NQ - 2 at least, so with NQ <= 4 no
    // thread still reads that slot or waits on its barrier (a waiter two phases behind would never wake).
    const int TBQ = kTB * QB, nblk = (ntile + kTB - 1) / kTB;
    auto request_meta = [&](int m) {
      const int e0 = m * TBQ, ne = min(n_ent - e0, TBQ);
      const uint32_t eb = (uint32_t)(ne * 4 + 15) & ~15u, wb = (uint32_t)(ne * G * 2 + 15) & ~15u;
      mbar_expect_tx(&meta_full[m % kMS], eb + wb);
      bulk_load(ent_ring[m % kMS], lst + e0, eb, &meta_full[m % kMS]);
      bulk_load(w_ring[m % kMS], wl + (size_t)e0 * G, wb, &meta_full[m % kMS]);
    };
    if (lane == 0) {
      request_meta(0);
      if (nblk > 1) request_meta(1);
    }
    const int row_base = (b * p.L) * p.h_q + h * G;      // tensor row of (token 0, first query head of the group)
    bool ok = true;
    for (int j = 0; j < ntile; ++j) {
      const int s = j % NQ;
      if (j >= NQ) {
        ok = cm_wait(&q_free[s], ((j / NQ) - 1) & 1) && !abort_s;
        if (!ok) { cm_fail(4010000 + j); break; }
      }
      const int m = j / kTB;
      if (j % kTB == 0) {
        if (m >= 1 && m + 1 < nblk && lane == 0) request_meta(m + 1);
        ok = cm_wait(&meta_full[m % kMS], (m / kMS) & 1);
        if (!ok) { cm_fail(4011000 + j); break; }
      }
      const int* ents = ent_ring[m % kMS] + (j % kTB) * QB;
      int rr[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int row = 4 * lane + i;
        const bool live = j * QB + (row >> gs) < n_ent;      // rows past the end of the list fetch row 0; their P is zero
        rr[i] = live ? row_base + (ents[row >> gs] >> kEntShift) * p.h_q + (row & (G - 1)) : row_base;
      }
      if (lane == 0) mbar_expect_tx(&q_full[s], QBYTES);
      __syncwarp();
#pragma unroll
      for (int db = 0; db < DB; ++db) {
        tma_gather4(Qs + s * QBYTES + db * 16384 + lane * 512, &tmQ, &q_full[s], db * 64, rr[0], rr[1], rr[2], rr[3]);
      }
    }
    if (!ok && lane == 0) abort_s = 1;
  } else if (warp == 8) {
    // =============================== TMA (once) + MMA issuer ====================================
    if (lane == 0) {
      mbar_expect_tx(&kv_full, 2 * KVBYTES);
#pragma unroll
      for (int db = 0; db < DB; ++db) {
        tma_load_2d(Ks + db * 8192, &tmK, &kv_full, h * D + db * 64, b * p.T + c * 64);
        tma_load_2d(Vs + db * 8192, &tmV, &kv_full, h * D + db * 64, b * p.T + c * 64);
      }
      constexpr uint32_t idesc_qk = idesc_bf16(128, 64, 0);
      constexpr uint32_t idesc_pv = idesc_bf16(128, D, 1);
      const DescWords q_d = desc_words_sw128(smem_u32(Qs), 16, 1024), k_d = desc_words_sw128(smem_u32(Ks), 16, 1024),
                      p_d = desc_words_sw128(smem_u32(Ps), 16, 1024), v_d = desc_words_sw128(smem_u32(Vs), 8192, 1024);
      auto issue_qk = [&](int sq, int sb) {   // sq: Q ring stage, sb: S buffer
        const uint32_t qb = q_d.lo + sq * (QBYTES >> 4);
        mma_ss_w<false>(tS + sb * 64, qb, q_d.hi, k_d.lo, k_d.hi, idesc_qk);
#pragma unroll
        for (int kk = 1; kk < D / 16; ++kk)
          mma_ss_w<true>(tS + sb * 64, qb + (((kk >> 2) * 16384 + (kk & 3) * 32) >> 4), q_d.hi,
                         k_d.lo + (((kk >> 2) * 8192 + (kk & 3) * 32) >> 4), k_d.hi, idesc_qk);
        mma_commit(&q_free[sq]);
        mma_commit(&s_full[sb]);
      };
      bool ok = cm_wait(&kv_full, 0) && cm_wait(&q_full[0], 0);
      if (ok) {
        tc_fence_after();
        issue_qk(0, 0);
      }
      for (int j = 0; ok && j < ntile; ++j) {
        const int sb = j & 1, u = j >> 1;
        if (abort_s) { ok = false; break; }
        if (j + 1 < ntile) {
          const int s1 = (j + 1) % NQ;
          ok = cm_wait(&q_full[s1], ((j + 1) / NQ) & 1);
          if (!ok) { cm_fail(4021000 + j); break; }
          tc_fence_after();
          issue_qk(s1, sb ^ 1);      // its S buffer was consumed by tile j - 1 (p_full waited for below, last iteration)
        }
        ok = cm_wait(&p_full[sb], u & 1);
        if (!ok) cm_fail(4022000 + j);
        if (ok && u >= 1) { ok = cm_wait(&o_free[sb], (u - 1) & 1); if (!ok) cm_fail(4023000 + j); }  // the O buffer's previous tile has been read out
        if (!ok) break;
        tc_fence_after();
        {
          const uint32_t a0 = p_d.lo + sb * (16384 >> 4);
          mma_ss_w<false>(tO + sb * D, a0, p_d.hi, v_d.lo, v_d.hi, idesc_pv);
#pragma unroll
          for (int kk = 1; kk < 4; ++kk)
            mma_ss_w<true>(tO + sb * D, a0 + ((kk * 32) >> 4), p_d.hi, v_d.lo + ((kk * 2048) >> 4), v_d.hi, idesc_pv);
        }
        mma_commit(&o_full[sb]);
      }
      if (!ok) { abort_s = 1; cm_fail(4020000); }
    }
  } else {
    // =============================== row warpgroups ==============================================
    const int r = tid & 127, wg = tid >> 7;                 // warpgroup wg takes tiles wg, wg + 2, ... and buffers wg
    const int g = r & (G - 1), hq = h * G + g, rp = r >> gs;
    const float scale_log2 = p.scale * kLog2e;
    const float slope = p.slope ? p.slope[hq] : 0.f;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    uint8_t* prow = Ps + wg * 16384;
    bool ok = true;
    for (int j = wg, u = 0; j < ntile; j += 2, ++u) {
      ok = cm_wait(&s_full[wg], u & 1);
      if (!ok) cm_fail(4031000 + j);
      ok = __all_sync(0xffffffffu, ok) && !abort_s;
      if (!ok) break;
      tc_fence_after();
      const int m = j / kTB;
      ok = cm_wait(&meta_full[m % kMS], (m / kMS) & 1);
      ok = __all_sync(0xffffffffu, ok) && !abort_s;
      if (!ok) break;
      const bool live = j * QB + rp < n_ent;
      const int ent = live ? ent_ring[m % kMS][(j % kTB) * QB + rp] : 0;
      const float wv = live ? to_f(w_ring[m % kMS][(j % kTB) * 128 + r]) : 0.f;
      const int rowt = live ? (int)(((int64_t)b * p.L + (ent >> kEntShift)) * p.h_q + hq) : -1;
      float sv[64];
      tmem_ld32(tS + lane_base + wg * 64, sv);
      tmem_ld32(tS + lane_base + wg * 64 + 32, sv + 32);
      tmem_ld_wait();
      if (live) {
        if (slope != 0.f) {
#pragma unroll
          for (int jj = 0; jj < 62; ++jj) sv[jj] -= slope * (float)(62 - jj);
        }
        if (p.mask_last) sv[63] = -CUDART_INF_F;
        float m4[4] = {sv[0], sv[1], sv[2], sv[3]};
#pragma unroll
        for (int jj = 4; jj < 64; ++jj) m4[jj & 3] = fmaxf(m4[jj & 3], sv[jj]);
        const float mb = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * scale_log2;
        float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int jj = 0; jj < 64; ++jj) {
          sv[jj] = ex2(fmaf(sv[jj], scale_log2, -mb));
          s4[jj & 3] += sv[jj];
        }
        const float f = wv / ((s4[0] + s4[1]) + (s4[2] + s4[3]));
#pragma unroll
        for (int jj = 0; jj < 64; ++jj) sv[jj] *= f;
        store_row_bf16_sw128(prow, r, sv);
      } else {
        store_row_zero_sw128(prow, r);
      }
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(&p_full[wg]);
      ok = cm_wait(&o_full[wg], u & 1);
      if (!ok) cm_fail(4032000 + j);
      ok = __all_sync(0xffffffffu, ok) && !abort_s;
      if (!ok) break;
      tc_fence_after();
      // O tile -> fp32 accumulator rows of the tokens, 64 columns at a time
#pragma unroll
      for (int sl = 0; sl < D / 64; ++sl)
        scatter_slice<64>(Stg + warp * StgGeom<64>::kWarpBytes, tO + lane_base + wg * D + sl * 64, rowt, o_acc, D, sl * 64, lane);
      tc_fence_before();
      mbar_arrive(&o_free[wg]);
    }
    if (!ok && lane == 0) { abort_s = 1; cm_fail(4030000); }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 8) tmem_dealloc(tmem, TM_COLS);
}

// fp32 accumulator -> bf16 output, 8 elements per thread
__global__ void __launch_bounds__(256) cm_round_kernel(const float* __restrict__ acc, bf16* __restrict__ out, int64_t n8) {
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= n8) return;
  const float4 a = *reinterpret_cast<const float4*>(acc + i * 8), c = *reinterpret_cast<const float4*>(acc + i * 8 + 4);
  __nv_bfloat162 hh[4] = {__floats2bfloat162_rn(a.x, a.y), __floats2bfloat162_rn(a.z, a.w), __floats2bfloat162_rn(c.x, c.y),
                          __floats2bfloat162_rn(c.z, c.w)};
  *reinterpret_cast<uint4*>(out + i * 8) = *reinterpret_cast<uint4*>(hh);
}

static bool cm_shape_ok(const SparseParams& p) {
  const int D = p.D;
  if (p.S != 64 || p.D != p.Dv || (D != 64 && D != 128)) return false;
  const int G = p.h_q / p.h_kv;
  if (G > 128 || (128 % G) != 0) return false;
  if (p.T < 64 || p.K > (1 << kEntShift) || p.L >= (1 << (31 - kEntShift))) return false;
  if ((int64_t)p.B * p.T >= (1ll << 31) || (int64_t)p.B * p.L * p.h_q >= (1ll << 31)) return false;
  if ((size_t)(p.T / 64) * 4 > 200 * 1024) return false;    // chunk histogram of the index build lives in shared memory
  if ((int64_t)p.L * p.K >= (1ll << 32)) return false;
  return true;
}

static size_t cm_fwd_smem(int D) {
  const int NQ = (D == 64) ? 4 : 2;
  return 1024 + 2 * (size_t)(D / 64) * 8192 + (size_t)NQ * (D / 64) * 16384 + 2 * 16384 + 8 * (size_t)StgGeom<64>::kWarpBytes;
}

// bytes of the inverse index at the start of the chunk-major workspaces (0: shape outside this path)
size_t sparse_cm_index_bytes(const SparseParams& p) {
  if (!cm_shape_ok(p)) return 0;
  return inv_layout(p.B, p.L, p.h_kv, p.h_q / p.h_kv, p.K, p.T / 64).total;
}

// workspace of the chunk-major forward: inverse index + fp32 output accumulator (0: shape outside this path)
size_t sparse_fwd_cm_workspace(const SparseParams& p) {
  if (!cm_shape_ok(p)) return 0;
  const InvLayout l = inv_layout(p.B, p.L, p.h_kv, p.h_q / p.h_kv, p.K, p.T / 64);
  return l.total + (size_t)p.B * p.L * p.h_q * p.D * sizeof(float);
}

// Returns HILS_ERR_UNSUPPORTED (without setting an error text) when the shape is outside this path.
int sparse_fwd_cm_launch(const SparseParams& p, void* workspace, cudaStream_t st) {
  if (!cm_shape_ok(p) || !workspace) return HILS_ERR_UNSUPPORTED;
  if (((uintptr_t)p.q | (uintptr_t)p.k | (uintptr_t)p.v | (uintptr_t)p.o | (uintptr_t)workspace) & 15) return HILS_ERR_UNSUPPORTED;
  const int D = p.D, nchunk = p.T / 64;
  const InvLayout l = inv_layout(p.B, p.L, p.h_kv, p.h_q / p.h_kv, p.K, nchunk);
  InvIndex ix;
  if (int rc = build_inverse_index(p, workspace, &ix, st)) return rc;
  float* o_acc = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + l.total);
  const size_t n_out = (size_t)p.B * p.L * p.h_q * D;
  cudaError_t e = cudaMemsetAsync(o_acc, 0, n_out * sizeof(float), st);
  if (e != cudaSuccess) return cuda_fail(e, "sparse_attn_fwd accumulator clear");
  CUtensorMap tmK, tmV;
  if (int rc = make_tmap_bf16_rows(&tmK, p.k, (uint64_t)p.B * p.T, (uint64_t)p.h_kv * D, (uint64_t)p.h_kv * D, 64)) return rc;
  if (int rc = make_tmap_bf16_rows(&tmV, p.v, (uint64_t)p.B * p.T, (uint64_t)p.h_kv * D, (uint64_t)p.h_kv * D, 64)) return rc;
  CUtensorMap tmQ;   // rows = (batch, token, query head), one row per box: the source of the row gathers
  if (int rc = make_tmap_bf16_rows(&tmQ, p.q, (uint64_t)p.B * p.L * p.h_q, D, D, 1)) return rc;
  const size_t smem = cm_fwd_smem(D);
  dim3 grid(nchunk, p.h_kv, p.B);
  if (D == 64) {
    cudaFuncSetAttribute(sparse_fwd_cm_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sparse_fwd_cm_kernel<64><<<grid, kCmThreads, smem, st>>>(p, ix, o_acc, tmK, tmV, tmQ);
  } else {
    cudaFuncSetAttribute(sparse_fwd_cm_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sparse_fwd_cm_kernel<128><<<grid, kCmThreads, smem, st>>>(p, ix, o_acc, tmK, tmV, tmQ);
  }
  cm_round_kernel<<<(unsigned)((n_out / 8 + 255) / 256), 256, 0, st>>>(o_acc, static_cast<bf16*>(p.o), (int64_t)(n_out / 8));
  HILS_LAUNCH_CHECK("sparse_attn_fwd (chunk-major path)");
  return HILS_OK;
}

// =================================================================================================
// backward: one kernel, chunk-major like the forward
// =================================================================================================
// Per tile of 128 owner rows of the chunk (Q and dO rows gathered by the producer warps):
//   MMA  : S = Q K^T and dP = dO V^T                                   (TMEM, 2 x 64 columns)
//   rows : P from S, dw = sum_j P_j dP_j (stored per (token, q head, slot)), dS = scale w P (dP - dw) and w P
//          as bf16 tiles in shared memory                                (ops/hils_fwd_bwd_head.py:651-757)
//   MMA  : dQ tile = dS K (TMEM, read out and added to the fp32 dQ accumulator of each row's token);
//          dK += dS^T Q and dV += (wP)^T dO accumulate in TMEM over ALL tiles of the chunk and are written
//          once at the end: no atomics on dK / dV, and their sums run in list order (deterministic).
// D = 64 keeps two S/dP accumulators, two dQ tiles and two dS / wP tiles and forms dK and dV in one stacked
// M = 128, N = 128 product per 16 rows (A = [dS^T ; (wP)^T], B = [Q | dO]; the diagonal blocks of the accumulator
// are dK and dV).  D = 128 has TMEM and shared memory for one of each.
template <int D>
__global__ void __launch_bounds__(kCmThreads, 1) sparse_bwd_cm_kernel(SparseParams p, InvIndex ix, float* __restrict__ dq_acc,
                                                                      const __grid_constant__ CUtensorMap tmK,
                                                                      const __grid_constant__ CUtensorMap tmV,
                                                                      const __grid_constant__ CUtensorMap tmQ,
                                                                      const __grid_constant__ CUtensorMap tmdO) {
  constexpr int DB = D / 64;
  constexpr int QBYTES = DB * 16384;
  constexpr int KVBYTES = DB * 8192;
  constexpr int NSB = (D == 64) ? 2 : 1;   // S/dP accumulators in TMEM
  constexpr int NDQ = (D == 64) ? 2 : 1;   // dQ tiles in TMEM
  constexpr int NDS = (D == 64) ? 2 : 1;   // dS / wP tiles in shared memory
  constexpr int NQ = (D == 64) ? 3 : 2;    // Q / dO ring (> NSB: tile j + NSB can be gathered while tile j is in use)
  constexpr int SLW = (D == 64) ? 32 : 16; // columns of a staged dQ slice (what shared memory is left for)
  constexpr int NS = D / SLW;
  constexpr int PIECES = D / 8;            // 16-byte pieces per row
  constexpr bool kStacked = (D == 64);
  // TMEM columns: S/dP [0, NSB*128), dQ [NSB*128, +NDQ*D), dK (and dV) after them
  constexpr uint32_t C_DQ = NSB * 128, C_DK = C_DQ + NDQ * D, C_DV = C_DK + D;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* Qs = smem;                      // NQ stages
  uint8_t* dOs = Qs + NQ * QBYTES;         // NQ stages
  uint8_t* Ks = dOs + NQ * QBYTES;
  uint8_t* Vs = Ks + KVBYTES;
  uint8_t* dSs = Vs + KVBYTES;             // NDS x 16 KB
  uint8_t* Pws = dSs + NDS * 16384;        // NDS x 16 KB
  uint8_t* StgB = Pws + NDS * 16384;       // staging rows of the 8 row warps (32 rows x SLW fp32 columns each)

  __shared__ uint64_t kv_full, qdo_full[4], qdo_free[4], sd_full[2], ds_full[2], ds_free[2], dq_full[2], dq_free[2], all_done;
  __shared__ uint32_t tmem_base_s;
  // metadata of the chunk's owner rows, streamed in blocks of kTB tiles by bulk copies: list entries and weights
  __shared__ __align__(16) int ent_ring[kMS][kTB * 128];
  __shared__ __align__(16) bf16 w_ring[kMS][kTB * 128];
  __shared__ uint64_t meta_full[kMS];
  __shared__ volatile int abort_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nchunk = p.T / 64;
  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const size_t bh = (size_t)b * p.h_kv + h;
  const uint32_t beg = ix.coff[bh * (nchunk + 1) + c];
  const int n_ent = (int)ix.tot[bh * nchunk + c];
  // G divides 128, so it is a power of two: rows map to (pair, group member) by shift and mask (a division by a
  // run-time G in the gather loop cost more than the copies themselves)
  const int G = p.h_q / p.h_kv, gs = 31 - __clz(G), QB = 128 >> gs;
  if (n_ent == 0) {
    // nobody selected this chunk: its key and value gradients are zero
    bf16* dk = static_cast<bf16*>(p.d_k_out) + (((size_t)b * p.T + (size_t)c * 64) * p.h_kv + h) * D;
    bf16* dv = static_cast<bf16*>(p.d_v_out) + (((size_t)b * p.T + (size_t)c * 64) * p.h_kv + h) * D;
    for (int i = tid; i < 64 * PIECES; i += kCmThreads) {
      const size_t off = (size_t)(i / PIECES) * p.h_kv * D + (i % PIECES) * 8;
      *reinterpret_cast<uint4*>(dk + off) = make_uint4(0u, 0u, 0u, 0u);
      *reinterpret_cast<uint4*>(dv + off) = make_uint4(0u, 0u, 0u, 0u);
    }
    return;
  }
  if (cm_failed_before()) return;
  const int ntile = (n_ent + QB - 1) / QB;
  const int32_t* lst = ix.list + bh * ix.cap + beg;
  const bf16* wl = ix.wlist + (bh * ix.cap + beg) * G;

  if (tid == 0) {
    mbar_init(&kv_full, 1);
    for (int s = 0; s < kMS; ++s) mbar_init(&meta_full[s], 1);
    mbar_init(&all_done, 1);
    for (int s = 0; s < NQ; ++s) {
      mbar_init(&qdo_full[s], 1);
      mbar_init(&qdo_free[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sd_full[s], 1);
      mbar_init(&ds_full[s], 128);
      mbar_init(&ds_free[s], 1);
      mbar_init(&dq_full[s], 1);
      mbar_init(&dq_free[s], 128);
    }
    mbar_init_fence();
    abort_s = 0;
  }
  if (warp == 8) tmem_alloc(&tmem_base_s, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  const uint32_t tdK = tmem + C_DK, tdV = tmem + C_DV;

  if (warp == 9) {
    // =============================== gather producer (one warp) =================================
    // The rows of a tile are fetched by TMA gather instructions, four rows each: lane l issues the gathers of rows
    // 4 l .. 4 l + 3 (one per 64-column block).  The TMA unit keeps the requests of several tiles in flight; this
    // warp only reads the tile's list entries and waits for a free ring stage.
    // Metadata block m = tiles kTB m .. kTB m + kTB - 1, slot m % kMS, fetched by bulk copies.  Block m + 1 is requested
    // when block m starts: its slot was last used by block m - 3, i.e. by tiles up to kTB (m - 2) - 1.  The ring wait of
    // tile kTB m has passed by then, which puts the row threads past tile kTB m - NQ - 2 at least, so with NQ <= 4 no
    // thread still reads that slot or waits on its barrier (a waiter two phases behind would never wake).
    const int TBQ = kTB * QB, nblk = (ntile + kTB - 1) / kTB;
    auto request_meta = [&](int m) {
      const int e0 = m * TBQ, ne = min(n_ent - e0, TBQ);
      const uint32_t eb = (uint32_t)(ne * 4 + 15) & ~15u, wb = (uint32_t)(ne * G * 2 + 15) & ~15u;
      mbar_expect_tx(&meta_full[m % kMS], eb + wb);
      bulk_load(ent_ring[m % kMS], lst + e0, eb, &meta_full[m % kMS]);
      bulk_load(w_ring[m % kMS], wl + (size_t)e0 * G, wb, &meta_full[m % kMS]);
    };
    if (lane == 0) {
      request_meta(0);
      if (nblk > 1) request_meta(1);
    }
    const int row_base = (b * p.L) * p.h_q + h * G;      // tensor row of (token 0, first query head of the group)
    bool ok = true;
    for (int j = 0; j < ntile; ++j) {
      const int s = j % NQ;
      if (j >= NQ) {
        ok = cm_wait(&qdo_free[s], ((j / NQ) - 1) & 1) && !abort_s;
        if (!ok) { cm_fail(5010000 + j); break; }
      }
      const int m = j / kTB;
      if (j % kTB == 0) {
        if (m >= 1 && m + 1 < nblk && lane == 0) request_meta(m + 1);
        ok = cm_wait(&meta_full[m % kMS], (m / kMS) & 1);
        if (!ok) { cm_fail(5011000 + j); break; }
      }
      const int* ents = ent_ring[m % kMS] + (j % kTB) * QB;
      int rr[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int row = 4 * lane + i;
        const bool live = j * QB + (row >> gs) < n_ent;      // rows past the end of the list fetch row 0; their P is zero
        rr[i] = live ? row_base + (ents[row >> gs] >> kEntShift) * p.h_q + (row & (G - 1)) : row_base;
      }
      if (lane == 0) mbar_expect_tx(&qdo_full[s], 2 * QBYTES);
      __syncwarp();
#pragma unroll
      for (int db = 0; db < DB; ++db) {
        tma_gather4(Qs + s * QBYTES + db * 16384 + lane * 512, &tmQ, &qdo_full[s], db * 64, rr[0], rr[1], rr[2], rr[3]);
        tma_gather4(dOs + s * QBYTES + db * 16384 + lane * 512, &tmdO, &qdo_full[s], db * 64, rr[0], rr[1], rr[2], rr[3]);
      }
    }
    if (!ok && lane == 0) abort_s = 1;
  } else if (warp == 8) {
    // =============================== TMA (once) + MMA issuer ====================================
    if (lane == 0) {
      mbar_expect_tx(&kv_full, 2 * KVBYTES);
#pragma unroll
      for (int db = 0; db < DB; ++db) {
        tma_load_2d(Ks + db * 8192, &tmK, &kv_full, h * D + db * 64, b * p.T + c * 64);
        tma_load_2d(Vs + db * 8192, &tmV, &kv_full, h * D + db * 64, b * p.T + c * 64);
      }
      constexpr uint32_t idesc_s = idesc_bf16(128, 64, 0);
      constexpr uint32_t idesc_dq = idesc_bf16(128, D, 1);
      constexpr uint32_t idesc_dkv = idesc_bf16(64, D, 1, 1);
      constexpr uint32_t idesc_st = idesc_bf16(128, 128, 1, 1);
      const DescWords q_d = desc_words_sw128(smem_u32(Qs), 16, 1024), do_d = desc_words_sw128(smem_u32(dOs), 16, 1024),
                      k_d = desc_words_sw128(smem_u32(Ks), 16, 1024), v_d = desc_words_sw128(smem_u32(Vs), 16, 1024),
                      kmn_d = desc_words_sw128(smem_u32(Ks), 8192, 1024), dsk_d = desc_words_sw128(smem_u32(dSs), 16, 1024),
                      qmn_d = desc_words_sw128(smem_u32(Qs), 16384, 1024), domn_d = desc_words_sw128(smem_u32(dOs), 16384, 1024),
                      ds_d = desc_words_sw128(smem_u32(dSs), 16384, 1024), pw_d = desc_words_sw128(smem_u32(Pws), 16384, 1024),
                      ast_d = desc_words_sw128(smem_u32(dSs), NDS * 16384, 1024),
                      bst_d = desc_words_sw128(smem_u32(Qs), NQ * QBYTES, 1024);
      bool ok = cm_wait(&kv_full, 0);
      auto issue_sdp = [&](int e) {   // S and dP of tile e
        const int sq = e % NQ, sb = e % NSB;
        ok = cm_wait(&qdo_full[sq], (e / NQ) & 1);
        if (!ok) { cm_fail(5021000 + e); return; }
        tc_fence_after();
        const uint32_t qb = q_d.lo + sq * (QBYTES >> 4), dob = do_d.lo + sq * (QBYTES >> 4);
        const uint32_t ts = tmem + sb * 128;
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
        mma_commit(&sd_full[e & 1]);
      };
      // Barriers are indexed by the tile's parity (= the warpgroup that owns the tile) even where both warpgroups
      // share one buffer: a warpgroup then meets the phases of its barriers in order.  (A parity wait on a barrier
      // whose earlier phase is still open would pass at once.)
      for (int e = 0; ok && e < NSB && e < ntile; ++e) issue_sdp(e);
      for (int j = 0; ok && j < ntile; ++j) {
        const int sq = j % NQ, db = j % NDS, qb = j % NDQ;
        if (abort_s) { ok = false; break; }
        ok = cm_wait(&ds_full[j & 1], (j >> 1) & 1);   // rows of tile j have read S/dP and written dS, wP
        if (!ok) { cm_fail(5022000 + j); break; }
        if (j >= NDQ) {                                   // the dQ tile's previous user (tile j - NDQ) has been read out
          ok = cm_wait(&dq_free[(j - NDQ) & 1], ((j - NDQ) >> 1) & 1);
          if (!ok) { cm_fail(5023000 + j); break; }
        }
        tc_fence_after();
        {
          const uint32_t a0 = dsk_d.lo + db * (16384 >> 4);
          const uint32_t tq = tmem + C_DQ + qb * D;
          mma_ss_w<false>(tq, a0, dsk_d.hi, kmn_d.lo, kmn_d.hi, idesc_dq);
#pragma unroll
          for (int kk = 1; kk < 4; ++kk)
            mma_ss_w<true>(tq, a0 + ((kk * 32) >> 4), dsk_d.hi, kmn_d.lo + ((kk * 2048) >> 4), kmn_d.hi, idesc_dq);
          mma_commit(&dq_full[j & 1]);
        }
        if (kStacked) {
          const uint32_t a0 = ast_d.lo + db * (16384 >> 4), b0 = bst_d.lo + sq * (QBYTES >> 4);
          mma_ss_wr(tdK, a0, ast_d.hi, b0, bst_d.hi, idesc_st, j > 0 ? 1u : 0u);
#pragma unroll
          for (int kk = 1; kk < 8; ++kk)   // 16 rows per step
            mma_ss_w<true>(tdK, a0 + ((kk * 2048) >> 4), ast_d.hi, b0 + ((kk * 2048) >> 4), bst_d.hi, idesc_st);
        } else {
          const uint32_t dsb = ds_d.lo + db * (16384 >> 4), pwb = pw_d.lo + db * (16384 >> 4);
          const uint32_t qmb = qmn_d.lo + sq * (QBYTES >> 4), domb = domn_d.lo + sq * (QBYTES >> 4);
          mma_ss_wr(tdK, dsb, ds_d.hi, qmb, qmn_d.hi, idesc_dkv, j > 0 ? 1u : 0u);
          mma_ss_wr(tdV, pwb, pw_d.hi, domb, domn_d.hi, idesc_dkv, j > 0 ? 1u : 0u);
#pragma unroll
          for (int kk = 1; kk < 8; ++kk) {
            mma_ss_w<true>(tdK, dsb + ((kk * 2048) >> 4), ds_d.hi, qmb + ((kk * 2048) >> 4), qmn_d.hi, idesc_dkv);
            mma_ss_w<true>(tdV, pwb + ((kk * 2048) >> 4), pw_d.hi, domb + ((kk * 2048) >> 4), domn_d.hi, idesc_dkv);
          }
        }
        mma_commit(&ds_free[j & 1]);
        mma_commit(&qdo_free[sq]);
        // The S/dP accumulator of tile j is free again.  Tile j + NSB goes after tile j's products, so the release of
        // tile j's ring stage never waits for a gather.
        if (j + NSB < ntile) issue_sdp(j + NSB);
      }
      if (ok) mma_commit(&all_done);
      if (!ok) { abort_s = 1; cm_fail(5029999); }
    }
  } else {
    // =============================== row warpgroups ==============================================
    const int r = tid & 127, wg = tid >> 7;                 // warpgroup wg takes tiles wg, wg + 2, ...
    const int g = r & (G - 1), hq = h * G + g, rp = r >> gs;
    const float scale_log2 = p.scale * kLog2e;
    const float slope = p.slope ? p.slope[hq] : 0.f;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    bf16* dwbase = static_cast<bf16*>(p.d_w);
    bool ok = true;
    for (int j = wg, u = 0; j < ntile; j += 2, ++u) {
      const int sb = j % NSB, db = j % NDS, qb = j % NDQ;
      ok = cm_wait(&sd_full[wg], u & 1);
      if (!ok) cm_fail(5031000 + j);
      ok = __all_sync(0xffffffffu, ok) && !abort_s;
      if (!ok) break;
      tc_fence_after();
      const int m = j / kTB;
      ok = cm_wait(&meta_full[m % kMS], (m / kMS) & 1);
      ok = __all_sync(0xffffffffu, ok) && !abort_s;
      if (!ok) break;
      const bool live = j * QB + rp < n_ent;
      const int ent = live ? ent_ring[m % kMS][(j % kTB) * QB + rp] : 0;
      const int k = ent & kEntSlotMask;
      const float wv = live ? to_f(w_ring[m % kMS][(j % kTB) * 128 + r]) : 0.f;
      const int rowt = live ? (int)(((int64_t)b * p.L + (ent >> kEntShift)) * p.h_q + hq) : -1;
      float sv[64], dp[64];
      const uint32_t tsd = tmem + lane_base + sb * 128;
      tmem_ld32(tsd, sv);
      tmem_ld32(tsd + 32, sv + 32);
      tmem_ld_wait();
      tmem_ld32(tsd + 64, dp);          // in flight while the S row is exponentiated
      tmem_ld32(tsd + 96, dp + 32);
      float esum = 1.f;
      if (live) esum = bwd_row_exp(sv, scale_log2, slope, p.mask_last);
      tmem_ld_wait64(dp);
      float dw = 0.f;
      if (live) dw = bwd_row_grad<true>(sv, dp, esum, wv, p.scale);
      if (j >= NDS) {                   // the dS / wP tile was last read by the products of tile j - NDS
        ok = cm_wait(&ds_free[(j - NDS) & 1], ((j - NDS) >> 1) & 1);
        if (!ok) cm_fail(5032000 + j);
        ok = __all_sync(0xffffffffu, ok) && !abort_s;
        if (!ok) break;
      }
      if (live) {
        store_row_bf16_sw128(dSs + db * 16384, r, sv);
        store_row_bf16_sw128(Pws + db * 16384, r, dp);
        dwbase[(int64_t)rowt * p.num_weights + k] = __float2bfloat16_rn(dw);
      } else {
        store_row_zero_sw128(dSs + db * 16384, r);
        store_row_zero_sw128(Pws + db * 16384, r);
      }
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(&ds_full[wg]);
      ok = cm_wait(&dq_full[wg], u & 1);
      if (!ok) cm_fail(5034000 + j);
      ok = __all_sync(0xffffffffu, ok) && !abort_s;
      if (!ok) break;
      tc_fence_after();
      // dQ tile -> fp32 accumulator rows of the tokens, SLW columns at a time
#pragma unroll
      for (int sl = 0; sl < NS; ++sl)
        scatter_slice<SLW>(StgB + warp * StgGeom<SLW>::kWarpBytes, tmem + lane_base + C_DQ + qb * D + sl * SLW, rowt, dq_acc, D,
                           sl * SLW, lane);
      tc_fence_before();
      mbar_arrive(&dq_free[wg]);
    }
    // ---- dK, dV of the chunk: TMEM -> bf16 -> global, once -------------------------------------
    if (ok) {
      ok = cm_wait(&all_done, 0);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (!ok && lane == 0) { abort_s = 1; cm_fail(5039999); }
    if (ok) tc_fence_after();
    if (kStacked) {
      // stacked accumulator (M = 128): TMEM lane = row; rows 0..63 hold dK in columns 0..63, rows 64..127 hold dV in
      // columns 64..127.  Warps 0, 1 of a warpgroup write dK rows, warps 2, 3 dV rows; warpgroup w takes the 32-column
      // half w.
      const int wq = warp & 3;
      const bool is_v = wq >= 2;
      const int64_t tokr = (int64_t)b * p.T + (int64_t)c * 64 + 32 * (wq & 1) + lane;
      float ov[32];
      if (ok) {
        tmem_ld32(tdK + lane_base + (is_v ? 64 : 0) + wg * 32, ov);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) ov[jj] = 0.f;
      }
      store32_bf16(static_cast<bf16*>(is_v ? p.d_v_out : p.d_k_out) + (tokr * p.h_kv + h) * D + wg * 32, ov);
    } else {
      // M = 64 accumulators: key row 16 * warp + lane lives in TMEM lane 32 * warp + lane, lanes 0..15 of each warp;
      // warpgroup 0 writes dK, warpgroup 1 writes dV
      const int krow = 16 * (warp & 3) + lane;
      const int64_t tok = (int64_t)b * p.T + (int64_t)c * 64 + krow;
      bf16* dst = static_cast<bf16*>(wg ? p.d_v_out : p.d_k_out) + (tok * p.h_kv + h) * D;
#pragma unroll
      for (int cb = 0; cb < D / 32; ++cb) {
        float ov[32];
        if (ok) {
          tmem_ld32((wg ? tdV : tdK) + lane_base + cb * 32, ov);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int jj = 0; jj < 32; ++jj) ov[jj] = 0.f;
        }
        if (lane < 16) store32_bf16(dst + cb * 32, ov);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 8) tmem_dealloc(tmem, 512);
}

static size_t cm_bwd_smem(int D) {
  const int NQ = (D == 64) ? 3 : 2, NDS = (D == 64) ? 2 : 1;
  return 1024 + 2 * (size_t)NQ * (D / 64) * 16384 + 2 * (size_t)(D / 64) * 8192 + 2 * (size_t)NDS * 16384 +
         8 * (D == 64 ? (size_t)StgGeom<32>::kWarpBytes : (size_t)StgGeom<16>::kWarpBytes);
}

// workspace of the chunk-major backward: inverse index + fp32 dQ accumulator (0: shape outside this path)
size_t sparse_bwd_cm_workspace(const SparseParams& p) {
  if (!cm_shape_ok(p)) return 0;
  const InvLayout l = inv_layout(p.B, p.L, p.h_kv, p.h_q / p.h_kv, p.K, p.T / 64);
  return l.total + (size_t)p.B * p.L * p.h_q * p.D * sizeof(float);
}

// built_index: the index a forward call over the same ids and weights left in its workspace, or null to build it here
int sparse_bwd_cm_launch(const SparseParams& p, void* d_k, void* d_v, void* workspace, cudaStream_t st, const void* built_index) {
  if (!cm_shape_ok(p) || !workspace) return HILS_ERR_UNSUPPORTED;
  if (((uintptr_t)p.q | (uintptr_t)p.k | (uintptr_t)p.v | (uintptr_t)p.d_o | (uintptr_t)p.d_q | (uintptr_t)d_k | (uintptr_t)d_v |
       (uintptr_t)workspace) & 15)
    return HILS_ERR_UNSUPPORTED;
  const int D = p.D, nchunk = p.T / 64;
  const InvLayout l = inv_layout(p.B, p.L, p.h_kv, p.h_q / p.h_kv, p.K, nchunk);
  InvIndex ix;
  if (built_index) {
    if ((uintptr_t)built_index & 15) return HILS_ERR_UNSUPPORTED;
    adopt_inverse_index(p, built_index, &ix);
  } else if (int rc = build_inverse_index(p, workspace, &ix, st)) {
    return rc;
  }
  float* dq_acc = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + l.total);
  const size_t n_q = (size_t)p.B * p.L * p.h_q * D;
  cudaError_t e = cudaMemsetAsync(dq_acc, 0, n_q * sizeof(float), st);
  if (e == cudaSuccess) e = cudaMemsetAsync(p.d_w, 0, (size_t)p.B * p.L * p.h_q * p.num_weights * 2, st);
  if (e == cudaSuccess && p.T % 64 != 0) {   // tokens after the last full chunk belong to no chunk
    e = cudaMemsetAsync(d_k, 0, (size_t)p.B * p.T * p.h_kv * D * 2, st);
    if (e == cudaSuccess) e = cudaMemsetAsync(d_v, 0, (size_t)p.B * p.T * p.h_kv * D * 2, st);
  }
  if (e != cudaSuccess) return cuda_fail(e, "sparse_attn_bwd accumulator clear");
  SparseParams pp = p;
  pp.d_k_out = d_k;
  pp.d_v_out = d_v;
  CUtensorMap tmK, tmV;
  if (int rc = make_tmap_bf16_rows(&tmK, p.k, (uint64_t)p.B * p.T, (uint64_t)p.h_kv * D, (uint64_t)p.h_kv * D, 64)) return rc;
  if (int rc = make_tmap_bf16_rows(&tmV, p.v, (uint64_t)p.B * p.T, (uint64_t)p.h_kv * D, (uint64_t)p.h_kv * D, 64)) return rc;
  CUtensorMap tmQ, tmdO;   // rows = (batch, token, query head), one row per box: the sources of the row gathers
  if (int rc = make_tmap_bf16_rows(&tmQ, p.q, (uint64_t)p.B * p.L * p.h_q, D, D, 1)) return rc;
  if (int rc = make_tmap_bf16_rows(&tmdO, p.d_o, (uint64_t)p.B * p.L * p.h_q, D, D, 1)) return rc;
  const size_t smem = cm_bwd_smem(D);
  dim3 grid(nchunk, p.h_kv, p.B);
  if (D == 64) {
    cudaFuncSetAttribute(sparse_bwd_cm_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sparse_bwd_cm_kernel<64><<<grid, kCmThreads, smem, st>>>(pp, ix, dq_acc, tmK, tmV, tmQ, tmdO);
  } else {
    cudaFuncSetAttribute(sparse_bwd_cm_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sparse_bwd_cm_kernel<128><<<grid, kCmThreads, smem, st>>>(pp, ix, dq_acc, tmK, tmV, tmQ, tmdO);
  }
  cm_round_kernel<<<(unsigned)((n_q / 8 + 255) / 256), 256, 0, st>>>(dq_acc, static_cast<bf16*>(p.d_q), (int64_t)(n_q / 8));
  HILS_LAUNCH_CHECK("sparse_attn_bwd (chunk-major path)");
  return HILS_OK;
}

// device-side error word of this file's kernels (0 = none); synchronises and clears
int take_status_sparse_cm() {
  int v = 0, zero = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  if (cudaMemcpyFromSymbol(&v, g_cm_status, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(g_cm_status, &zero, sizeof(int));
  return v;
}

}  // namespace hils
