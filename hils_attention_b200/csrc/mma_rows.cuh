// Few query rows against many bf16 key rows on the warp-level tensor cores, without shared-memory staging.
//
// mma.sync.m16n8k16 wants, per thread, B registers b0 = B[k=2j,2j+1][n] and b1 = B[k=2j+8,2j+9][n]
// (j = lane%4, n = lane/4).  A dot product does not care about the order of its D terms, so the k index
// of every pair of k-steps is permuted such that a thread's four B registers of the pair are eight
// CONSECUTIVE bf16 of one key row: lane (n, j) reads 16 bytes = elements 32s+8j .. 32s+8j+7 of key n;
// elements 0,1 / 2,3 feed k-step 2s, elements 4,5 / 6,7 feed k-step 2s+1.  The A fragments (query rows)
// are built with the same permutation.  Every 64-byte segment a warp load touches is fully used.
#pragma once
#include "common.cuh"

namespace hils {

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// A fragments of up to 16 query rows held as fp32 in q_s[row][D] (rows >= G read as zero); NK = D/16.
// `row_of(r)` maps fragment row r (0..15) to the row of q_s, or -1 for a zero row.
template <int NK, typename RowOf>
__device__ __forceinline__ void make_q_frags(const float* q_s, int lane, uint32_t (&af)[NK][4], RowOf row_of) {
  constexpr int D = NK * 16;
  const int r0 = row_of(lane >> 2), r1 = row_of((lane >> 2) + 8), j = lane & 3;
#pragma unroll
  for (int kk = 0; kk < NK; ++kk) {
    const int d = 32 * (kk >> 1) + 8 * j + 4 * (kk & 1);
    const float* a = q_s + max(r0, 0) * D + d;
    const float* b = q_s + max(r1, 0) * D + d;
    af[kk][0] = (r0 >= 0) ? pack_bf16(a[0], a[1]) : 0u;
    af[kk][1] = (r1 >= 0) ? pack_bf16(b[0], b[1]) : 0u;
    af[kk][2] = (r0 >= 0) ? pack_bf16(a[2], a[3]) : 0u;
    af[kk][3] = (r1 >= 0) ? pack_bf16(b[2], b[3]) : 0u;
  }
}

// Dot products of the fragment rows with 32 consecutive key rows (row stride rs elements, rows >= n are
// clamped to row n-1: the caller ignores them).  c[u] = accumulators of keys 8u .. 8u+7:
// c[u][0..1] = row lane/4, keys 8u+2j, 8u+2j+1;  c[u][2..3] = row lane/4+8, same keys.
template <int NK>
__device__ __forceinline__ void dot32_mma(const uint32_t (&af)[NK][4], const bf16* kbase, int64_t rs, int n, int lane,
                                          float (&c)[4][4]) {
  const int kr = lane >> 2, j = lane & 3;
  uint4 kv[4][NK / 2];
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int key = min(u * 8 + kr, n - 1);
    const bf16* row = kbase + (int64_t)key * rs + 8 * j;
#pragma unroll
    for (int s = 0; s < NK / 2; ++s) kv[u][s] = *reinterpret_cast<const uint4*>(row + 32 * s);
  }
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    c[u][0] = c[u][1] = c[u][2] = c[u][3] = 0.f;
#pragma unroll
    for (int s = 0; s < NK / 2; ++s) {
      asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                   : "+f"(c[u][0]), "+f"(c[u][1]), "+f"(c[u][2]), "+f"(c[u][3])
                   : "r"(af[2 * s][0]), "r"(af[2 * s][1]), "r"(af[2 * s][2]), "r"(af[2 * s][3]), "r"(kv[u][s].x), "r"(kv[u][s].y));
      asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                   : "+f"(c[u][0]), "+f"(c[u][1]), "+f"(c[u][2]), "+f"(c[u][3])
                   : "r"(af[2 * s + 1][0]), "r"(af[2 * s + 1][1]), "r"(af[2 * s + 1][2]), "r"(af[2 * s + 1][3]), "r"(kv[u][s].z),
                     "r"(kv[u][s].w));
    }
  }
}

// out[g * ostride + j] = <q_g, K_j> for j < n <= 64
template <int NK>
__device__ __forceinline__ void score_rows_mma(const uint32_t (&af)[NK][4], const bf16* kbase, int64_t rs, int n, int G,
                                               float* out, int ostride, int lane) {
  const int kr = lane >> 2, j = lane & 3;
#pragma unroll
  for (int k0 = 0; k0 < 64; k0 += 32) {       // unrolled: the loads of the second group may start before the first's math
    if (k0 >= n) break;
    float c[4][4];
    dot32_mma<NK>(af, kbase + (int64_t)k0 * rs, rs, n - k0, lane, c);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int key0 = k0 + u * 8 + 2 * j;
      if (kr < G) {
        if (key0 < n) out[kr * ostride + key0] = c[u][0];
        if (key0 + 1 < n) out[kr * ostride + key0 + 1] = c[u][1];
      }
      if (kr + 8 < G) {
        if (key0 < n) out[(kr + 8) * ostride + key0] = c[u][2];
        if (key0 + 1 < n) out[(kr + 8) * ostride + key0 + 1] = c[u][3];
      }
    }
  }
}

// acc[g][0..7] += sum_j p[g * pstride + j] * V_j[sub*8 .. sub*8+7] over the rows this lane's group visits
template <int NK, int GM>
__device__ __forceinline__ void pv_rows16(const float* p_s, int pstride, const bf16* vbase, int64_t rs, int n, int G,
                                          float (&acc)[GM][8], int lane) {
  constexpr int LPR = 2 * NK, RPI = 32 / LPR;          // lanes per row, rows per load instruction
  const int sub = lane % LPR, rg = lane / LPR;
  for (int j0 = 0; j0 < n; j0 += RPI * 8) {
    uint4 vv[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int jr = min(j0 + u * RPI + rg, n - 1);
      vv[u] = *reinterpret_cast<const uint4*>(vbase + (int64_t)jr * rs + sub * 8);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int jr = j0 + u * RPI + rg;
      if (jr < n) {
        const uint32_t w4[4] = {vv[u].x, vv[u].y, vv[u].z, vv[u].w};
        float f[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          f[2 * e] = __uint_as_float(w4[e] << 16);
          f[2 * e + 1] = __uint_as_float(w4[e] & 0xffff0000u);
        }
#pragma unroll
        for (int g = 0; g < GM; ++g) {
          if (g < G) {
            const float pj = p_s[g * pstride + jr];
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[g][e] = fmaf(pj, f[e], acc[g][e]);
          }
        }
      }
    }
  }
}

// sum over the row groups of a warp; afterwards lanes < D/8 hold the totals of columns lane*8 .. lane*8+7
template <int NK, int GM>
__device__ __forceinline__ void pv_reduce(float (&acc)[GM][8]) {
  constexpr int LPR = 2 * NK;
#pragma unroll
  for (int off = LPR; off < 32; off <<= 1)
#pragma unroll
    for (int g = 0; g < GM; ++g)
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[g][e] += __shfl_xor_sync(0xffffffffu, acc[g][e], off);
}

}  // namespace hils
