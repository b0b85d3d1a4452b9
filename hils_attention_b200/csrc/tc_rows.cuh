// Row helpers shared by the tensor-core kernels: one thread owns one row of a [128 x 64] tile.
#pragma once
#include "common.cuh"
#include "umma.cuh"

namespace hils {

using umma::sw128_off;

constexpr float kLog2e = 1.4426950408889634f;

// 64 fp32 values -> bf16 row of a [128 x 128 B] tile stored with the 128-byte swizzle
__device__ __forceinline__ void store_row_bf16_sw128(uint8_t* tile, int r, const float* v) {
#pragma unroll
  for (int c8 = 0; c8 < 8; ++c8) {
    __nv_bfloat162 hh[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) hh[e] = __floats2bfloat162_rn(v[c8 * 8 + 2 * e], v[c8 * 8 + 2 * e + 1]);
    *reinterpret_cast<uint4*>(tile + sw128_off(r, c8)) = *reinterpret_cast<uint4*>(hh);
  }
}
__device__ __forceinline__ void store_row_zero_sw128(uint8_t* tile, int r) {
#pragma unroll
  for (int c8 = 0; c8 < 8; ++c8) *reinterpret_cast<uint4*>(tile + sw128_off(r, c8)) = make_uint4(0u, 0u, 0u, 0u);
}


// copy this thread's row (D bf16, contiguous in global memory) into a [128 x D] swizzled tile made of
// D/64 column blocks of 16 KB; rows that do not exist are zero-filled
template <int D>
__device__ __forceinline__ void load_row_to_tile(uint8_t* tile, int r, const bf16* row, bool valid) {
#pragma unroll
  for (int c = 0; c < D / 8; ++c) {
    uint4 x = make_uint4(0u, 0u, 0u, 0u);
    if (valid) x = *reinterpret_cast<const uint4*>(row + c * 8);
    *reinterpret_cast<uint4*>(tile + (c >> 3) * 16384 + sw128_off(r, c & 7)) = x;
  }
}

// 32 fp32 values -> 32 bf16 written to global memory (64 B)
__device__ __forceinline__ void store32_bf16(bf16* dst, const float* v) {
#pragma unroll
  for (int c8 = 0; c8 < 4; ++c8) {
    __nv_bfloat162 hh[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) hh[e] = __floats2bfloat162_rn(v[c8 * 8 + 2 * e], v[c8 * 8 + 2 * e + 1]);
    *reinterpret_cast<uint4*>(dst + c8 * 8) = *reinterpret_cast<uint4*>(hh);
  }
}

// Backward row arithmetic in two phases, so that the dP row can still be in flight from TMEM while the
// first phase works on the S row.
// Phase A: S row in sv  ->  e_j = exp(scale (S_j - max)) in sv; returns sum_j e_j.
__device__ __forceinline__ float bwd_row_exp(float* sv, float scale_log2, float slope, int mask_last) {
  if (slope != 0.f) {
#pragma unroll
    for (int j = 0; j < 62; ++j) sv[j] -= slope * (float)(62 - j);
  }
  if (mask_last) sv[63] = -CUDART_INF_F;
  // reductions use four interleaved partial accumulators: a single dependent chain of 64 operations
  // would leave the thread waiting on arithmetic latency most of the time
  float m4[4] = {sv[0], sv[1], sv[2], sv[3]};
#pragma unroll
  for (int j = 4; j < 64; ++j) m4[j & 3] = fmaxf(m4[j & 3], sv[j]);
  const float m = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
  const float mb = m * scale_log2;
  float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int j = 0; j < 64; ++j) {
    sv[j] = umma::ex2(fmaf(sv[j], scale_log2, -mb));
    s4[j & 3] += sv[j];
  }
  return (s4[0] + s4[1]) + (s4[2] + s4[3]);
}
// Phase B: e row in sv, dP row in dp  ->  dS row in sv (= scale w P (dP - dw)) and, when kWantWP, the
// w*P row in dp; returns dw = sum_j P_j dP_j.  P_j = e_j / sum is never formed: the factors fold into
// one multiplier per product.
template <bool kWantWP>
__device__ __forceinline__ float bwd_row_grad(float* sv, float* dp, float sum, float wsum, float scale) {
  const float inv = 1.f / sum;
  float d4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int j = 0; j < 64; ++j) d4[j & 3] = fmaf(sv[j], dp[j], d4[j & 3]);
  const float dw = ((d4[0] + d4[1]) + (d4[2] + d4[3])) * inv;
  const float c = scale * wsum * inv, cdw = -c * dw, wp = wsum * inv;
#pragma unroll
  for (int j = 0; j < 64; ++j) {
    const float e = sv[j];
    sv[j] = e * fmaf(c, dp[j], cdw);
    if (kWantWP) dp[j] = wp * e;
  }
  return dw;
}

}  // namespace hils
