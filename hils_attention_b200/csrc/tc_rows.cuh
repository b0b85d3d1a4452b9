// Row helpers shared by the tensor-core kernels: one thread owns one row of a [128 x 64] tile.
#pragma once
#include "common.cuh"
#include "umma.cuh"

namespace hils {

using umma::sw128_off;

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

}  // namespace hils
