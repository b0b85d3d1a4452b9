// Shared helpers for the hils_b200 kernels: element-type loads/stores, warp reductions,
// error reporting of the C ABI.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/hils_b200.h"

namespace hils {

typedef __nv_bfloat16 bf16;

// ---- error text of the C ABI (per host thread) -------------------------------------------
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

#define HILS_REQUIRE(cond, ...)            \
  do {                                     \
    if (!(cond)) {                         \
      hils::set_error(__VA_ARGS__);        \
      return HILS_ERR_BAD_ARG;             \
    }                                      \
  } while (0)

#define HILS_LAUNCH_CHECK(what)                               \
  do {                                                        \
    cudaError_t _e = cudaGetLastError();                      \
    if (_e != cudaSuccess) return hils::cuda_fail(_e, what);  \
  } while (0)

// ---- element access ------------------------------------------------------------------------
__device__ __forceinline__ float to_f(float x) { return x; }
__device__ __forceinline__ float to_f(bf16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float x) { return __float2bfloat16_rn(x); }

// Load 4 consecutive elements as floats (p must be 16-byte aligned for float, 8-byte for bf16).
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const bf16* p) {
  uint2 u = *reinterpret_cast<const uint2*>(p);
  __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&u.x);
  __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162*>(&u.y);
  float2 fa = __bfloat1622float2(a), fb = __bfloat1622float2(b);
  return make_float4(fa.x, fa.y, fb.x, fb.y);
}
// Load 2 consecutive elements as floats
__device__ __forceinline__ float2 load2(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 load2(const bf16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&a);
  u.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}

// ---- warp reductions -----------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// dot of a float vector in shared memory with a row of T in global memory (D % 4 == 0)
template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ qs, const T* __restrict__ row, int D) {
  float acc = 0.f;
  for (int d = 0; d < D; d += 4) {
    float4 a = *reinterpret_cast<const float4*>(qs + d);
    float4 b = load4(row + d);
    acc = fmaf(a.x, b.x, acc);
    acc = fmaf(a.y, b.y, acc);
    acc = fmaf(a.z, b.z, acc);
    acc = fmaf(a.w, b.w, acc);
  }
  return acc;
}

__host__ __device__ __forceinline__ int floor_div(int a, int b) {
  int q = a / b;
  return ((a % b != 0) && ((a < 0) != (b < 0))) ? q - 1 : q;
}

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// fp32 accumulator -> element type, 4 elements per thread
template <typename T>
__global__ void cast_from_f32_kernel(const float* __restrict__ src, T* __restrict__ dst, int64_t n4) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n4) store4(dst + i * 4, *reinterpret_cast<const float4*>(src + i * 4));
}

template <typename T>
inline void launch_cast_from_f32(const float* src, T* dst, int64_t n, cudaStream_t st) {
  const int64_t n4 = n / 4;
  if (n4 > 0) cast_from_f32_kernel<T><<<(unsigned)((n4 + 255) / 256), 256, 0, st>>>(src, dst, n4);
}

}  // namespace hils
