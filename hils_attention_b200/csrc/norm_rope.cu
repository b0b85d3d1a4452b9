// Per-head RMSNorm followed by the rotary embedding, one pass over the tensor, forward and backward.
//
// Upstream of the attention path the reference normalises q, k and the landmark query per head
// (models/FlashHiLS/modeling_olmo_hils.py:105-111: fp32 statistics, the normalised tensor rounded to the
// input dtype, then multiplied by the weight) and rotates them (ops/rope_tilelang_fp32.py:96-181: fp32
// x*cos + rotate_half(x)*sin, rounded once; backward = the same rotation with -sin).  As separate ops that
// is three reads and three writes of the tensor; here one warp owns a (token, head) row, keeps it in
// registers and reads/writes it once.  Lane l holds the rotation pairs (d, d + D/2) for d = l, l+32, ...
#include "common.cuh"

namespace hils {

constexpr int kNrWarps = 8;
constexpr int kNrMaxPairs = 4;     // D <= 256

struct NormRopeParams {
  const void* x; const void* weight; const void* cos; const void* sin;
  void* out; float* rstd;
  const void* d_out; void* d_x; float* d_weight;
  int64_t rows;        // B * L * H
  int L, H, D, cos_batched, cs_f32;
  float eps;
};

template <typename CS>
__device__ __forceinline__ float cs_at(const void* p, int64_t i) { return to_f(static_cast<const CS*>(p)[i]); }

template <typename T>
__global__ void __launch_bounds__(32 * kNrWarps) norm_rope_fwd_kernel(NormRopeParams p) {
  const int lane = threadIdx.x & 31;
  const int half = p.D >> 1, npair = (half + 31) >> 5;
  const T* x = static_cast<const T*>(p.x);
  T* out = static_cast<T*>(p.out);
  const T* w = static_cast<const T*>(p.weight);
  for (int64_t r = (int64_t)blockIdx.x * kNrWarps + (threadIdx.x >> 5); r < p.rows; r += (int64_t)gridDim.x * kNrWarps) {
    const int64_t tok = r / p.H;                           // b * L + l
    const int64_t cs_row = (p.cos_batched ? tok : tok % p.L) * p.D;
    float lo[kNrMaxPairs], hi[kNrMaxPairs];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kNrMaxPairs; ++i) {
      const int d = lane + 32 * i;
      lo[i] = hi[i] = 0.f;
      if (i < npair && d < half) {
        lo[i] = to_f(x[r * p.D + d]);
        hi[i] = to_f(x[r * p.D + d + half]);
        ss = fmaf(lo[i], lo[i], fmaf(hi[i], hi[i], ss));
      }
    }
    if (w) {
      ss = warp_sum(ss);
      const float rstd = rsqrtf(ss / (float)p.D + p.eps);
      if (lane == 0 && p.rstd) p.rstd[r] = rstd;
#pragma unroll
      for (int i = 0; i < kNrMaxPairs; ++i) {
        const int d = lane + 32 * i;
        if (i < npair && d < half) {
          lo[i] = to_f(from_f<T>(to_f(w[d]) * to_f(from_f<T>(lo[i] * rstd))));
          hi[i] = to_f(from_f<T>(to_f(w[d + half]) * to_f(from_f<T>(hi[i] * rstd))));
        }
      }
    }
#pragma unroll
    for (int i = 0; i < kNrMaxPairs; ++i) {
      const int d = lane + 32 * i;
      if (i < npair && d < half) {
        float o1 = lo[i], o2 = hi[i];
        if (p.cos) {
          float c1, s1, c2, s2;
          if (p.cs_f32) {
            c1 = cs_at<float>(p.cos, cs_row + d); s1 = cs_at<float>(p.sin, cs_row + d);
            c2 = cs_at<float>(p.cos, cs_row + d + half); s2 = cs_at<float>(p.sin, cs_row + d + half);
          } else {
            c1 = cs_at<bf16>(p.cos, cs_row + d); s1 = cs_at<bf16>(p.sin, cs_row + d);
            c2 = cs_at<bf16>(p.cos, cs_row + d + half); s2 = cs_at<bf16>(p.sin, cs_row + d + half);
          }
          o1 = lo[i] * c1 - hi[i] * s1;
          o2 = hi[i] * c2 + lo[i] * s2;
        }
        out[r * p.D + d] = from_f<T>(o1);
        out[r * p.D + d + half] = from_f<T>(o2);
      }
    }
  }
}

// d_y = rotation of d_out with -sin (rounded to T, as the rotary op's own backward returns it);
// RMSNorm backward: n = x*rstd, dn = d_y*w, d_x = rstd*(dn - n*mean(dn*n)), d_w += d_y*n.
template <typename T>
__global__ void __launch_bounds__(32 * kNrWarps) norm_rope_bwd_kernel(NormRopeParams p) {
  __shared__ float dw_s[kNrWarps][64 * kNrMaxPairs];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int half = p.D >> 1, npair = (half + 31) >> 5;
  const T* x = static_cast<const T*>(p.x);
  const T* go = static_cast<const T*>(p.d_out);
  T* dx = static_cast<T*>(p.d_x);
  const T* w = static_cast<const T*>(p.weight);
  float dwl[kNrMaxPairs], dwh[kNrMaxPairs];
#pragma unroll
  for (int i = 0; i < kNrMaxPairs; ++i) dwl[i] = dwh[i] = 0.f;
  for (int64_t r = (int64_t)blockIdx.x * kNrWarps + warp; r < p.rows; r += (int64_t)gridDim.x * kNrWarps) {
    const int64_t tok = r / p.H;
    const int64_t cs_row = (p.cos_batched ? tok : tok % p.L) * p.D;
    float gl[kNrMaxPairs], gh[kNrMaxPairs], nl[kNrMaxPairs], nh[kNrMaxPairs];
    const float rstd = w ? p.rstd[r] : 1.f;
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < kNrMaxPairs; ++i) {
      const int d = lane + 32 * i;
      gl[i] = gh[i] = nl[i] = nh[i] = 0.f;
      if (i < npair && d < half) {
        float g1 = to_f(go[r * p.D + d]), g2 = to_f(go[r * p.D + d + half]);
        if (p.cos) {
          float c1, s1, c2, s2;
          if (p.cs_f32) {
            c1 = cs_at<float>(p.cos, cs_row + d); s1 = cs_at<float>(p.sin, cs_row + d);
            c2 = cs_at<float>(p.cos, cs_row + d + half); s2 = cs_at<float>(p.sin, cs_row + d + half);
          } else {
            c1 = cs_at<bf16>(p.cos, cs_row + d); s1 = cs_at<bf16>(p.sin, cs_row + d);
            c2 = cs_at<bf16>(p.cos, cs_row + d + half); s2 = cs_at<bf16>(p.sin, cs_row + d + half);
          }
          // transpose of (o1 = y1 c1 - y2 s1, o2 = y2 c2 + y1 s2)
          const float y1 = g1 * c1 + g2 * s2, y2 = g2 * c2 - g1 * s1;
          g1 = to_f(from_f<T>(y1));
          g2 = to_f(from_f<T>(y2));
        }
        gl[i] = g1; gh[i] = g2;
        if (w) {
          nl[i] = to_f(x[r * p.D + d]) * rstd;
          nh[i] = to_f(x[r * p.D + d + half]) * rstd;
          dwl[i] = fmaf(g1, nl[i], dwl[i]);
          dwh[i] = fmaf(g2, nh[i], dwh[i]);
          gl[i] = g1 * to_f(w[d]);
          gh[i] = g2 * to_f(w[d + half]);
          dot = fmaf(gl[i], nl[i], fmaf(gh[i], nh[i], dot));
        }
      }
    }
    if (w) dot = warp_sum(dot) / (float)p.D;
#pragma unroll
    for (int i = 0; i < kNrMaxPairs; ++i) {
      const int d = lane + 32 * i;
      if (i < npair && d < half) {
        dx[r * p.D + d] = from_f<T>(w ? rstd * (gl[i] - nl[i] * dot) : gl[i]);
        dx[r * p.D + d + half] = from_f<T>(w ? rstd * (gh[i] - nh[i] * dot) : gh[i]);
      }
    }
  }
  if (w && p.d_weight) {
#pragma unroll
    for (int i = 0; i < kNrMaxPairs; ++i) {
      dw_s[warp][lane + 32 * i] = dwl[i];
      dw_s[warp][64 * kNrMaxPairs / 2 + lane + 32 * i] = dwh[i];
    }
    __syncthreads();
    for (int e = threadIdx.x; e < p.D; e += 32 * kNrWarps) {
      const int slot = (e < half) ? e : 64 * kNrMaxPairs / 2 + (e - half);
      float s = 0.f;
      for (int wv = 0; wv < kNrWarps; ++wv) s += dw_s[wv][slot];
      if (s != 0.f) atomicAdd(p.d_weight + e, s);
    }
  }
}

static int check_norm_rope(int B, int L, int H, int D, int dtype, int cs_dtype, const void* cos, const void* sin) {
  HILS_REQUIRE(B > 0 && L >= 0 && H > 0 && D > 0, "norm_rope: bad size");
  HILS_REQUIRE(D % 2 == 0 && D <= 64 * kNrMaxPairs, "norm_rope: D (%d) must be even and at most 256", D);
  HILS_REQUIRE(dtype == HILS_BF16 || dtype == HILS_F32, "norm_rope: unknown dtype %d", dtype);
  HILS_REQUIRE(cs_dtype == HILS_BF16 || cs_dtype == HILS_F32, "norm_rope: unknown cos/sin dtype %d", cs_dtype);
  HILS_REQUIRE((cos == nullptr) == (sin == nullptr), "norm_rope: cos and sin go together");
  return HILS_OK;
}

}  // namespace hils

using namespace hils;

static unsigned norm_rope_grid(int64_t rows) {
  const int64_t ctas = (rows + kNrWarps - 1) / kNrWarps;
  return (unsigned)std::min<int64_t>(ctas, 148 * 16);
}

extern "C" int hils_norm_rope_fwd(const void* x, const void* weight, const void* cos, const void* sin, void* out,
                                  float* rstd, int B, int L, int H, int D, int cos_batched, float eps, int dtype,
                                  int cs_dtype, void* stream) {
  if (int rc = check_norm_rope(B, L, H, D, dtype, cs_dtype, cos, sin)) return rc;
  const int64_t rows = (int64_t)B * L * H;
  if (rows == 0) return HILS_OK;
  HILS_REQUIRE(x && out, "norm_rope_fwd: null pointer");
  NormRopeParams p = {};
  p.x = x; p.weight = weight; p.cos = cos; p.sin = sin; p.out = out; p.rstd = rstd;
  p.rows = rows; p.L = L; p.H = H; p.D = D; p.cos_batched = cos_batched; p.cs_f32 = cs_dtype == HILS_F32; p.eps = eps;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == HILS_BF16) norm_rope_fwd_kernel<bf16><<<norm_rope_grid(rows), 32 * kNrWarps, 0, st>>>(p);
  else norm_rope_fwd_kernel<float><<<norm_rope_grid(rows), 32 * kNrWarps, 0, st>>>(p);
  HILS_LAUNCH_CHECK("norm_rope_fwd");
  return HILS_OK;
}

extern "C" int hils_norm_rope_bwd(const void* x, const void* weight, const void* cos, const void* sin,
                                  const float* rstd, const void* d_out, void* d_x, float* d_weight, int B, int L,
                                  int H, int D, int cos_batched, int dtype, int cs_dtype, void* stream) {
  if (int rc = check_norm_rope(B, L, H, D, dtype, cs_dtype, cos, sin)) return rc;
  const int64_t rows = (int64_t)B * L * H;
  cudaStream_t st = (cudaStream_t)stream;
  if (weight && d_weight) {
    const cudaError_t e = cudaMemsetAsync(d_weight, 0, sizeof(float) * (size_t)D, st);
    if (e != cudaSuccess) return cuda_fail(e, "norm_rope_bwd (memset)");
  }
  if (rows == 0) return HILS_OK;
  HILS_REQUIRE(d_out && d_x && (!weight || (x && rstd)), "norm_rope_bwd: null pointer");
  NormRopeParams p = {};
  p.x = x; p.weight = weight; p.cos = cos; p.sin = sin; p.rstd = const_cast<float*>(rstd);
  p.d_out = d_out; p.d_x = d_x; p.d_weight = d_weight;
  p.rows = rows; p.L = L; p.H = H; p.D = D; p.cos_batched = cos_batched; p.cs_f32 = cs_dtype == HILS_F32;
  if (dtype == HILS_BF16) norm_rope_bwd_kernel<bf16><<<norm_rope_grid(rows), 32 * kNrWarps, 0, st>>>(p);
  else norm_rope_bwd_kernel<float><<<norm_rope_grid(rows), 32 * kNrWarps, 0, st>>>(p);
  HILS_LAUNCH_CHECK("norm_rope_bwd");
  return HILS_OK;
}
