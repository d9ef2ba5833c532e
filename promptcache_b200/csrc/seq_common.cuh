// Shared helpers of the sequence-batch kernels (libpromptcache_b200_seq.so): error plumbing, typed loads / stores for the
// two compute types, block reductions.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "../../include/promptcache_b200_seq.h"

#define PCS_API extern "C" __attribute__((visibility("default")))

namespace pcs {

int set_error(int code, const char* fmt, ...);
void count_launch(int n = 1);

#define PCS_CHECK_CUDA(expr)                                                                        \
  do {                                                                                              \
    cudaError_t _e = (expr);                                                                        \
    if (_e != cudaSuccess)                                                                          \
      return pcs::set_error(PCS_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
  } while (0)

#define PCS_REQUIRE(cond, ...)                                         \
  do {                                                                 \
    if (!(cond)) return pcs::set_error(PCS_ERR_INVALID, __VA_ARGS__);  \
  } while (0)

// dispatch a templated launch on the run-time type code
#define PCS_DISPATCH(dtype, ...)                                                    \
  do {                                                                              \
    if ((dtype) == PCS_BF16) { using T = __nv_bfloat16; __VA_ARGS__; }              \
    else if ((dtype) == PCS_F32) { using T = float; __VA_ARGS__; }                  \
    else return pcs::set_error(PCS_ERR_INVALID, "unknown dtype code %d", (dtype));  \
  } while (0)

__device__ __forceinline__ float ldf(const float* p) { return *p; }
__device__ __forceinline__ float ldf(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// kVec<T>: elements of one 16-byte load
template <typename T> struct Vec;
template <> struct Vec<float> { static constexpr int n = 4; };
template <> struct Vec<__nv_bfloat16> { static constexpr int n = 8; };

__device__ __forceinline__ void ld16(const float* p, float (&o)[4]) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
}
__device__ __forceinline__ void ld16(const __nv_bfloat16* p, float (&o)[8]) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    o[2 * i] = f.x;
    o[2 * i + 1] = f.y;
  }
}

// 32-bit rows in pieces of the compute type's 16-byte element count, and 16-byte stores of converted values
__device__ __forceinline__ void ldx(const float* p, float (&o)[4]) { ld16(p, o); }
__device__ __forceinline__ void ldx(const float* p, float (&o)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
__device__ __forceinline__ void stx(float* p, const float (&v)[4]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
__device__ __forceinline__ void stx(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void st16(float* p, const float (&v)[4]) { stx(p, v); }
__device__ __forceinline__ void st16(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}

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
// Sum over the block (blockDim.x a multiple of 32, at most 1024); `red` holds 33 floats.  Every thread gets the result,
// and the order of the additions is fixed by the block size alone.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  v = warp_sum(v);
  __syncthreads();  // `red` may still be read from a previous call
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? red[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

__device__ __forceinline__ float sigmoidf_(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float softplusf_(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float logsigmoidf_(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

// sine and cosine of pos * f: the angle is formed and reduced modulo 2 pi in 64-bit, then evaluated in 32-bit on [-pi, pi]
__device__ __forceinline__ void angle_sincos(int pos, double f, float* s, float* c) {
  const double a = static_cast<double>(pos) * f;
  const double r = a - 6.283185307179586476925 * rint(a * 0.15915494309189533577);
  sincosf(static_cast<float>(r), s, c);
}

// The gated activation of a feed-forward, by value (a kernel argument): PCS_GLU_SILU: silu(g) * u;
// PCS_GLU_CLAMPED_SWISH: g' = min(g, limit), u' = clamp(u, -limit, limit), g' * sigmoid(alpha * g') * (u' + 1).
// PCS_ACT_RELU2 and PCS_ACT_GELU_ERF have no gate branch (`gated()` is false): the first argument alone is used.
struct GluAct {
  int kind;
  float alpha, limit;
  __host__ GluAct() : kind(PCS_GLU_SILU), alpha(1.f), limit(0.f) {}
  __host__ explicit GluAct(const pcs_glu_act* a) : kind(a ? a->kind : PCS_GLU_SILU), alpha(a ? a->alpha : 1.f), limit(a ? a->limit : 0.f) {}
  __host__ __device__ __forceinline__ bool gated() const { return kind == PCS_GLU_SILU || kind == PCS_GLU_CLAMPED_SWISH; }
  __device__ __forceinline__ float operator()(float g, float u) const {
    if (kind == PCS_ACT_RELU2) {
      const float r = fmaxf(g, 0.f);
      return r * r;
    }
    if (kind == PCS_ACT_GELU_ERF) return 0.5f * g * (1.f + erff(g * 0.70710678118654752440f));
    if (kind == PCS_GLU_CLAMPED_SWISH) {
      g = fminf(g, limit);
      u = fminf(fmaxf(u, -limit), limit);
      return g * sigmoidf_(alpha * g) * (u + 1.f);
    }
    return g * sigmoidf_(g) * u;
  }
};

}  // namespace pcs
