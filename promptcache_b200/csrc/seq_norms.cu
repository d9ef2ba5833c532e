// Sequence-batch support kernels: error state of the library, embedding, RMS norm, the gated output norm with layer scale
// and residual sum, xIELU.  The residual stream is 32-bit; statistics and gates are evaluated in 32-bit in both types.
#include <stdarg.h>
#include <stdio.h>

#include <atomic>

#include "seq_common.cuh"

namespace pcs {

static thread_local char g_err[512] = "";
static std::atomic<long long> g_launches{0};

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

template <typename T>
__global__ void __launch_bounds__(256) embed_kernel(const T* __restrict__ table, const int64_t* __restrict__ ids,
                                                    float* __restrict__ out, int width, int vocab, float scale) {
  const int t = blockIdx.x;
  long long id = ids[t];
  if (id < 0 || id >= vocab) id = 0;
  const T* row = table + id * width;
  float* o = out + static_cast<long long>(t) * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) o[i] = ldf(row + i) * scale;
}

template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_kernel(const float* __restrict__ x, const int32_t* __restrict__ rows,
                                                      const T* __restrict__ w, T* __restrict__ out, int width, float eps) {
  __shared__ float red[33];
  const int r = blockIdx.x;
  const float* xr = x + static_cast<long long>(rows ? rows[r] : r) * width;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) ss = fmaf(xr[i], xr[i], ss);
  ss = block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / static_cast<float>(width) + eps);
  T* o = out + static_cast<long long>(r) * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) stf(o + i, xr[i] * inv * ldf(w + i));
}

// One block per row.  u = y * sigmoid(g) is kept in shared memory between the statistics pass and the update.
template <typename T>
__global__ void __launch_bounds__(256) gate_norm_add_kernel(const pcs_gna_params p) {
  extern __shared__ float u[];  // [width]
  __shared__ float red[33];
  const int r = blockIdx.x, W = p.width;
  const T* y = static_cast<const T*>(p.y) + static_cast<long long>(r) * p.y_stride;
  const float* y32 = p.y_f32 ? static_cast<const float*>(p.y) + static_cast<long long>(r) * p.y_stride : nullptr;
  const T* g = p.g ? static_cast<const T*>(p.g) + static_cast<long long>(r) * p.g_stride : nullptr;
  const T* w = static_cast<const T*>(p.w);
  const T* ls = static_cast<const T*>(p.ls);
  float* x = p.x + static_cast<long long>(r) * W;
  float ss = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float v = y32 ? y32[i] : ldf(y + i);
    if (g) v *= sigmoidf_(ldf(g + i));
    u[i] = v;
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / static_cast<float>(W) + p.eps);
  float s2 = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float v = u[i] * inv * (p.w_offset + ldf(w + i));
    if (ls) v *= ldf(ls + i);
    const float xn = x[i] + v;
    x[i] = xn;
    u[i] = xn;
    s2 = fmaf(xn, xn, s2);
  }
  if (p.next_w == nullptr) return;
  s2 = block_sum(s2, red);
  const float inv2 = 1.f / sqrtf(s2 / static_cast<float>(W) + p.eps);
  const T* nw = static_cast<const T*>(p.next_w);
  T* h = static_cast<T*>(p.h_out) + static_cast<long long>(r) * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) stf(h + i, u[i] * inv2 * (p.w_offset + ldf(nw + i)));
}

// The same row operation for rows of at most 256 * PPT 16-byte pieces whose pointers and strides are 16-byte aligned: a
// thread keeps its pieces in registers, and EVERY operand (y, the gate, x, the three weight vectors) is requested before the
// first reduction, so that one memory round trip is exposed instead of three.
template <typename T, int PPT>
__global__ void __launch_bounds__(256) gate_norm_add_vec_kernel(const pcs_gna_params p) {
  constexpr int N = Vec<T>::n;
  __shared__ float red[33];
  const int r = blockIdx.x, W = p.width;
  const T* y = static_cast<const T*>(p.y) + static_cast<long long>(r) * p.y_stride;
  const T* g = p.g ? static_cast<const T*>(p.g) + static_cast<long long>(r) * p.g_stride : nullptr;
  const T* w = static_cast<const T*>(p.w);
  const T* ls = static_cast<const T*>(p.ls);
  const T* nw = static_cast<const T*>(p.next_w);
  float* x = p.x + static_cast<long long>(r) * W;
  float v[PPT][N], wv[PPT][N], lv[PPT][N], xv[PPT][N], nv[PPT][N];
#pragma unroll
  for (int u = 0; u < PPT; ++u) {
    const int i = (threadIdx.x + u * 256) * N;
    if (i < W) {
      if (p.y_f32) ldx(reinterpret_cast<const float*>(p.y) + static_cast<long long>(r) * p.y_stride + i, v[u]);
      else ld16(y + i, v[u]);
      ld16(w + i, wv[u]);
      ldx(x + i, xv[u]);
      if (ls) ld16(ls + i, lv[u]);
      if (nw) ld16(nw + i, nv[u]);
      if (g) {
        float gv[N];
        ld16(g + i, gv);
#pragma unroll
        for (int e = 0; e < N; ++e) v[u][e] *= sigmoidf_(gv[e]);
      }
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int u = 0; u < PPT; ++u)
    if ((threadIdx.x + u * 256) * N < W) {
#pragma unroll
      for (int e = 0; e < N; ++e) ss = fmaf(v[u][e], v[u][e], ss);
    }
  ss = block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / static_cast<float>(W) + p.eps);
  float s2 = 0.f;
#pragma unroll
  for (int u = 0; u < PPT; ++u) {
    const int i = (threadIdx.x + u * 256) * N;
    if (i < W) {
#pragma unroll
      for (int e = 0; e < N; ++e) {
        float t = v[u][e] * inv * (p.w_offset + wv[u][e]);
        if (ls) t *= lv[u][e];
        xv[u][e] += t;
        s2 = fmaf(xv[u][e], xv[u][e], s2);
      }
      stx(x + i, xv[u]);
    }
  }
  if (nw == nullptr) return;
  s2 = block_sum(s2, red);
  const float inv2 = 1.f / sqrtf(s2 / static_cast<float>(W) + p.eps);
  T* h = static_cast<T*>(p.h_out) + static_cast<long long>(r) * W;
#pragma unroll
  for (int u = 0; u < PPT; ++u) {
    const int i = (threadIdx.x + u * 256) * N;
    if (i < W) {
      float o[N];
#pragma unroll
      for (int e = 0; e < N; ++e) o[e] = xv[u][e] * inv2 * (p.w_offset + nv[u][e]);
      st16(h + i, o);
    }
  }
}

// 16-byte pieces: `width`, both strides and both pointers are multiples of a piece
template <typename T>
__global__ void __launch_bounds__(256) xielu_vec_kernel(const T* __restrict__ z, long long z_stride, T* __restrict__ out,
                                                        long long out_stride, const T* __restrict__ a, int width) {
  constexpr int N = Vec<T>::n;
  const int r = blockIdx.x;
  const float ap = softplusf_(ldf(a)), an = 0.5f + softplusf_(ldf(a + 1));
  const T* zr = z + r * z_stride;
  T* o = out + r * out_stride;
  for (int i = (blockIdx.y * blockDim.x + threadIdx.x) * N; i < width; i += gridDim.y * blockDim.x * N) {
    float v[N], f[N];
    ld16(zr + i, v);
#pragma unroll
    for (int e = 0; e < N; ++e) f[e] = v[e] > 0.f ? fmaf(ap * v[e], v[e], 0.5f * v[e]) : fmaf(an, expm1f(v[e]) - v[e], 0.5f * v[e]);
    st16(o + i, f);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) xielu_kernel(const T* __restrict__ z, long long z_stride, T* __restrict__ out,
                                                    long long out_stride, const T* __restrict__ a, int width) {
  const int r = blockIdx.x;
  const float ap = softplusf_(ldf(a)), an = 0.5f + softplusf_(ldf(a + 1));
  const T* zr = z + r * z_stride;
  T* o = out + r * out_stride;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < width; i += gridDim.y * blockDim.x) {
    const float v = ldf(zr + i);
    const float f = v > 0.f ? fmaf(ap * v, v, 0.5f * v) : fmaf(an, expm1f(v) - v, 0.5f * v);
    stf(o + i, f);
  }
}

// One block per row: the weighted sum of the terms' rows in shared memory, then the norm.
template <typename T>
__global__ void __launch_bounds__(256) depth_mix_kernel(const pcs_depthmix_params p) {
  extern __shared__ float u[];  // [width]
  __shared__ float red[33];
  const int r = blockIdx.x, W = p.width;
  const long long row = p.rows ? p.rows[r] : r;
  const float* src = p.xs + row * W;
  if (p.y) {  // the newest term's residual sum first: x += (offset + w) * rms(y)
    float* xl = const_cast<float*>(src) + static_cast<long long>(p.n_terms - 1) * p.term_stride;
    const T* y = static_cast<const T*>(p.y) + row * p.y_stride;
    const float* y32 = p.y_f32 ? static_cast<const float*>(p.y) + row * p.y_stride : nullptr;
    const T* yw = static_cast<const T*>(p.y_w);
    float sy = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      const float v = y32 ? y32[i] : ldf(y + i);
      u[i] = v;
      sy = fmaf(v, v, sy);
    }
    sy = block_sum(sy, red);
    const float inv_y = 1.f / sqrtf(sy / static_cast<float>(W) + p.eps);
    for (int i = threadIdx.x; i < W; i += blockDim.x) xl[i] += (p.w_offset + ldf(yw + i)) * u[i] * inv_y;
    __syncthreads();  // the sum below reads the row with another thread mapping
  }
  const bool vec = (W & 3) == 0 && (p.term_stride & 3) == 0 && (reinterpret_cast<uintptr_t>(p.xs) & 15) == 0;
  float ss = 0.f;
  if (vec) {
    for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int j = 0; j < p.n_terms; ++j) {
        const float c = p.coef[j];
        const float4 v = *reinterpret_cast<const float4*>(src + j * p.term_stride + i);
        a.x = fmaf(c, v.x, a.x); a.y = fmaf(c, v.y, a.y); a.z = fmaf(c, v.z, a.z); a.w = fmaf(c, v.w, a.w);
      }
      u[i] = a.x; u[i + 1] = a.y; u[i + 2] = a.z; u[i + 3] = a.w;
      ss = fmaf(a.x, a.x, fmaf(a.y, a.y, fmaf(a.z, a.z, fmaf(a.w, a.w, ss))));
    }
  } else {
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      float a = 0.f;
      for (int j = 0; j < p.n_terms; ++j) a = fmaf(p.coef[j], src[j * p.term_stride + i], a);
      u[i] = a;
      ss = fmaf(a, a, ss);
    }
  }
  __syncthreads();
  if (p.x_out) {
    float* xo = p.x_out + static_cast<long long>(r) * W;
    for (int i = threadIdx.x; i < W; i += blockDim.x) xo[i] = u[i];
  }
  if (p.next_w == nullptr) return;
  ss = block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / static_cast<float>(W) + p.eps);
  const T* nw = static_cast<const T*>(p.next_w);
  T* h = static_cast<T*>(p.h_out) + static_cast<long long>(r) * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) stf(h + i, u[i] * inv * (p.w_offset + ldf(nw + i)));
}

}  // namespace pcs

PCS_API int pcs_depth_mix(const pcs_depthmix_params* p, void* stream) {
  PCS_REQUIRE(p, "pcs_depth_mix: null params");
  if (p->n_rows == 0) return PCS_OK;
  PCS_REQUIRE(p->xs && p->coef && p->n_terms > 0 && p->n_rows > 0 && p->width > 0, "pcs_depth_mix: bad arguments");
  PCS_REQUIRE(p->x_out || p->next_w, "pcs_depth_mix: nothing to write");
  PCS_REQUIRE(p->next_w == nullptr || p->h_out != nullptr, "pcs_depth_mix: next_w needs h_out");
  PCS_REQUIRE(p->y == nullptr || p->y_w != nullptr, "pcs_depth_mix: the residual sum needs its norm weight");
  const size_t smem = static_cast<size_t>(p->width) * sizeof(float);
  PCS_REQUIRE(smem <= 200 * 1024, "pcs_depth_mix: width %d exceeds the shared-memory row", p->width);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (smem > 48 * 1024)
    PCS_DISPATCH(p->dtype, PCS_CHECK_CUDA(cudaFuncSetAttribute(pcs::depth_mix_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)));
  PCS_DISPATCH(p->dtype, pcs::depth_mix_kernel<T><<<p->n_rows, 256, smem, st>>>(*p));
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}

PCS_API int pcs_version(void) { return PCS_ABI_VERSION; }
PCS_API const char* pcs_last_error(void) { return pcs::g_err; }
PCS_API int64_t pcs_launch_count(void) { return pcs::g_launches.load(std::memory_order_relaxed); }

PCS_API int pcs_embed(const void* table, const int64_t* ids, float* out, int n_tokens, int width, int vocab, float scale,
                      int dtype, void* stream) {
  if (n_tokens == 0) return PCS_OK;
  PCS_REQUIRE(table && ids && out && n_tokens > 0 && width > 0 && vocab > 0, "pcs_embed: bad arguments");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  PCS_DISPATCH(dtype, pcs::embed_kernel<T><<<n_tokens, 256, 0, st>>>(static_cast<const T*>(table), ids, out, width, vocab, scale));
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}

PCS_API int pcs_rmsnorm(const float* x, const int32_t* rows, const void* w, void* out, int n_rows, int width, float eps,
                        int dtype, void* stream) {
  if (n_rows == 0) return PCS_OK;
  PCS_REQUIRE(x && w && out && n_rows > 0 && width > 0, "pcs_rmsnorm: bad arguments");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  PCS_DISPATCH(dtype, pcs::rmsnorm_kernel<T><<<n_rows, 256, 0, st>>>(x, rows, static_cast<const T*>(w), static_cast<T*>(out), width, eps));
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}

PCS_API int pcs_gate_norm_add(const pcs_gna_params* p, void* stream) {
  PCS_REQUIRE(p, "pcs_gate_norm_add: null params");
  if (p->n_rows == 0) return PCS_OK;
  PCS_REQUIRE(p->x && p->y && p->w && p->n_rows > 0 && p->width > 0, "pcs_gate_norm_add: bad arguments");
  PCS_REQUIRE(p->next_w == nullptr || p->h_out != nullptr, "pcs_gate_norm_add: next_w needs h_out");
  const size_t smem = static_cast<size_t>(p->width) * sizeof(float);
  PCS_REQUIRE(smem <= 200 * 1024, "pcs_gate_norm_add: width %d exceeds the shared-memory row", p->width);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (smem > 48 * 1024) {
    PCS_DISPATCH(p->dtype, PCS_CHECK_CUDA(cudaFuncSetAttribute(pcs::gate_norm_add_kernel<T>,
                                                              cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)));
  }
  // rows that fit the register kernel (at most 512 aligned 16-byte pieces) take it
  const int piece = p->dtype == PCS_BF16 ? 8 : 4;
  const long long esz = p->dtype == PCS_BF16 ? 2 : 4;
  auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  const bool vec = p->width % piece == 0 && p->width <= 512 * piece && (p->y_stride * (p->y_f32 ? 4 : esz)) % 16 == 0 && al(p->x) && al(p->y) && al(p->w) &&
                   (p->g == nullptr || (al(p->g) && (p->g_stride * esz) % 16 == 0)) && (p->ls == nullptr || al(p->ls)) &&
                   (p->next_w == nullptr || (al(p->next_w) && al(p->h_out)));
  if (vec) {
    if (p->width <= 256 * piece) PCS_DISPATCH(p->dtype, pcs::gate_norm_add_vec_kernel<T, 1><<<p->n_rows, 256, 0, st>>>(*p));
    else PCS_DISPATCH(p->dtype, pcs::gate_norm_add_vec_kernel<T, 2><<<p->n_rows, 256, 0, st>>>(*p));
    PCS_CHECK_CUDA(cudaGetLastError());
    pcs::count_launch();
    return PCS_OK;
  }
  PCS_DISPATCH(p->dtype, pcs::gate_norm_add_kernel<T><<<p->n_rows, 256, smem, st>>>(*p));
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}

PCS_API int pcs_xielu(const void* z, int64_t z_stride, void* out, int64_t out_stride, const void* a, int n_rows, int width,
                      int dtype, void* stream) {
  if (n_rows == 0) return PCS_OK;
  PCS_REQUIRE(z && out && a && n_rows > 0 && width > 0, "pcs_xielu: bad arguments");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int piece = dtype == PCS_BF16 ? 8 : 4;
  const long long esz = dtype == PCS_BF16 ? 2 : 4;
  if (width % piece == 0 && (z_stride * esz) % 16 == 0 && (out_stride * esz) % 16 == 0 && (reinterpret_cast<uintptr_t>(z) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
    const int per_row = (width / piece + 255) / 256;
    dim3 vgrid(n_rows, per_row > 64 ? 64 : per_row);
    PCS_DISPATCH(dtype, pcs::xielu_vec_kernel<T><<<vgrid, 256, 0, st>>>(static_cast<const T*>(z), z_stride, static_cast<T*>(out), out_stride,
                                                                        static_cast<const T*>(a), width));
    PCS_CHECK_CUDA(cudaGetLastError());
    pcs::count_launch();
    return PCS_OK;
  }
  dim3 grid(n_rows, (width + 255) / 256 > 64 ? 64 : (width + 255) / 256);
  PCS_DISPATCH(dtype, pcs::xielu_kernel<T><<<grid, 256, 0, st>>>(static_cast<const T*>(z), z_stride, static_cast<T*>(out), out_stride,
                                                                 static_cast<const T*>(a), width));
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}
