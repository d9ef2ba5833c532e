// Residual sum of several sublayer results and layer norms (weight, no bias) of the new stream.
//
// A layer whose sublayers run side by side reads ONE stream x through two norms and adds all results at once:
//     x += a0 y0 + a1 y1 + a2 y2;   h1 = ln(x) * w1;   h2 = ln(x) * w2,   ln(x) = (x - mean) / sqrt(var + eps),
// so the sum of layer i and both input norms of layer i + 1 are one launch and one pass over the row.  One block per row; the
// new row is kept in shared memory (or, for rows of at most 256 * PPT aligned 16-byte pieces, in registers with every operand
// requested before the first reduction).  Mean and variance are formed in two passes (the variance from the deviations), in
// 32-bit, with an order of additions that depends on the width alone.  With `rows` the kernel norms a subset of the rows
// (the final norm on the rows whose logits are wanted) and adds nothing.
#include "seq_common.cuh"

namespace pcs {

template <typename T>
__device__ __forceinline__ float addend(const pcs_addln_params& p, int j, long long r, int i) {
  if (p.y_f32[j]) return static_cast<const float*>(p.y[j])[r * p.y_stride[j] + i];
  return ldf(static_cast<const T*>(p.y[j]) + r * p.y_stride[j] + i);
}

template <typename T>
__global__ void __launch_bounds__(256) add_layer_norm_kernel(const pcs_addln_params p) {
  extern __shared__ float u[];  // [width]
  __shared__ float red[33];
  const int r = blockIdx.x, W = p.width;
  const long long row = p.rows ? p.rows[r] : r;
  float* x = p.x + row * W;
  float s = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float v = x[i];
    if (p.n_addends > 0) {
      float a = 0.f;   // the sublayers' results are summed first, then added to the stream
      for (int j = 0; j < p.n_addends; ++j) a = fmaf(p.y_mult[j], addend<T>(p, j, row, i), a);
      v += a;
      x[i] = v;
    }
    u[i] = v;
    s += v;
  }
  if (p.w1 == nullptr && p.w2 == nullptr) return;
  const float mu = block_sum(s, red) / static_cast<float>(W);
  float q = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) { const float d = u[i] - mu; q = fmaf(d, d, q); }
  const float inv = 1.f / sqrtf(block_sum(q, red) / static_cast<float>(W) + p.eps);
  const T* w1 = static_cast<const T*>(p.w1);
  const T* w2 = static_cast<const T*>(p.w2);
  T* h1 = static_cast<T*>(p.h1) + static_cast<long long>(r) * W;
  T* h2 = static_cast<T*>(p.h2) + static_cast<long long>(r) * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float d = (u[i] - mu) * inv;
    if (w1) stf(h1 + i, d * ldf(w1 + i));
    if (w2) stf(h2 + i, d * ldf(w2 + i));
  }
}

// Rows of at most 256 * PPT pieces, everything 16-byte aligned: the row lives in registers.
template <typename T, int PPT>
__global__ void __launch_bounds__(256) add_layer_norm_vec_kernel(const pcs_addln_params p) {
  constexpr int N = Vec<T>::n;
  __shared__ float red[33];
  const int r = blockIdx.x, W = p.width;
  const long long row = p.rows ? p.rows[r] : r;
  float* x = p.x + row * W;
  const T* w1 = static_cast<const T*>(p.w1);
  const T* w2 = static_cast<const T*>(p.w2);
  float xv[PPT][N], yv[3][PPT][N], w1v[PPT][N], w2v[PPT][N];
#pragma unroll
  for (int k = 0; k < PPT; ++k) {
    const int i = (threadIdx.x + k * 256) * N;
    if (i < W) {
      ldx(x + i, xv[k]);
#pragma unroll
      for (int j = 0; j < 3; ++j)
        if (j < p.n_addends) {
          if (p.y_f32[j]) ldx(static_cast<const float*>(p.y[j]) + row * p.y_stride[j] + i, yv[j][k]);
          else ld16(static_cast<const T*>(p.y[j]) + row * p.y_stride[j] + i, yv[j][k]);
        }
      if (w1) ld16(w1 + i, w1v[k]);
      if (w2) ld16(w2 + i, w2v[k]);
    }
  }
  float s = 0.f;
#pragma unroll
  for (int k = 0; k < PPT; ++k) {
    const int i = (threadIdx.x + k * 256) * N;
    if (i < W) {
      if (p.n_addends > 0) {
#pragma unroll
        for (int e = 0; e < N; ++e) {
          float a = 0.f;
#pragma unroll
          for (int j = 0; j < 3; ++j)
            if (j < p.n_addends) a = fmaf(p.y_mult[j], yv[j][k][e], a);
          xv[k][e] += a;
        }
        stx(x + i, xv[k]);
      }
#pragma unroll
      for (int e = 0; e < N; ++e) s += xv[k][e];
    }
  }
  if (w1 == nullptr && w2 == nullptr) return;
  const float mu = block_sum(s, red) / static_cast<float>(W);
  float q = 0.f;
#pragma unroll
  for (int k = 0; k < PPT; ++k) {
    const int i = (threadIdx.x + k * 256) * N;
    if (i < W) {
#pragma unroll
      for (int e = 0; e < N; ++e) { xv[k][e] -= mu; q = fmaf(xv[k][e], xv[k][e], q); }
    }
  }
  const float inv = 1.f / sqrtf(block_sum(q, red) / static_cast<float>(W) + p.eps);
  T* h1 = static_cast<T*>(p.h1) + static_cast<long long>(r) * W;
  T* h2 = static_cast<T*>(p.h2) + static_cast<long long>(r) * W;
#pragma unroll
  for (int k = 0; k < PPT; ++k) {
    const int i = (threadIdx.x + k * 256) * N;
    if (i < W) {
      float o[N];
      if (w1) {
#pragma unroll
        for (int e = 0; e < N; ++e) o[e] = xv[k][e] * inv * w1v[k][e];
        st16(h1 + i, o);
      }
      if (w2) {
#pragma unroll
        for (int e = 0; e < N; ++e) o[e] = xv[k][e] * inv * w2v[k][e];
        st16(h2 + i, o);
      }
    }
  }
}

}  // namespace pcs

PCS_API int pcs_add_layer_norm(const pcs_addln_params* p, void* stream) {
  PCS_REQUIRE(p, "pcs_add_layer_norm: null params");
  if (p->n_rows == 0) return PCS_OK;
  PCS_REQUIRE(p->x && p->n_rows > 0 && p->width > 0 && p->n_addends >= 0 && p->n_addends <= 3, "pcs_add_layer_norm: bad arguments");
  PCS_REQUIRE(p->rows == nullptr || p->n_addends == 0, "pcs_add_layer_norm: a row subset takes no addends");
  PCS_REQUIRE((p->w1 == nullptr || p->h1 != nullptr) && (p->w2 == nullptr || p->h2 != nullptr), "pcs_add_layer_norm: a weight vector needs its output");
  PCS_REQUIRE(p->w1 || p->w2 || p->n_addends > 0, "pcs_add_layer_norm: nothing to do");
  for (int j = 0; j < p->n_addends; ++j) PCS_REQUIRE(p->y[j] != nullptr, "pcs_add_layer_norm: addend %d is null", j);
  const size_t smem = static_cast<size_t>(p->width) * sizeof(float);
  PCS_REQUIRE(smem <= 200 * 1024, "pcs_add_layer_norm: width %d exceeds the shared-memory row", p->width);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int piece = p->dtype == PCS_BF16 ? 8 : 4;
  const long long esz = p->dtype == PCS_BF16 ? 2 : 4;
  auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  bool vec = p->width % piece == 0 && p->width <= 512 * piece && al(p->x) && al(p->w1) && al(p->w2) && al(p->h1) && al(p->h2);
  for (int j = 0; j < p->n_addends; ++j) vec = vec && al(p->y[j]) && (p->y_stride[j] * (p->y_f32[j] ? 4 : esz)) % 16 == 0;
  if (vec) {
    if (p->width <= 256 * piece) PCS_DISPATCH(p->dtype, (pcs::add_layer_norm_vec_kernel<T, 1><<<p->n_rows, 256, 0, st>>>(*p)));
    else PCS_DISPATCH(p->dtype, (pcs::add_layer_norm_vec_kernel<T, 2><<<p->n_rows, 256, 0, st>>>(*p)));
  } else {
    if (smem > 48 * 1024)
      PCS_DISPATCH(p->dtype, PCS_CHECK_CUDA(cudaFuncSetAttribute(pcs::add_layer_norm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)));
    PCS_DISPATCH(p->dtype, pcs::add_layer_norm_kernel<T><<<p->n_rows, 256, smem, st>>>(*p));
  }
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}
