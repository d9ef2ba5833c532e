// Mixture of experts: the router, the chosen experts for a handful of rows, and the weighted sum into the residual stream.
//
// pcs_moe_route      one block per token.  Warps share the router's outputs (a 32-bit dot product each, lanes over K), then
//                    warp 0 alone does the rest in shared memory: softmax over all outputs (or a sigmoid of each), choice scores
//                    (score + correction), the groups' scores (their best choice score, or the sum of their few best), the best
//                    groups, and `top` rounds of an arg-max whose ties go to the lower index.  The weights handed on are the plain
//                    scores, optionally over the sum of the chosen ones and times a constant.  A second dot product gives the
//                    shared expert's gate.  Every sum has an order that depends on the sizes alone.
// pcs_moe_rows_up    block = (pair, 8 features): a warp owns two features, its lanes share K in 16-byte pieces with the gate
// pcs_moe_rows_down  and up rows of both features in flight; the expert's weights are read once per pair.  Any number of
//                    pairs may be given (the 32-bit path of prompts uses it too); the products of prompts in bfloat16 go
//                    through the grouped tensor-core kernel (seq_moe_gemm.cu).
// pcs_moe_combine    one block per token: x += mult * (sum_k w_k * (expert result | the input itself) + gate * shared result),
//                    in the order of the choices.
#include "seq_common.cuh"

namespace pcs {

constexpr int kMaxRouterOutputs = 1024;

// arg-max over c[0 .. n) by one warp; ties: the lower index.  Every lane returns the result.
__device__ __forceinline__ int warp_argmax(const float* c, int n, int lane, float* best_out) {
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int e = lane; e < n; e += 32) {
    const float v = c[e];
    if (v > bv || (bi == 0x7fffffff && v == bv)) { bv = v; bi = e; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  *best_out = bv;
  return bi;
}

// lanes share K in 16-byte pieces; four independent partial sums per lane (pieces lane, lane + 32, ... go round them), so
// that four loads of each operand are in flight and no sum waits for the one before.  The order depends on K alone.
template <typename T>
__device__ __forceinline__ float warp_dot(const T* __restrict__ a, const T* __restrict__ b, int K, int lane, bool vec) {
  constexpr int N = Vec<T>::n;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  if (vec) {
    int k = lane * N;
    for (; k + 96 * N < K; k += 128 * N) {
      float a0[N], a1[N], a2[N], a3[N], b0[N], b1[N], b2[N], b3[N];
      ld16(a + k, a0); ld16(a + k + 32 * N, a1); ld16(a + k + 64 * N, a2); ld16(a + k + 96 * N, a3);
      ld16(b + k, b0); ld16(b + k + 32 * N, b1); ld16(b + k + 64 * N, b2); ld16(b + k + 96 * N, b3);
#pragma unroll
      for (int e = 0; e < N; ++e) {
        s0 = fmaf(a0[e], b0[e], s0);
        s1 = fmaf(a1[e], b1[e], s1);
        s2 = fmaf(a2[e], b2[e], s2);
        s3 = fmaf(a3[e], b3[e], s3);
      }
    }
    for (; k < K; k += 32 * N) {
      float av[N], bv[N];
      ld16(a + k, av);
      ld16(b + k, bv);
#pragma unroll
      for (int e = 0; e < N; ++e) s0 = fmaf(av[e], bv[e], s0);
    }
  } else {
    for (int k = lane; k < K; k += 32) s0 = fmaf(ldf(a + k), ldf(b + k), s0);
  }
  return warp_sum((s0 + s1) + (s2 + s3));
}

__host__ __device__ __forceinline__ bool aligned16(const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; }

// One warp, one token: z holds the router's logits on entry.  Softmax, choice scores, group limits and `top` arg-max rounds.
__device__ __forceinline__ void route_select(const pcs_route_params& p, int t, int lane, float* z, float* c, float* gs) {
  const int E = p.n_outputs;
  float m = -INFINITY;
  if (p.bias) {
    for (int e = lane; e < E; e += 32) z[e] += p.bias[e];
  }
  if (p.score_fn == 1) {  // every output's own sigmoid
    for (int e = lane; e < E; e += 32) {
      const float s = sigmoidf_(z[e]);
      z[e] = s;
      c[e] = s + (p.correction ? p.correction[e] : 0.f);
    }
  } else {
    for (int e = lane; e < E; e += 32) m = fmaxf(m, z[e]);
    m = warp_max(m);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) { const float w = expf(z[e] - m); z[e] = w; sum += w; }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
    for (int e = lane; e < E; e += 32) {
      const float s = z[e] * inv;
      z[e] = s;
      c[e] = s + (p.correction ? p.correction[e] : 0.f);
    }
  }
  __syncwarp();
  const int G = p.n_groups, per = E / G;
  if (G > 1 && p.keep_groups < G) {
    const int nb = min(max(p.group_best, 1), per);
    for (int g = lane; g < G; g += 32) {
      float b = -INFINITY;
      if (nb == 1) {
        for (int e = g * per; e < (g + 1) * per; ++e) b = fmaxf(b, c[e]);
      } else {  // the sum of the group's nb largest choice scores: nb rounds over the group, each below the last one taken
        float sum_b = 0.f, last = INFINITY;
        int last_e = -1;
        for (int r = 0; r < nb; ++r) {
          float bv = -INFINITY;
          int be = -1;
          for (int e = g * per; e < (g + 1) * per; ++e) {
            const float v = c[e];
            const bool free_e = v < last || (v == last && e > last_e);   // not taken by an earlier round (ties go by index)
            if (free_e && (v > bv || be < 0)) { bv = v; be = e; }
          }
          sum_b += bv;
          last = bv;
          last_e = be;
        }
        b = sum_b;
      }
      gs[g] = b;
      gs[G + g] = 0.f;
    }
    __syncwarp();
    // the best groups: a taken group leaves the next rounds (its score becomes minus infinity) and is marked in gs[G + g]
    for (int r = 0; r < p.keep_groups; ++r) {
      float bv;
      const int g = warp_argmax(gs, G, lane, &bv);
      __syncwarp();
      if (lane == 0) { gs[g] = -INFINITY; gs[G + g] = 1.f; }
      __syncwarp();
    }
  }
  const bool limited = G > 1 && p.keep_groups < G;
  if (limited) {
    for (int e = lane; e < E; e += 32)
      if (gs[G + e / per] != 1.f) c[e] = -INFINITY;
    __syncwarp();
  }
  for (int k = 0; k < p.top; ++k) {
    float bv;
    const int e = warp_argmax(c, E, lane, &bv);
    __syncwarp();
    if (lane == 0) {
      p.idx[static_cast<long long>(t) * p.top + k] = e;
      p.wgt[static_cast<long long>(t) * p.top + k] = z[e];
      c[e] = -INFINITY;
    }
    __syncwarp();
  }
  if (p.renorm && lane == 0) {  // the softmax over the chosen outputs alone: their scores divided by their sum, in the order of the choices
    float* w = p.wgt + static_cast<long long>(t) * p.top;
    float sum_k = 0.f;
    for (int k = 0; k < p.top; ++k) sum_k += w[k];
    const float inv_k = 1.f / (sum_k + p.renorm_eps);
    for (int k = 0; k < p.top; ++k) w[k] *= inv_k;
  }
  if (p.wgt_scale != 0.f && p.wgt_scale != 1.f && lane == 0) {
    float* w = p.wgt + static_cast<long long>(t) * p.top;
    for (int k = 0; k < p.top; ++k) w[k] *= p.wgt_scale;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) moe_route_kernel(const pcs_route_params p) {
  __shared__ float z[kMaxRouterOutputs];   // logits, then scores
  __shared__ float c[kMaxRouterOutputs];   // choice scores (minus infinity once taken or not allowed)
  __shared__ float gs[kMaxRouterOutputs];  // the groups' scores
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, E = p.n_outputs, K = p.width;
  const T* h = static_cast<const T*>(p.h) + static_cast<long long>(t) * p.h_stride;
  const T* wr = static_cast<const T*>(p.w_router);
  const bool vec = K % Vec<T>::n == 0 && aligned16(h) && aligned16(wr) && (p.h_stride * sizeof(T)) % 16 == 0;
  for (int e = warp; e < E; e += 8) {
    const float d = warp_dot(h, wr + static_cast<long long>(e) * K, K, lane, vec);
    if (lane == 0) z[e] = d;
  }
  if (p.w_sg && warp == 7) {
    const T* ws = static_cast<const T*>(p.w_sg);
    const float d = warp_dot(h, ws, K, lane, vec && aligned16(ws));
    if (lane == 0) p.shared_gate[t] = sigmoidf_(d);
  }
  __syncthreads();
  if (warp != 0) return;
  route_select(p, t, lane, z, c, gs);
}

// The same with one WARP per token (many tokens): the eight warps of a block walk the router's rows together, so a row comes
// from L2 once per eight tokens; each warp then selects for its own token.  Results equal the block-per-token kernel's.
constexpr int kWarpRouteOutputs = 256;
template <typename T>
__global__ void __launch_bounds__(256) moe_route_warp_kernel(const pcs_route_params p) {
  __shared__ float buf[8][4 * kWarpRouteOutputs];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, E = p.n_outputs, K = p.width;
  const int t = blockIdx.x * 8 + warp;
  if (t >= p.n_tokens) return;
  float* z = buf[warp];
  float* c = z + kWarpRouteOutputs;
  float* gs = c + kWarpRouteOutputs;
  const T* h = static_cast<const T*>(p.h) + static_cast<long long>(t) * p.h_stride;
  const T* wr = static_cast<const T*>(p.w_router);
  const bool vec = K % Vec<T>::n == 0 && aligned16(h) && aligned16(wr) && (p.h_stride * sizeof(T)) % 16 == 0;
  for (int e = 0; e < E; ++e) {
    const float d = warp_dot(h, wr + static_cast<long long>(e) * K, K, lane, vec);
    if (lane == 0) z[e] = d;
  }
  if (p.w_sg) {
    const T* ws = static_cast<const T*>(p.w_sg);
    const float d = warp_dot(h, ws, K, lane, vec && aligned16(ws));
    if (lane == 0) p.shared_gate[t] = sigmoidf_(d);
  }
  __syncwarp();
  route_select(p, t, lane, z, c, gs);
}

// block = (pair, 8 features); warp w owns features n0 + 2w, n0 + 2w + 1
template <typename T>
__global__ void __launch_bounds__(128) moe_rows_up_kernel(const T* __restrict__ h, long long h_stride, const T* __restrict__ w_gu,
                                                          const int32_t* __restrict__ idx, T* __restrict__ act, int top, int n_experts,
                                                          int ff, int K, bool vec, const GluAct glu) {
  const int pr = blockIdx.x, e = idx[pr];
  if (e >= n_experts || e < 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* x = h + static_cast<long long>(pr / top) * h_stride;
  const bool gated = glu.gated();   // without a gate branch an expert has ff rows, not 2 ff
  const T* wg = w_gu + static_cast<long long>(e) * (gated ? 2 : 1) * ff * K;
  const T* wu = wg + static_cast<long long>(ff) * K;
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int n = blockIdx.y * 8 + warp * 2 + u;
    if (n >= ff) return;
    const float g = warp_dot(x, wg + static_cast<long long>(n) * K, K, lane, vec);
    const float v = gated ? warp_dot(x, wu + static_cast<long long>(n) * K, K, lane, vec) : 0.f;
    if (lane == 0) stf(act + static_cast<long long>(pr) * ff + n, glu(g, v));
  }
}

template <typename T>
__global__ void __launch_bounds__(128) moe_rows_down_kernel(const T* __restrict__ act, const T* __restrict__ w_down, const int32_t* __restrict__ idx,
                                                            float* __restrict__ y, int n_experts, int ff, int W, bool vec) {
  const int pr = blockIdx.x, e = idx[pr];
  if (e >= n_experts || e < 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* a = act + static_cast<long long>(pr) * ff;
  const T* wd = w_down + static_cast<long long>(e) * W * ff;
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int n = blockIdx.y * 8 + warp * 2 + u;
    if (n >= W) return;
    const float d = warp_dot(a, wd + static_cast<long long>(n) * ff, ff, lane, vec);
    if (lane == 0) y[static_cast<long long>(pr) * W + n] = d;
  }
}

constexpr int kCombineMaxTop = 64;

// One block per token.  The token's choices (weight, row of y or "the input itself") are read once into shared memory; the
// channels then go in 16-byte pieces where the pointers allow.
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) moe_combine_kernel(const pcs_combine_params p) {
  constexpr int N = Vec<T>::n;
  __shared__ float w_s[kCombineMaxTop];
  __shared__ long long row_s[kCombineMaxTop];   // -1: a pass-through choice
  const int t = blockIdx.x, W = p.width;
  if (threadIdx.x < p.top) {
    const long long pr = static_cast<long long>(t) * p.top + threadIdx.x;
    w_s[threadIdx.x] = p.wgt[pr];
    row_s[threadIdx.x] = p.idx[pr] < p.n_experts ? (p.y_row ? static_cast<long long>(p.y_row[pr]) : pr) : -1;
  }
  __syncthreads();
  float* x = p.x + static_cast<long long>(t) * W;
  const T* h = static_cast<const T*>(p.h) + static_cast<long long>(t) * p.h_stride;
  const T* ys = p.ys ? static_cast<const T*>(p.ys) + static_cast<long long>(t) * p.ys_stride : nullptr;
  const float sg = (ys && p.shared_gate) ? p.shared_gate[t] : 1.f;
  const bool y32 = p.y_dtype == PCS_F32;
  if (VEC) {
    for (int i = threadIdx.x * N; i < W; i += 256 * N) {
      float a[N], v[N], xv[N];
#pragma unroll
      for (int e = 0; e < N; ++e) a[e] = 0.f;
      for (int k = 0; k < p.top; ++k) {
        const long long row = row_s[k];
        if (row < 0) ld16(h + i, v);
        else if (y32) ldx(static_cast<const float*>(p.y) + row * W + i, v);
        else ld16(static_cast<const T*>(p.y) + row * W + i, v);
        const float w = w_s[k];
#pragma unroll
        for (int e = 0; e < N; ++e) a[e] = fmaf(w, v[e], a[e]);
      }
      if (ys) {
        ld16(ys + i, v);
#pragma unroll
        for (int e = 0; e < N; ++e) a[e] = fmaf(sg, v[e], a[e]);
      }
      if (p.overwrite) {
#pragma unroll
        for (int e = 0; e < N; ++e) xv[e] = p.mult * a[e];
      } else {
        ldx(x + i, xv);
#pragma unroll
        for (int e = 0; e < N; ++e) xv[e] = fmaf(p.mult, a[e], xv[e]);
      }
      stx(x + i, xv);
    }
  } else {
    for (int i = threadIdx.x; i < W; i += 256) {
      float a = 0.f;
      for (int k = 0; k < p.top; ++k) {
        const long long row = row_s[k];
        const float v = row < 0 ? ldf(h + i) : (y32 ? static_cast<const float*>(p.y)[row * W + i] : ldf(static_cast<const T*>(p.y) + row * W + i));
        a = fmaf(w_s[k], v, a);
      }
      if (ys) a = fmaf(sg, ldf(ys + i), a);
      x[i] = p.overwrite ? p.mult * a : fmaf(p.mult, a, x[i]);
    }
  }
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(256) silu_mul_kernel(const T* __restrict__ gu, long long gu_stride, T* __restrict__ out, int ff, const GluAct glu) {
  constexpr int N = Vec<T>::n;
  const int r = blockIdx.x;
  const T* g = gu + r * gu_stride;
  T* o = out + static_cast<long long>(r) * ff;
  const bool gated = glu.gated();
  if (VEC) {
    for (int i = (blockIdx.y * 256 + threadIdx.x) * N; i < ff; i += gridDim.y * 256 * N) {
      float a[N], u[N];
      ld16(g + i, a);
      if (gated) ld16(g + ff + i, u);
#pragma unroll
      for (int e = 0; e < N; ++e) a[e] = glu(a[e], gated ? u[e] : 0.f);
      st16(o + i, a);
    }
  } else {
    for (int i = blockIdx.y * 256 + threadIdx.x; i < ff; i += gridDim.y * 256) {
      const float a = ldf(g + i);
      stf(o + i, glu(a, gated ? ldf(g + ff + i) : 0.f));
    }
  }
}

}  // namespace pcs

PCS_API int pcs_moe_route(const pcs_route_params* p, void* stream) {
  PCS_REQUIRE(p, "pcs_moe_route: null params");
  if (p->n_tokens == 0) return PCS_OK;
  PCS_REQUIRE(p->h && p->w_router && p->idx && p->wgt && p->width > 0, "pcs_moe_route: null tensor");
  PCS_REQUIRE(p->n_outputs > 0 && p->n_outputs <= pcs::kMaxRouterOutputs / 2, "pcs_moe_route: %d router outputs (at most %d)", p->n_outputs,
              pcs::kMaxRouterOutputs / 2);
  PCS_REQUIRE(p->top > 0 && p->n_groups > 0 && p->n_outputs % p->n_groups == 0 && p->keep_groups > 0 && p->keep_groups <= p->n_groups,
              "pcs_moe_route: bad top / groups (%d outputs, %d groups, %d kept)", p->n_outputs, p->n_groups, p->keep_groups);
  PCS_REQUIRE(p->top <= p->keep_groups * (p->n_outputs / p->n_groups), "pcs_moe_route: top %d exceeds the outputs of the kept groups", p->top);
  PCS_REQUIRE(p->w_sg == nullptr || p->shared_gate != nullptr, "pcs_moe_route: the shared gate needs its output");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (p->n_tokens >= 64 && p->n_outputs <= pcs::kWarpRouteOutputs)
    PCS_DISPATCH(p->dtype, pcs::moe_route_warp_kernel<T><<<(p->n_tokens + 7) / 8, 256, 0, st>>>(*p));
  else
    PCS_DISPATCH(p->dtype, pcs::moe_route_kernel<T><<<p->n_tokens, 256, 0, st>>>(*p));
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}

PCS_API int pcs_moe_rows_up(const void* h, int64_t h_stride, const void* w_gu, const int32_t* idx, void* act, int n_pairs, int top, int n_experts,
                            int ff, int width, const pcs_glu_act* glu, int dtype, void* stream) {
  if (n_pairs == 0 || n_experts == 0) return PCS_OK;
  PCS_REQUIRE(h && w_gu && idx && act && n_pairs > 0 && top > 0 && ff > 0 && width > 0, "pcs_moe_rows_up: bad arguments");
  const long long esz = dtype == PCS_BF16 ? 2 : 4;
  const bool vec = (width * esz) % 16 == 0 && (h_stride * esz) % 16 == 0 && pcs::aligned16(h) && pcs::aligned16(w_gu);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 grid(n_pairs, (ff + 7) / 8);
  PCS_DISPATCH(dtype, pcs::moe_rows_up_kernel<T><<<grid, 128, 0, st>>>(static_cast<const T*>(h), h_stride, static_cast<const T*>(w_gu), idx,
                                                                       static_cast<T*>(act), top, n_experts, ff, width, vec, pcs::GluAct(glu)));
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}

PCS_API int pcs_moe_rows_down(const void* act, const void* w_down, const int32_t* idx, float* y, int n_pairs, int n_experts, int ff, int width,
                              int dtype, void* stream) {
  if (n_pairs == 0 || n_experts == 0) return PCS_OK;
  PCS_REQUIRE(act && w_down && idx && y && n_pairs > 0 && ff > 0 && width > 0, "pcs_moe_rows_down: bad arguments");
  const long long esz = dtype == PCS_BF16 ? 2 : 4;
  const bool vec = (ff * esz) % 16 == 0 && pcs::aligned16(act) && pcs::aligned16(w_down);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 grid(n_pairs, (width + 7) / 8);
  PCS_DISPATCH(dtype, pcs::moe_rows_down_kernel<T><<<grid, 128, 0, st>>>(static_cast<const T*>(act), static_cast<const T*>(w_down), idx, y, n_experts,
                                                                         ff, width, vec));
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}

PCS_API int pcs_moe_combine(const pcs_combine_params* p, void* stream) {
  PCS_REQUIRE(p, "pcs_moe_combine: null params");
  if (p->n_tokens == 0) return PCS_OK;
  PCS_REQUIRE(p->x && p->idx && p->wgt && p->h && p->n_tokens > 0 && p->width > 0 && p->top > 0, "pcs_moe_combine: bad arguments");
  PCS_REQUIRE(p->y || p->n_experts == 0, "pcs_moe_combine: expert results missing");
  PCS_REQUIRE(p->top <= pcs::kCombineMaxTop, "pcs_moe_combine: top %d exceeds %d", p->top, pcs::kCombineMaxTop);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int piece = p->dtype == PCS_BF16 ? 8 : 4;
  const long long esz = p->dtype == PCS_BF16 ? 2 : 4;
  const bool vec = p->width % piece == 0 && pcs::aligned16(p->x) && pcs::aligned16(p->y) && pcs::aligned16(p->h) && (p->h_stride * esz) % 16 == 0 &&
                   (p->ys == nullptr || (pcs::aligned16(p->ys) && (p->ys_stride * esz) % 16 == 0));
  if (vec) PCS_DISPATCH(p->dtype, (pcs::moe_combine_kernel<T, true><<<p->n_tokens, 256, 0, st>>>(*p)));
  else PCS_DISPATCH(p->dtype, (pcs::moe_combine_kernel<T, false><<<p->n_tokens, 256, 0, st>>>(*p)));
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}

PCS_API int pcs_silu_mul(const void* gu, int64_t gu_stride, void* out, int n_rows, int ff, int dtype, void* stream) {
  return pcs_glu_mul(gu, gu_stride, out, n_rows, ff, nullptr, dtype, stream);
}

PCS_API int pcs_glu_mul(const void* gu, int64_t gu_stride, void* out, int n_rows, int ff, const pcs_glu_act* glu, int dtype, void* stream) {
  if (n_rows == 0 || ff == 0) return PCS_OK;
  PCS_REQUIRE(gu && out && n_rows > 0 && ff > 0, "pcs_glu_mul: bad arguments");
  PCS_REQUIRE(glu == nullptr || (glu->kind >= PCS_GLU_SILU && glu->kind <= PCS_ACT_GELU_ERF), "pcs_glu_mul: unknown activation %d", glu->kind);
  const pcs::GluAct act(glu);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int piece = dtype == PCS_BF16 ? 8 : 4;
  const long long esz = dtype == PCS_BF16 ? 2 : 4;
  const bool vec = ff % piece == 0 && (gu_stride * esz) % 16 == 0 && pcs::aligned16(gu) && pcs::aligned16(out);
  dim3 grid(n_rows, vec ? (ff / piece + 255) / 256 : (ff + 1023) / 1024);
  if (vec) PCS_DISPATCH(dtype, (pcs::silu_mul_kernel<T, true><<<grid, 256, 0, st>>>(static_cast<const T*>(gu), gu_stride, static_cast<T*>(out), ff, act)));
  else PCS_DISPATCH(dtype, (pcs::silu_mul_kernel<T, false><<<grid, 256, 0, st>>>(static_cast<const T*>(gu), gu_stride, static_cast<T*>(out), ff, act)));
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}
