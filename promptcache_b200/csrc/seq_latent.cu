// Low-rank (latent) attention over the slot pool.
//
// A token's keys and values of all heads are functions of one latent vector c (kv_rank numbers) and one rotated key part
// (rot_dim numbers, shared by the heads):  k_h = [U_k,h c | rot],  v_h = U_v,h c.  Only [c | rot] is cached, one row per
// token.  Attention then runs in one of two equivalent forms:
//   expanded   (prompts)   k_h and v_h of the whole context are formed by one matrix product from the cached latents and
//                          written to a dense per-step pool (pcs_latent_expand); plain multi-head attention over it;
//   latent     (decoding)  the query's plain part is carried into the latent space, q'_h = U_k,h^T q_h, so the score is
//                          q'_h . c + q_rot . rot and the cached rows serve as keys AND (their leading kv_rank numbers) as
//                          values of every head; the result is carried back by U_v,h.
// pcs_latent_prep   one block per token: RMS norms (32-bit statistics) of the query latent and of c, rotation of the
//                   shared key part by the token's position, append of [c | rot] to the pool.
// pcs_latent_q      one block per token: rotation of every head's rotated query part; optionally packs [q'_h | rotated part].
// pcs_latent_gather / pcs_latent_expand   context rows out of the pool, and per-head rows into the dense pool.
// pcs_head_gate     the per-head output gate sigmoid(g[t, h]).
// Rotation pairs coordinate i with i + rot_dim / 2; cos and sin carry a common multiplier (a frequency rescaling's
// attention factor).  Angles are formed in 64-bit from a host-made frequency table.
#include "seq_common.cuh"

namespace pcs {

constexpr int kLatMaxRotPairs = 256;

template <typename T>
__global__ void __launch_bounds__(256) latent_prep_kernel(const pcs_latent_prep_params p) {
  __shared__ float red[33];
  __shared__ float2 sc[kLatMaxRotPairs];
  const int t = blockIdx.x;
  const int b = p.tok_seq[t], pos = p.tok_pos[t], slot = p.seq_slot[b];
  const T* row = static_cast<const T*>(p.proj) + static_cast<long long>(t) * p.row_stride;
  const int Q = p.q_rank, C = p.kv_rank, R = p.rot_dim, half = R / 2;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float sn, cs;
    angle_sincos(pos, p.freqs[i], &sn, &cs);
    sc[i] = make_float2(sn * p.rot_mult, cs * p.rot_mult);
  }
  if (p.cq_out) {
    const T* cq = row + p.cq_off;
    float ss = 0.f;
    for (int i = threadIdx.x; i < Q; i += blockDim.x) { const float v = ldf(cq + i); ss = fmaf(v, v, ss); }
    ss = block_sum(ss, red);
    const float inv = 1.f / sqrtf(ss / static_cast<float>(Q) + p.eps);
    const T* w = static_cast<const T*>(p.cq_norm_w);
    T* o = static_cast<T*>(p.cq_out) + static_cast<long long>(t) * Q;
    for (int i = threadIdx.x; i < Q; i += blockDim.x) stf(o + i, ldf(cq + i) * inv * ldf(w + i));
  }
  const T* ckv = row + p.ckv_off;
  float ss = 0.f;
  for (int i = threadIdx.x; i < C; i += blockDim.x) { const float v = ldf(ckv + i); ss = fmaf(v, v, ss); }
  ss = block_sum(ss, red);  // its barriers also publish sc
  const float inv = 1.f / sqrtf(ss / static_cast<float>(C) + p.eps);
  const T* w = static_cast<const T*>(p.ckv_norm_w);
  T* dst = static_cast<T*>(p.pool) + (static_cast<long long>(slot) * p.cap + pos) * (C + R);
  for (int i = threadIdx.x; i < C; i += blockDim.x) stf(dst + i, ldf(ckv + i) * inv * ldf(w + i));
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float u = ldf(ckv + C + i), v = ldf(ckv + C + half + i);
    stf(dst + C + i, u * sc[i].y - v * sc[i].x);
    stf(dst + C + half + i, v * sc[i].y + u * sc[i].x);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) latent_q_kernel(const pcs_latent_q_params p) {
  __shared__ float2 sc[kLatMaxRotPairs];
  const long long t = blockIdx.x;
  const int pos = p.tok_pos[t];
  const int H = p.n_heads, D = p.dim, R = p.rot_dim, half = R / 2, C = p.kv_rank;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float sn, cs;
    angle_sincos(pos, p.freqs[i], &sn, &cs);
    sc[i] = make_float2(sn * p.rot_mult, cs * p.rot_mult);
  }
  __syncthreads();
  const T* q = static_cast<const T*>(p.q) + t * H * (D + R);
  const int lead = p.q_lat ? C : D;   // numbers in front of the rotated part of an output head
  T* qo = static_cast<T*>(p.q_out) + t * H * (lead + R);
  const int tid0 = blockIdx.y * blockDim.x + threadIdx.x, nthr = gridDim.y * blockDim.x;   // a token's work is spread over gridDim.y blocks
  for (int e = tid0; e < H * half; e += nthr) {
    const int h = e / half, i = e - h * half;
    const T* s = q + h * (D + R) + D;
    const float u = ldf(s + i), v = ldf(s + half + i);
    T* d = qo + h * (lead + R) + lead;
    stf(d + i, u * sc[i].y - v * sc[i].x);
    stf(d + half + i, v * sc[i].y + u * sc[i].x);
  }
  if (p.q_lat) {
    const T* ql = static_cast<const T*>(p.q_lat) + t * p.lat_tok_stride;
    for (int e = tid0; e < H * C; e += nthr) {
      const int h = e / C, c = e - h * C;
      qo[h * (C + R) + c] = ql[h * p.lat_head_stride + c];
    }
  } else if (p.q_out != p.q) {
    for (int e = tid0; e < H * D; e += nthr) {
      const int h = e / D, c = e - h * D;
      qo[h * (D + R) + c] = q[h * (D + R) + c];
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) latent_gather_kernel(const T* __restrict__ pool, int cap, int row_width, int width, T* __restrict__ out,
                                                            const int32_t* __restrict__ ctx_seq, const int32_t* __restrict__ ctx_pos,
                                                            const int32_t* __restrict__ seq_slot) {
  const long long n = blockIdx.x;
  const int slot = seq_slot[ctx_seq[n]], pos = ctx_pos[n];
  const T* src = pool + (static_cast<long long>(slot) * cap + pos) * row_width;
  T* dst = out + n * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = src[i];
}

template <typename T>
__global__ void __launch_bounds__(256) latent_expand_kernel(const pcs_latent_expand_params p) {
  const long long n = blockIdx.x;
  const int b = p.ctx_seq[n], pos = p.ctx_pos[n], slot = p.seq_slot[b];
  const int H = p.n_heads, D = p.dim, V = p.vdim, R = p.rot_dim, C = p.kv_rank;
  const T* kv = static_cast<const T*>(p.kv) + n * p.kv_stride;
  const T* rot = static_cast<const T*>(p.pool) + (static_cast<long long>(slot) * p.cap + pos) * (C + R) + C;
  T* kd = static_cast<T*>(p.k_dense) + (static_cast<long long>(b) * H * p.cap_dense + pos) * (D + R);
  T* vd = static_cast<T*>(p.v_dense) + (static_cast<long long>(b) * H * p.cap_dense + pos) * V;
  const long long k_head = static_cast<long long>(p.cap_dense) * (D + R), v_head = static_cast<long long>(p.cap_dense) * V;
  for (int e = threadIdx.x; e < H * (D + R); e += blockDim.x) {
    const int h = e / (D + R), i = e - h * (D + R);
    kd[h * k_head + i] = i < D ? kv[h * D + i] : rot[i - D];
  }
  for (int e = threadIdx.x; e < H * V; e += blockDim.x) {
    const int h = e / V, i = e - h * V;
    vd[h * v_head + i] = kv[H * D + e];
  }
}

template <typename T>
__global__ void __launch_bounds__(256) head_gate_kernel(const T* __restrict__ o, long long o_tok_stride, long long o_head_stride, const T* __restrict__ g,
                                                        long long g_stride, T* __restrict__ out, int H, int V) {
  const long long t = blockIdx.x;
  for (int e = blockIdx.y * blockDim.x + threadIdx.x; e < H * V; e += gridDim.y * blockDim.x) {
    const int h = e / V, c = e - h * V;
    stf(out + t * H * V + e, ldf(o + t * o_tok_stride + h * o_head_stride + c) * sigmoidf_(ldf(g + t * g_stride + h)));
  }
}

}  // namespace pcs

PCS_API int pcs_latent_prep(const pcs_latent_prep_params* p, void* stream) {
  PCS_REQUIRE(p, "pcs_latent_prep: null params");
  if (p->n_tokens == 0) return PCS_OK;
  PCS_REQUIRE(p->proj && p->ckv_norm_w && p->pool && p->tok_seq && p->tok_pos && p->seq_slot, "pcs_latent_prep: null tensor");
  PCS_REQUIRE(p->cq_out == nullptr || (p->cq_norm_w != nullptr && p->q_rank > 0), "pcs_latent_prep: the query latent needs its norm weight and size");
  PCS_REQUIRE(p->kv_rank > 0 && p->rot_dim >= 0 && p->rot_dim % 2 == 0 && p->rot_dim <= 2 * pcs::kLatMaxRotPairs && (p->rot_dim == 0 || p->freqs) && p->cap > 0,
              "pcs_latent_prep: bad sizes kv_rank=%d rot_dim=%d cap=%d", p->kv_rank, p->rot_dim, p->cap);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  PCS_DISPATCH(p->dtype, pcs::latent_prep_kernel<T><<<p->n_tokens, 256, 0, st>>>(*p));
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}

PCS_API int pcs_latent_q(const pcs_latent_q_params* p, void* stream) {
  PCS_REQUIRE(p, "pcs_latent_q: null params");
  if (p->n_tokens == 0) return PCS_OK;
  PCS_REQUIRE(p->q && p->q_out && p->tok_pos, "pcs_latent_q: null tensor");
  PCS_REQUIRE(p->n_heads > 0 && p->dim >= 0 && p->rot_dim >= 0 && p->rot_dim % 2 == 0 && p->rot_dim <= 2 * pcs::kLatMaxRotPairs && (p->rot_dim == 0 || p->freqs),
              "pcs_latent_q: bad sizes H=%d dim=%d rot_dim=%d", p->n_heads, p->dim, p->rot_dim);
  PCS_REQUIRE(p->q_lat == nullptr || (p->kv_rank > 0 && p->q_out != p->q), "pcs_latent_q: latent queries need kv_rank and an output of their own");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // few tokens (decoding): a token's copies are spread over several blocks, two elements per thread
  const int per_token = p->n_heads * ((p->q_lat ? p->kv_rank : (p->q_out != p->q ? p->dim : 0)) + p->rot_dim / 2);
  int ny = p->n_tokens >= 256 ? 1 : (per_token + 511) / 512;
  if (ny > 64) ny = 64;
  if (ny < 1) ny = 1;
  PCS_DISPATCH(p->dtype, pcs::latent_q_kernel<T><<<dim3(p->n_tokens, ny), 256, 0, st>>>(*p));
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}

PCS_API int pcs_latent_gather(const void* pool, int cap, int row_width, int width, void* out, const int32_t* ctx_seq, const int32_t* ctx_pos,
                              const int32_t* seq_slot, int n_ctx, int dtype, void* stream) {
  if (n_ctx == 0) return PCS_OK;
  PCS_REQUIRE(pool && out && ctx_seq && ctx_pos && seq_slot && cap > 0 && width > 0 && width <= row_width, "pcs_latent_gather: bad arguments");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  PCS_DISPATCH(dtype, pcs::latent_gather_kernel<T><<<n_ctx, 256, 0, st>>>(static_cast<const T*>(pool), cap, row_width, width, static_cast<T*>(out), ctx_seq,
                                                                          ctx_pos, seq_slot));
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}

PCS_API int pcs_latent_expand(const pcs_latent_expand_params* p, void* stream) {
  PCS_REQUIRE(p, "pcs_latent_expand: null params");
  if (p->n_ctx == 0) return PCS_OK;
  PCS_REQUIRE(p->kv && p->pool && p->k_dense && p->v_dense && p->ctx_seq && p->ctx_pos && p->seq_slot, "pcs_latent_expand: null tensor");
  PCS_REQUIRE(p->n_heads > 0 && p->dim >= 0 && p->vdim > 0 && p->kv_rank > 0 && p->rot_dim >= 0 && p->cap > 0 && p->cap_dense > 0, "pcs_latent_expand: bad sizes");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  PCS_DISPATCH(p->dtype, pcs::latent_expand_kernel<T><<<p->n_ctx, 256, 0, st>>>(*p));
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}

PCS_API int pcs_head_gate(const void* o, int64_t o_tok_stride, int64_t o_head_stride, const void* g, int64_t g_stride, void* out, int n_tokens,
                          int n_heads, int vdim, int dtype, void* stream) {
  if (n_tokens == 0) return PCS_OK;
  PCS_REQUIRE(o && g && out && n_heads > 0 && vdim > 0, "pcs_head_gate: bad arguments");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int ny = n_tokens >= 256 ? 1 : (n_heads * vdim + 511) / 512;
  if (ny > 64) ny = 64;
  PCS_DISPATCH(dtype, pcs::head_gate_kernel<T><<<dim3(n_tokens, ny), 256, 0, st>>>(static_cast<const T*>(o), o_tok_stride, o_head_stride, static_cast<const T*>(g),
                                                                        g_stride, static_cast<T*>(out), n_heads, vdim));
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}
