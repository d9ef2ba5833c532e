// Rotation of queries and keys by position, unit-RMS values, and the append of K/V rows to the slot pool.
//
// One block per token; the token's sines and cosines are formed once, in shared memory, for all heads.  A coordinate pair
// of a head, (2i, 2i+1) or (i, i + rot_dims/2), turns by the angle pos * freqs[i]:
// (u, v) -> (u cos a - v sin a, v cos a + u sin a).  The frequency table comes from the host in 64-bit, so any spacing or
// rescaling of the frequencies is the caller's; the angle is formed and reduced modulo 2 pi in 64-bit (three operations) and
// its sine and cosine are taken in 32-bit of an argument in [-pi, pi], which keeps them exact to 32-bit rounding at any position.
// Coordinates past rot_dims pass unchanged.  Every value head may be divided by its root mean square (one warp per head).
// Query and key heads may first be divided by their own root mean square and multiplied by a weight vector that all heads share
// (one warp per head forms the factor, in 32-bit; the normed value is rotated without being rounded in between).
#include "seq_common.cuh"

namespace pcs {

constexpr int kMaxRotPairs = 256;  // rot_dims <= 512
constexpr int kMaxNormHeads = 512; // query + key heads of a layer with head norms

// src: `heads` heads of `dim` coordinates; dst(head) gives the head's destination; sc: the token's (sin, cos) per pair;
// inv (per head) and w (per coordinate): the head norm's factors, or null
template <typename T, typename Dst>
__device__ __forceinline__ void rotate_heads(const T* src, int heads, int dim, int rot, int interleaved, const float2* sc, const float* inv,
                                             const T* w, Dst dst) {
  const int half = rot / 2, per = half + (dim - rot);  // work items per head: rotated pairs, then single coordinates
  for (int e = threadIdx.x; e < heads * per; e += blockDim.x) {
    const int hd = e / per, i = e - hd * per;
    const T* s = src + hd * dim;
    T* d = dst(hd);
    const float f = inv ? inv[hd] : 1.f;
    if (i < half) {
      const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
      const float sn = sc[i].x, cs = sc[i].y;
      float u = ldf(s + a), v = ldf(s + b);
      if (w) { u *= f * ldf(w + a); v *= f * ldf(w + b); }
      stf(d + a, u * cs - v * sn);
      stf(d + b, v * cs + u * sn);
    } else {
      const int c = rot + (i - half);
      if (w) stf(d + c, ldf(s + c) * f * ldf(w + c));
      else d[c] = s[c];
    }
  }
}

// 1 / sqrt(mean(head^2) + eps) of `heads` heads, one warp per head
template <typename T>
__device__ __forceinline__ void head_inv_rms(const T* src, int heads, int dim, float eps, float* inv) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int hd = warp; hd < heads; hd += blockDim.x >> 5) {
    float ss = 0.f;
    for (int i = lane; i < dim; i += 32) { const float x = ldf(src + hd * dim + i); ss = fmaf(x, x, ss); }
    ss = warp_sum(ss);
    if (lane == 0) inv[hd] = 1.f / sqrtf(ss / static_cast<float>(dim) + eps);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) rope_kv_prep_kernel(const pcs_rope_params p) {
  const int t = blockIdx.x;
  const int b = p.tok_seq[t], pos = p.tok_pos[t], slot = p.seq_slot[b];
  const T* row = static_cast<const T*>(p.qkv) + static_cast<long long>(t) * p.row_stride;
  const int D = p.dim, V = p.vdim;
  __shared__ float2 sc[kMaxRotPairs];  // the token's angles, shared by all heads
  __shared__ float inv[kMaxNormHeads]; // the head norms' factors: query heads, then key heads
  for (int i = threadIdx.x; i < p.rot_dims / 2; i += blockDim.x) angle_sincos(pos, p.freqs[i], &sc[i].x, &sc[i].y);
  if (p.q_norm_w) head_inv_rms(row + p.q_off, p.n_heads, D, p.eps, inv);
  if (p.k_norm_w && p.k_off >= 0) head_inv_rms(row + p.k_off, p.n_kv_heads, D, p.eps, inv + p.n_heads);
  __syncthreads();
  T* qo = static_cast<T*>(p.q_out) + static_cast<long long>(t) * p.n_heads * D;
  rotate_heads(row + p.q_off, p.n_heads, D, p.rot_dims, p.interleaved, sc, p.q_norm_w ? inv : nullptr, static_cast<const T*>(p.q_norm_w),
               [&](int hd) { return qo + hd * D; });
  if (p.k_off < 0) return;
  T* kp = static_cast<T*>(p.k_pool) + static_cast<long long>(slot) * p.n_kv_heads * p.cap * D;
  rotate_heads(row + p.k_off, p.n_kv_heads, D, p.rot_dims, p.interleaved, sc, p.k_norm_w ? inv + p.n_heads : nullptr,
               static_cast<const T*>(p.k_norm_w), [&](int hd) { return kp + (static_cast<long long>(hd) * p.cap + pos) * D; });
  T* vp = static_cast<T*>(p.v_pool) + static_cast<long long>(slot) * p.n_kv_heads * p.cap * V;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int hd = warp; hd < p.n_kv_heads; hd += blockDim.x >> 5) {
    const T* v = row + p.v_off + hd * V;
    float inv = 1.f;
    if (p.v_unit_rms) {
      float ss = 0.f;
      for (int i = lane; i < V; i += 32) { const float x = ldf(v + i); ss = fmaf(x, x, ss); }
      ss = warp_sum(ss);
      inv = 1.f / sqrtf(ss / static_cast<float>(V) + p.eps);
    }
    T* d = vp + (static_cast<long long>(hd) * p.cap + pos) * V;
    for (int i = lane; i < V; i += 32) stf(d + i, ldf(v + i) * inv);
  }
}

}  // namespace pcs

PCS_API int pcs_rope_kv_prep(const pcs_rope_params* p, void* stream) {
  PCS_REQUIRE(p, "pcs_rope_kv_prep: null params");
  if (p->n_tokens == 0) return PCS_OK;
  PCS_REQUIRE(p->qkv && p->q_out && p->tok_seq && p->tok_pos && p->seq_slot, "pcs_rope_kv_prep: null tensor");
  PCS_REQUIRE(p->k_off < 0 || (p->k_pool && p->v_pool && p->cap > 0), "pcs_rope_kv_prep: keys and values need their pools");
  PCS_REQUIRE(p->n_heads > 0 && p->n_kv_heads > 0 && p->dim > 0 && p->vdim > 0, "pcs_rope_kv_prep: bad sizes");
  PCS_REQUIRE(p->rot_dims >= 0 && p->rot_dims <= p->dim && p->rot_dims % 2 == 0 && (p->rot_dims == 0 || p->freqs) && p->rot_dims <= 2 * pcs::kMaxRotPairs,
              "pcs_rope_kv_prep: rot_dims %d must be even, at most dim %d and %d, with a frequency table", p->rot_dims, p->dim, 2 * pcs::kMaxRotPairs);
  PCS_REQUIRE((!p->q_norm_w && !p->k_norm_w) || p->n_heads + p->n_kv_heads <= pcs::kMaxNormHeads, "pcs_rope_kv_prep: head norms serve at most %d query + key heads",
              pcs::kMaxNormHeads);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  PCS_DISPATCH(p->dtype, pcs::rope_kv_prep_kernel<T><<<p->n_tokens, 256, 0, st>>>(*p));
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}
