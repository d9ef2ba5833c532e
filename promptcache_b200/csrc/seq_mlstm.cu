// Matrix-memory recurrent layer (mLSTM) over the slot pool.
//
// Per head, with log input gate i_t, log forget gate f_t and a running maximum m (m_0 = 0):
//     m_t = max(f_t + m_{t-1}, i_t)
//     S_t = exp(f_t + m_{t-1} - m_t) S_{t-1} + exp(i_t - m_t) k_t v_t^T          (S: dim x vdim)
//     n_t = exp(f_t + m_{t-1} - m_t) n_{t-1} + exp(i_t - m_t) k_t
//     o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
// followed by o_t / rms(o_t) per head, the norm weight and the output gate sigmoid(g_t).  S, n, m live in 32-bit floats in
// the slot pool and are carried from step to step; a sequence whose slot holds no tokens yet starts from zero.
//
// pcs_mlstm_gates  one block per token: the two gate pre-activations of every head as 32-bit dot products, capped by
//                  cap * tanh(. / cap); the forget gate additionally through logsigmoid.
// pcs_mlstm_scan   the token-by-token recurrence, one block per sequence, head and slice of value columns (state in registers
//                  for dim <= 256, else in shared memory), then the per-head output norm with the output gate and the commit
//                  of the new n and m.
#include "seq_common.cuh"

namespace pcs {

template <typename T>
__global__ void __launch_bounds__(256) mlstm_gates_kernel(const T* __restrict__ h, long long h_stride, const T* __restrict__ w_i,
                                                          const T* __restrict__ w_f, const float* __restrict__ b_i,
                                                          const float* __restrict__ b_f, float* __restrict__ ig,
                                                          float* __restrict__ fg, int width, int heads, float cap) {
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const T* hr = h + t * h_stride;
  constexpr int N = Vec<T>::n;
  const bool vec = width % N == 0 && (h_stride * sizeof(T)) % 16 == 0 && ((reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(w_i) |
                                                                             reinterpret_cast<uintptr_t>(w_f)) & 15) == 0;
  for (int o = warp; o < 2 * heads; o += nw) {
    const int head = o >> 1, is_f = o & 1;
    const T* w = (is_f ? w_f : w_i) + static_cast<long long>(head) * width;
    float a = 0.f;
    if (vec) {  // 16-byte pieces, two accumulators
      float a1 = 0.f;
      for (int i = lane * N; i < width; i += 32 * N) {
        float hv[N], wv[N];
        ld16(hr + i, hv);
        ld16(w + i, wv);
#pragma unroll
        for (int e = 0; e < N; e += 2) { a = fmaf(hv[e], wv[e], a); a1 = fmaf(hv[e + 1], wv[e + 1], a1); }
      }
      a += a1;
    } else {
      for (int i = lane; i < width; i += 32) a = fmaf(ldf(hr + i), ldf(w + i), a);
    }
    a = warp_sum(a);
    if (lane == 0) {
      const float z = cap * tanhf((a + (is_f ? b_f[head] : b_i[head])) / cap);
      if (is_f) fg[static_cast<long long>(t) * heads + head] = logsigmoidf_(z);
      else ig[static_cast<long long>(t) * heads + head] = z;
    }
  }
}

// Grid (sequence, head, slice of value columns): the columns of S evolve independently given the gates, k and q, so a head's
// state is cut into slices of VS columns, one block each (a 256 x 512 state does not fit one SM's shared memory, and a
// decode step gets heads x slices blocks instead of heads).  The scalar n . q is recomputed by every slice; only slice 0
// stores n and m.  The block writes the unnormalised o_t = S_t^T q_t / den into a 32-bit buffer; the per-head norm needs all
// slices and runs afterwards (mlstm_out_kernel).  blockDim.x = round_up(VS * R, 32): thread (r, c) owns rows r, r + R, ...
// of column c; threads past VS * R only take part in loads and reductions.
template <typename T>
__global__ void __launch_bounds__(1024) mlstm_scan_kernel(const pcs_mlstm_params p, float* __restrict__ o_raw,
                                                          float* __restrict__ nm_new, int VS, int R) {
  extern __shared__ float sm[];
  __shared__ float red[33];
  const int D = p.dim, V = p.vdim, H = p.heads;
  const int v0 = blockIdx.z * VS, vs = min(VS, V - v0);
  float* S = sm;                 // [D][VS]
  float* nvec = S + D * VS;      // [D]
  float* ks = nvec + D;          // [D]
  float* qs = ks + D;            // [D]
  float* vsm = qs + D;           // [VS]
  float* part = vsm + VS;        // [R][VS]
  const int b = blockIdx.x, head = blockIdx.y, tid = threadIdx.x, nthr = blockDim.x;
  const int slot = p.seq_slot[b], pos0 = p.seq_pos0[b], len = p.seq_len[b], off = p.seq_off[b];
  if (len <= 0) return;
  float* Sg = p.s_pool + (static_cast<long long>(slot) * H + head) * D * V;
  float* ng = p.n_pool + (static_cast<long long>(slot) * H + head) * D;
  float* mg = p.m_pool + static_cast<long long>(slot) * H + head;
  const bool fresh = pos0 == 0;
  for (int e = tid; e < D * vs; e += nthr) {
    const int d = e / vs, c = e - d * vs;
    S[d * VS + c] = fresh ? 0.f : Sg[d * V + v0 + c];
  }
  for (int d = tid; d < D; d += nthr) nvec[d] = fresh ? 0.f : ng[d];
  float m = fresh ? 0.f : *mg;
  const int c = tid % VS, r = tid / VS;
  const bool active = r < R && c < vs;
  __syncthreads();
  for (int i = 0; i < len; ++i) {
    const long long t = off + i;
    const T* row = static_cast<const T*>(p.proj) + t * p.row_stride;
    for (int d = tid; d < D; d += nthr) {
      ks[d] = ldf(row + p.k_off + head * D + d);
      qs[d] = ldf(row + p.q_off + head * D + d) * p.q_scale;
    }
    for (int e = tid; e < vs; e += nthr) vsm[e] = ldf(row + p.v_off + head * V + v0 + e);
    const float ig = p.ig[t * H + head], fg = p.fg[t * H + head];
    const float m_new = fmaxf(fg + m, ig);
    const float a = expf(fg + m - m_new), bb = expf(ig - m_new);
    m = m_new;
    __syncthreads();
    float nq = 0.f;
    for (int d = tid; d < D; d += nthr) {
      const float nn = fmaf(a, nvec[d], bb * ks[d]);
      nvec[d] = nn;
      nq = fmaf(nn, qs[d], nq);
    }
    if (active) {
      const float bv = bb * vsm[c];
      float num = 0.f;
      for (int d = r; d < D; d += R) {
        const float sv = fmaf(a, S[d * VS + c], ks[d] * bv);
        S[d * VS + c] = sv;
        num = fmaf(sv, qs[d], num);
      }
      part[r * VS + c] = num;
    }
    nq = block_sum(nq, red);  // its barriers also publish `part`
    const float den = fmaxf(fabsf(nq), expf(-m)) + 1e-6f;
    if (tid < vs) {
      float o = 0.f;
      for (int rr = 0; rr < R; ++rr) o += part[rr * VS + tid];
      o_raw[t * (static_cast<long long>(H) * V) + head * V + v0 + tid] = o / den;
    }
    __syncthreads();  // ks / qs / vsm / part are rewritten by the next token
  }
  for (int e = tid; e < D * vs; e += nthr) {
    const int d = e / vs, cc = e - d * vs;
    Sg[d * V + v0 + cc] = S[d * VS + cc];
  }
  // the other slices of this head may not have read the old n and m yet: the new ones are parked and committed afterwards
  if (blockIdx.z == 0) {
    float* dst = nm_new + (static_cast<long long>(b) * H + head) * (D + 1);
    for (int d = tid; d < D; d += nthr) dst[d] = nvec[d];
    if (tid == 0) dst[D] = m;
  }
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem))), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem))), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

constexpr int kScanRing = 24;   // shared-memory slots of tokens whose k / q / v / gates are in flight or waiting
constexpr int kScanAhead = 16;  // tokens requested ahead of the arithmetic
constexpr int kScanGroup = 4;   // tokens computed between two block barriers

// DR consecutive elements at p (aligned to their total size) as floats; bfloat16 is widened with integer operations
template <int N>
__device__ __forceinline__ void ld_vec(const float* p, float (&o)[N]) {
  if constexpr (N >= 4) {
#pragma unroll
    for (int i = 0; i < N; i += 4) {
      const float4 v = *reinterpret_cast<const float4*>(p + i);
      o[i] = v.x; o[i + 1] = v.y; o[i + 2] = v.z; o[i + 3] = v.w;
    }
  } else if constexpr (N == 2) {
    const float2 v = *reinterpret_cast<const float2*>(p);
    o[0] = v.x; o[1] = v.y;
  } else {
    o[0] = p[0];
  }
}
template <int N>
__device__ __forceinline__ void ld_vec(const __nv_bfloat16* p, float (&o)[N]) {
  if constexpr (N == 1) {
    o[0] = __uint_as_float(static_cast<uint32_t>(*reinterpret_cast<const unsigned short*>(p)) << 16);
  } else {
    uint32_t w[N / 2];
    if constexpr (N == 8) {
      const uint4 v = *reinterpret_cast<const uint4*>(p);
      w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
    } else if constexpr (N == 4) {
      const uint2 v = *reinterpret_cast<const uint2*>(p);
      w[0] = v.x; w[1] = v.y;
    } else {
      w[0] = *reinterpret_cast<const uint32_t*>(p);
    }
#pragma unroll
    for (int i = 0; i < N / 2; ++i) {
      o[2 * i] = __uint_as_float(w[i] << 16);
      o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
}

// The same recurrence with the state in REGISTERS (dim <= 256, 16-byte aligned projections).  A warp owns 8 value columns;
// lane l owns the DR = ceil(dim / 32) rows l*DR .. l*DR + DR - 1 of them, so a thread keeps a DR x 8 patch of S, and every
// warp keeps its own copy of n (DR values per lane) so that n . q needs no block-wide exchange.  Per token a thread does
// 2 * DR * 8 fused multiply-adds from 2 * DR + 8 shared-memory values; the 8 column sums over the 32 lanes are one
// reduce-scatter butterfly (9 shuffles).  k, q, v and the gates of the next tokens arrive through a ring of kScanRing
// shared-memory slots filled by cp.async, kScanAhead tokens ahead of the arithmetic; kScanGroup tokens are computed between two
// block barriers (their independent parts overlap), and no global-memory latency is exposed.  The order of every sum is fixed by DR alone: a token's result does not depend on how the
// sequence is cut into steps, on the batch, or on the number of warps per block.
template <typename T, int DR>
__global__ void __launch_bounds__(512) mlstm_scan_reg_kernel(const pcs_mlstm_params p, float* __restrict__ o_raw,
                                                             float* __restrict__ nm_new, int W) {
  extern __shared__ __align__(16) unsigned char ring[];
  constexpr int ES = static_cast<int>(sizeof(T)), PER = 16 / ES;
  const int D = p.dim, V = p.vdim, H = p.heads;
  const int slot_bytes = (2 * D + 8 * W) * ES + 16;  // k[D] q[D] v[8W] ig fg (pad)
  const int b = blockIdx.x, head = blockIdx.y, v0 = blockIdx.z * 8 * W;
  const int tid = threadIdx.x, nthr = blockDim.x, warp = tid >> 5, lane = tid & 31;
  const int slot = p.seq_slot[b], pos0 = p.seq_pos0[b], len = p.seq_len[b], off = p.seq_off[b];
  if (len <= 0) return;
  const int c0 = v0 + warp * 8, d0 = lane * DR;
  const int ncol = max(0, min(8, V - c0));
  const T* proj = static_cast<const T*>(p.proj);
  const int ck = D / PER, cv = 8 * W / PER;
  // what this thread copies per token is the same for every token: up to 3 pieces, described once
  //   kind 0: 16 bytes of the projection row   1: 16 zero bytes   2: the input gate   3: the forget gate   4: nothing
  int kind[3], src[3], dst[3];
#pragma unroll
  for (int j = 0; j < 3; ++j) {
    const int e = tid + j * nthr;
    kind[j] = 4;
    src[j] = dst[j] = 0;
    if (e < ck) {
      kind[j] = 0; src[j] = p.k_off + head * D + e * PER; dst[j] = e * 16;
    } else if (e < 2 * ck) {
      kind[j] = 0; src[j] = p.q_off + head * D + (e - ck) * PER; dst[j] = D * ES + (e - ck) * 16;
    } else if (e < 2 * ck + cv) {
      const int c = e - 2 * ck, col = v0 + c * PER;
      kind[j] = col < V ? 0 : 1; src[j] = p.v_off + head * V + col; dst[j] = 2 * D * ES + c * 16;
    } else if (e == 2 * ck + cv) {
      kind[j] = 2; dst[j] = (2 * D + 8 * W) * ES;
    } else if (e == 2 * ck + cv + 1) {
      kind[j] = 3; dst[j] = (2 * D + 8 * W) * ES + 4;
    }
  }
  auto issue = [&](int i) {  // token i of this entry into slot i % kScanRing
    const long long t = off + i;
    unsigned char* s = ring + (i % kScanRing) * slot_bytes;
    const T* row = proj + t * p.row_stride;
#pragma unroll
    for (int j = 0; j < 3; ++j) {
      if (kind[j] == 0) cp_async16(s + dst[j], row + src[j]);
      else if (kind[j] == 1) *reinterpret_cast<uint4*>(s + dst[j]) = make_uint4(0u, 0u, 0u, 0u);
      else if (kind[j] == 2) cp_async4(s + dst[j], p.ig + t * H + head);
      else if (kind[j] == 3) cp_async4(s + dst[j], p.fg + t * H + head);
    }
  };
  for (int i = 0; i < kScanAhead; ++i) {
    if (i < len) issue(i);
    cp_async_commit();
  }
  float* Sg = p.s_pool + (static_cast<long long>(slot) * H + head) * D * V;
  const float* ng = p.n_pool + (static_cast<long long>(slot) * H + head) * D;
  const bool fresh = pos0 == 0;
  float S[DR][8], nreg[DR];
#pragma unroll
  for (int r = 0; r < DR; ++r) {
    const int d = d0 + r;
    nreg[r] = (!fresh && d < D) ? ng[d] : 0.f;
#pragma unroll
    for (int c = 0; c < 8; ++c) S[r][c] = (!fresh && d < D && c < ncol) ? Sg[static_cast<long long>(d) * V + c0 + c] : 0.f;
  }
  float m = fresh ? 0.f : p.m_pool[static_cast<long long>(slot) * H + head];
  for (int i0 = 0; i0 < len; i0 += kScanGroup) {
    cp_async_wait<kScanAhead - kScanGroup>();  // this thread's copies of tokens i0 .. i0 + 3 have landed ...
    __syncthreads();                           // ... and everybody's; the slots of the previous groups have been read by all warps
#pragma unroll
    for (int u = 0; u < kScanGroup; ++u) {
      if (i0 + kScanAhead + u < len) issue(i0 + kScanAhead + u);
      cp_async_commit();
    }
#pragma unroll
    for (int u = 0; u < kScanGroup; ++u) {
    const int i = i0 + u;
    if (i >= len) break;
    const long long t = off + i;
    const unsigned char* cur = ring + (i % kScanRing) * slot_bytes;
    const T* kb = reinterpret_cast<const T*>(cur);
    const T* qb = kb + D;
    const T* vb = qb + D;
    const float ig = *reinterpret_cast<const float*>(cur + (2 * D + 8 * W) * ES);
    const float fg = *reinterpret_cast<const float*>(cur + (2 * D + 8 * W) * ES + 4);
    float kk[DR], qq[DR], vv[8];
    if (d0 < D) {  // dim is a multiple of the 16-byte element count, so a lane's DR rows are inside or outside as a whole ...
      ld_vec<DR>(kb + d0, kk);
      ld_vec<DR>(qb + d0, qq);
    }
#pragma unroll
    for (int r = 0; r < DR; ++r) {  // ... except 8 float rows over a dim that is 4 mod 8
      const bool ok = d0 + r < D;
      kk[r] = ok ? kk[r] : 0.f;
      qq[r] = ok ? qq[r] * p.q_scale : 0.f;
    }
    ld_vec<8>(vb + warp * 8, vv);
    const float m_new = fmaxf(fg + m, ig);
    const float a = expf(fg + m - m_new), bb = expf(ig - m_new);
    m = m_new;
    float nq = 0.f;
#pragma unroll
    for (int r = 0; r < DR; ++r) {
      nreg[r] = fmaf(a, nreg[r], bb * kk[r]);
      nq = fmaf(nreg[r], qq[r], nq);
    }
    nq = warp_sum(nq);
    const float den = fmaxf(fabsf(nq), expf(-m)) + 1e-6f;
    float num[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const float bv = bb * vv[c];
      float acc = 0.f;
#pragma unroll
      for (int r = 0; r < DR; ++r) {
        S[r][c] = fmaf(a, S[r][c], kk[r] * bv);
        acc = fmaf(S[r][c], qq[r], acc);
      }
      num[c] = acc;
    }
    // reduce-scatter over the lanes: afterwards lane l holds the sum of column ((l >> 4) & 1) * 4 + ((l >> 3) & 1) * 2 + ((l >> 2) & 1)
    float x4[4], x2[2], x1;
    {
      const bool up = lane & 16;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float recv = __shfl_xor_sync(0xffffffffu, up ? num[j] : num[j + 4], 16);
        x4[j] = (up ? num[j + 4] : num[j]) + recv;
      }
    }
    {
      const bool up = lane & 8;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float recv = __shfl_xor_sync(0xffffffffu, up ? x4[j] : x4[j + 2], 8);
        x2[j] = (up ? x4[j + 2] : x4[j]) + recv;
      }
    }
    {
      const bool up = lane & 4;
      const float recv = __shfl_xor_sync(0xffffffffu, up ? x2[0] : x2[1], 4);
      x1 = (up ? x2[1] : x2[0]) + recv;
    }
    x1 += __shfl_xor_sync(0xffffffffu, x1, 2);
    x1 += __shfl_xor_sync(0xffffffffu, x1, 1);
    const int col = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
    if ((lane & 3) == 0 && col < ncol) o_raw[t * (static_cast<long long>(H) * V) + head * V + c0 + col] = x1 / den;
    }
  }
#pragma unroll
  for (int r = 0; r < DR; ++r) {
    const int d = d0 + r;
    if (d < D) {
#pragma unroll
      for (int c = 0; c < 8; ++c)
        if (c < ncol) Sg[static_cast<long long>(d) * V + c0 + c] = S[r][c];
    }
  }
  // other blocks of this head may not have read the old n and m yet: the new ones are parked and committed afterwards
  if (blockIdx.z == 0 && warp == 0) {
    float* dst = nm_new + (static_cast<long long>(b) * H + head) * (D + 1);
#pragma unroll
    for (int r = 0; r < DR; ++r)
      if (d0 + r < D) dst[d0 + r] = nreg[r];
    if (lane == 0) dst[D] = m;
  }
}

__global__ void __launch_bounds__(128) mlstm_commit_kernel(const pcs_mlstm_params p, const float* __restrict__ nm_new) {
  const int b = blockIdx.x, head = blockIdx.y, D = p.dim, H = p.heads;
  if (p.seq_len[b] <= 0) return;
  const int slot = p.seq_slot[b];
  const float* src = nm_new + (static_cast<long long>(b) * H + head) * (D + 1);
  float* ng = p.n_pool + (static_cast<long long>(slot) * H + head) * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) ng[d] = src[d];
  if (threadIdx.x == 0) p.m_pool[static_cast<long long>(slot) * H + head] = src[D];
}

// out[t, head, :] = o / rms(o) * norm_w * sigmoid(g): one block per (token, head).
template <typename T>
__global__ void __launch_bounds__(256) mlstm_out_kernel(const pcs_mlstm_params p, const float* __restrict__ o_raw) {
  __shared__ float red[33];
  const long long t = blockIdx.x;
  const int head = blockIdx.y, V = p.vdim, H = p.heads;
  const float* o = o_raw + t * (static_cast<long long>(H) * V) + head * V;
  const T* g = static_cast<const T*>(p.proj) + t * p.row_stride + p.g_off + head * V;
  const T* nw = static_cast<const T*>(p.norm_w) + head * V;
  float ss = 0.f;
  for (int c = threadIdx.x; c < V; c += blockDim.x) ss = fmaf(o[c], o[c], ss);
  ss = block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / static_cast<float>(V) + p.eps);
  T* out = static_cast<T*>(p.out) + t * (static_cast<long long>(H) * V) + head * V;
  for (int c = threadIdx.x; c < V; c += blockDim.x) stf(out + c, o[c] * inv * ldf(nw + c) * sigmoidf_(ldf(g + c)));
}

}  // namespace pcs

namespace pcs {
int launch_mlstm_chunk(const pcs_mlstm_params& p, float* nm_new, cudaStream_t st);
constexpr int kChunkMinLen = 24;  // shorter steps (decoding, tails of a prompt) go token by token
}  // namespace pcs

PCS_API int pcs_mlstm_gates(const void* h, int64_t h_stride, const void* w_i, const void* w_f, const float* b_i, const float* b_f,
                            float* ig, float* fg, int n_tokens, int width, int heads, float cap, int dtype, void* stream) {
  if (n_tokens == 0) return PCS_OK;
  PCS_REQUIRE(h && w_i && w_f && b_i && b_f && ig && fg && width > 0 && heads > 0 && cap > 0.f, "pcs_mlstm_gates: bad arguments");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  PCS_DISPATCH(dtype, pcs::mlstm_gates_kernel<T><<<n_tokens, 256, 0, st>>>(static_cast<const T*>(h), h_stride, static_cast<const T*>(w_i),
                                                                           static_cast<const T*>(w_f), b_i, b_f, ig, fg, width, heads, cap));
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}

PCS_API int pcs_mlstm_scan(const pcs_mlstm_params* p, void* stream) {
  PCS_REQUIRE(p, "pcs_mlstm_scan: null params");
  if (p->n_seqs == 0 || p->n_tokens == 0) return PCS_OK;
  PCS_REQUIRE(p->proj && p->ig && p->fg && p->norm_w && p->out && p->s_pool && p->n_pool && p->m_pool && p->seq_slot && p->seq_pos0 &&
              p->seq_len && p->seq_off && p->o_raw, "pcs_mlstm_scan: null tensor");
  PCS_REQUIRE(p->heads > 0 && p->heads <= 65535 && p->dim > 0 && p->vdim > 0 && p->n_tokens > 0, "pcs_mlstm_scan: bad sizes");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float* nm_new = p->o_raw + static_cast<long long>(p->n_tokens) * p->heads * p->vdim;  // behind the raw outputs
  const int es = p->dtype == PCS_BF16 ? 2 : 4, per = 16 / es;
  const bool aligned = p->dim % per == 0 && p->vdim % per == 0 && p->q_off % per == 0 && p->k_off % per == 0 && p->v_off % per == 0 &&
                       p->row_stride % per == 0 && reinterpret_cast<uintptr_t>(p->proj) % 16 == 0;
  if (p->impl == 0 && p->dtype == PCS_BF16 && aligned && p->dim % 16 == 0 && p->dim <= 256 && p->max_len >= pcs::kChunkMinLen) {
    // prompts in bfloat16: 64 tokens at a time on the tensor cores
    if (int rc = pcs::launch_mlstm_chunk(*p, nm_new, st)) return rc;
  } else if (p->impl != 1 && p->dim <= 256 && aligned) {
    // register-resident state: warps per block halve until the launch has two blocks per SM (or 2 warps are left)
    int W = 16;
    while (W > 1 && 8 * (W / 2) >= p->vdim) W /= 2;
    auto blocks = [&](int w) { return static_cast<long long>(p->n_seqs) * p->heads * ((p->vdim + 8 * w - 1) / (8 * w)); };
    while (W > 2 && blocks(W) < 2 * 148) W /= 2;
    if (W < 2) W = 2;
    const int DR = p->dim <= 32 ? 1 : p->dim <= 64 ? 2 : p->dim <= 128 ? 4 : 8;
    const size_t smem = static_cast<size_t>(pcs::kScanRing) * ((2 * p->dim + 8 * W) * es + 16);
    if (smem > 48 * 1024) {
#define PCS_SCAN_ATTR(DRV) PCS_DISPATCH(p->dtype, PCS_CHECK_CUDA(cudaFuncSetAttribute(pcs::mlstm_scan_reg_kernel<T, DRV>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024)))
      if (DR == 1) PCS_SCAN_ATTR(1);
      else if (DR == 2) PCS_SCAN_ATTR(2);
      else if (DR == 4) PCS_SCAN_ATTR(4);
      else PCS_SCAN_ATTR(8);
#undef PCS_SCAN_ATTR
    }
    dim3 grid(p->n_seqs, p->heads, (p->vdim + 8 * W - 1) / (8 * W));
#define PCS_SCAN_REG(DRV) PCS_DISPATCH(p->dtype, (pcs::mlstm_scan_reg_kernel<T, DRV><<<grid, 32 * W, smem, st>>>(*p, p->o_raw, nm_new, W)))
    if (DR == 1) PCS_SCAN_REG(1);
    else if (DR == 2) PCS_SCAN_REG(2);
    else if (DR == 4) PCS_SCAN_REG(4);
    else PCS_SCAN_REG(8);
#undef PCS_SCAN_REG
    PCS_CHECK_CUDA(cudaGetLastError());
  } else {
    // slice width: at most 128 columns, and small enough that the slice of S fits shared memory
    int VS = p->vdim < 128 ? p->vdim : 128;
    while (VS > 8 && static_cast<size_t>(p->dim) * VS * sizeof(float) > 160 * 1024) VS /= 2;
    int R = 512 / VS;
    if (R < 1) R = 1;
    if (R > p->dim) R = p->dim;
    const int slices = (p->vdim + VS - 1) / VS;
    const int threads = ((VS * R + 31) / 32) * 32;
    const size_t smem = (static_cast<size_t>(p->dim) * VS + 3 * p->dim + VS + static_cast<size_t>(R) * VS) * sizeof(float);
    PCS_REQUIRE(smem <= 220 * 1024, "pcs_mlstm_scan: a state of %d rows exceeds shared memory", p->dim);
    if (smem > 48 * 1024) {
      PCS_DISPATCH(p->dtype, PCS_CHECK_CUDA(cudaFuncSetAttribute(pcs::mlstm_scan_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                                220 * 1024)));
    }
    dim3 grid(p->n_seqs, p->heads, slices);
    PCS_DISPATCH(p->dtype, pcs::mlstm_scan_kernel<T><<<grid, threads, smem, st>>>(*p, p->o_raw, nm_new, VS, R));
    PCS_CHECK_CUDA(cudaGetLastError());
  }
  pcs::mlstm_commit_kernel<<<dim3(p->n_seqs, p->heads), 128, 0, st>>>(*p, nm_new);
  PCS_CHECK_CUDA(cudaGetLastError());
  dim3 grid2(p->n_tokens, p->heads);
  PCS_DISPATCH(p->dtype, pcs::mlstm_out_kernel<T><<<grid2, 256, 0, st>>>(*p, p->o_raw));
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch(3);
  return PCS_OK;
}
