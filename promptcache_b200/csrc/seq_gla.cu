// Gated linear attention over the slot pool.
//
// Per head, with a decay per key channel alpha_t = exp(ld_t) in (0, 1):
//     S_t = diag(alpha_t) S_{t-1} + k_t v_t^T          (S: dim x vdim; the decay scales the rows, which belong to key channels)
//     o_t = S_t^T q_t
// followed by o_t / rms(o_t) per head, one norm weight vector for all heads, and the gate silu(g_t).  S lives in 32-bit floats
// in the slot pool and is carried from step to step; a sequence whose slot holds no tokens yet starts from zero.  Decays,
// their logarithms and the state are 32-bit in both compute types; q, k, v and g come from the projections in the compute type.
//
// pcs_gla_decay  one block per token: z = A2 a + b per channel from the low-rank input a (32-bit sums), ld = logsigmoid(z) / tau.
// pcs_gla_scan   the token-by-token recurrence, one block per (sequence, head, slice of value columns): state in registers
//                (dim <= 256, 16-byte aligned projections) or in shared memory, then the per-head output norm with the gate.
#include "seq_common.cuh"
#include "seq_mma.cuh"

namespace pcs {

template <typename T>
__global__ void __launch_bounds__(256) gla_decay_kernel(const T* __restrict__ a, long long a_stride, const T* __restrict__ a2,
                                                        const float* __restrict__ a2_b, float* __restrict__ ld, int n_channels, int rank,
                                                        float inv_tau) {
  extern __shared__ float as[];  // the token's low-rank input
  const long long t = blockIdx.x;
  for (int r = threadIdx.x; r < rank; r += blockDim.x) as[r] = ldf(a + t * a_stride + r);
  __syncthreads();
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < n_channels; c += gridDim.y * blockDim.x) {
    const T* w = a2 + static_cast<long long>(c) * rank;
    float z = 0.f;
    for (int r = 0; r < rank; ++r) z = fmaf(ldf(w + r), as[r], z);
    z += a2_b ? a2_b[c] : 0.f;
    ld[t * n_channels + c] = logsigmoidf_(z) * inv_tau;
  }
}

// Many tokens: block = (256 channels, kDecayTokens tokens).  The block's rows of A2 sit in shared memory transposed (a thread reads
// its own channel's numbers without bank conflicts) and the tokens' low-rank inputs beside them (broadcast reads); a thread
// owns one channel and walks the tokens, so the stores of a token are contiguous over the threads.  The sum runs over r in
// increasing order as in the kernel above: both give the same bits.
constexpr int kDecayTokens = 32;
template <typename T>
__global__ void __launch_bounds__(256) gla_decay_tile_kernel(const T* __restrict__ a, long long a_stride, const T* __restrict__ a2,
                                                             const float* __restrict__ a2_b, float* __restrict__ ld, int n_tokens, int n_channels,
                                                             int rank, float inv_tau) {
  extern __shared__ float sm[];
  float* w = sm;                 // [rank][256]
  float* as = sm + rank * 256;   // [kDecayTokens][rank]
  const int c = blockIdx.x * 256 + threadIdx.x, t0 = blockIdx.y * kDecayTokens;
  const int nt = min(kDecayTokens, n_tokens - t0);
  for (int e = threadIdx.x; e < 256 * rank; e += 256) {
    const int cc = e / rank, r = e - cc * rank, ch = blockIdx.x * 256 + cc;
    w[r * 256 + cc] = ch < n_channels ? ldf(a2 + static_cast<long long>(ch) * rank + r) : 0.f;
  }
  for (int e = threadIdx.x; e < nt * rank; e += 256) {
    const int i = e / rank, r = e - i * rank;
    as[e] = ldf(a + static_cast<long long>(t0 + i) * a_stride + r);
  }
  __syncthreads();
  if (c >= n_channels) return;
  const float bias = a2_b ? a2_b[c] : 0.f;
  for (int i = 0; i < nt; ++i) {
    float z = 0.f;
    for (int r = 0; r < rank; ++r) z = fmaf(w[r * 256 + threadIdx.x], as[i * rank + r], z);
    ld[static_cast<long long>(t0 + i) * n_channels + c] = logsigmoidf_(z + bias) * inv_tau;
  }
}

// Grid (sequence, head, slice of value columns): the columns of S evolve independently given the decays, k and q.  Thread
// (r, c) owns rows r, r + R, ... of column c of the slice; threads past VS * R only take part in loads.
template <typename T>
__global__ void __launch_bounds__(1024) gla_scan_kernel(const pcs_gla_params p, int VS, int R) {
  extern __shared__ float sm[];
  const int D = p.dim, V = p.vdim, H = p.heads;
  const int v0 = blockIdx.z * VS, vs = min(VS, V - v0);
  float* S = sm;               // [D][VS]
  float* ks = S + D * VS;      // [D]
  float* qs = ks + D;          // [D]
  float* as = qs + D;          // [D] decay
  float* vsm = as + D;         // [VS]
  float* part = vsm + VS;      // [R][VS]
  const int b = blockIdx.x, head = blockIdx.y, tid = threadIdx.x, nthr = blockDim.x;
  const int slot = p.seq_slot[b], pos0 = p.seq_pos0[b], len = p.seq_len[b], off = p.seq_off[b];
  if (len <= 0) return;
  float* Sg = p.s_pool + (static_cast<long long>(slot) * H + head) * D * V;
  const bool fresh = pos0 == 0;
  for (int e = tid; e < D * vs; e += nthr) {
    const int d = e / vs, c = e - d * vs;
    S[d * VS + c] = fresh ? 0.f : Sg[d * V + v0 + c];
  }
  const int c = tid % VS, r = tid / VS;
  const bool active = r < R && c < vs;
  __syncthreads();
  for (int i = 0; i < len; ++i) {
    const long long t = off + i;
    const T* row = static_cast<const T*>(p.proj) + t * p.row_stride;
    const float* ldr = p.ld + t * (static_cast<long long>(H) * D) + head * D;
    for (int d = tid; d < D; d += nthr) {
      ks[d] = ldf(row + p.k_off + head * D + d);
      qs[d] = ldf(row + p.q_off + head * D + d) * p.q_scale;
      as[d] = expf(ldr[d]);
    }
    for (int e = tid; e < vs; e += nthr) vsm[e] = ldf(row + p.v_off + head * V + v0 + e);
    __syncthreads();
    if (active) {
      const float vv = vsm[c];
      float num = 0.f;
      for (int d = r; d < D; d += R) {
        const float sv = fmaf(as[d], S[d * VS + c], ks[d] * vv);
        S[d * VS + c] = sv;
        num = fmaf(sv, qs[d], num);
      }
      part[r * VS + c] = num;
    }
    __syncthreads();
    if (tid < vs) {
      float o = 0.f;
      for (int rr = 0; rr < R; ++rr) o += part[rr * VS + tid];
      p.o_raw[t * (static_cast<long long>(H) * V) + head * V + v0 + tid] = o;
    }
    __syncthreads();  // ks / qs / as / vsm / part are rewritten by the next token
  }
  for (int e = tid; e < D * vs; e += nthr) {
    const int d = e / vs, cc = e - d * vs;
    Sg[d * V + v0 + cc] = S[d * VS + cc];
  }
}

constexpr int kGlaRing = 24;   // shared-memory slots of tokens whose k / q / v / decays are in flight or waiting
constexpr int kGlaAhead = 16;  // tokens requested ahead of the arithmetic
constexpr int kGlaGroup = 4;   // tokens computed between two block barriers

template <int N>
__device__ __forceinline__ void ldv(const float* p, float (&o)[N]) {
#pragma unroll
  for (int i = 0; i < N; ++i) o[i] = p[i];
}
template <int N>
__device__ __forceinline__ void ldv(const __nv_bfloat16* p, float (&o)[N]) {
#pragma unroll
  for (int i = 0; i < N; ++i) o[i] = __bfloat162float(p[i]);
}

// The same recurrence with the state in REGISTERS.  A warp owns 8 value columns; lane l owns the DR = ceil(dim / 32) rows
// l*DR .. l*DR + DR - 1 of them, so a thread keeps a DR x 8 patch of S.  Per token a thread does 2 * DR * 8 fused
// multiply-adds from 3 * DR + 8 shared-memory values; the 8 column sums over the 32 lanes are one reduce-scatter butterfly.
// k, q, v (compute type) and the log decays (32-bit) of the next tokens arrive through a ring of shared-memory slots filled by
// cp.async, kGlaAhead tokens ahead of the arithmetic; kGlaGroup tokens are computed between two block barriers.  The order of
// every sum is fixed by DR alone: a token's result does not depend on how the sequence is cut into steps or on the batch.
template <typename T, int DR>
__global__ void __launch_bounds__(512) gla_scan_reg_kernel(const pcs_gla_params p, int W) {
  extern __shared__ __align__(16) unsigned char ring[];
  constexpr int ES = static_cast<int>(sizeof(T)), PER = 16 / ES;
  const int D = p.dim, V = p.vdim, H = p.heads;
  const int slot_bytes = (2 * D + 8 * W) * ES + D * 4;  // k[D] q[D] v[8W] (compute type), ld[D] (32-bit)
  const int b = blockIdx.x, head = blockIdx.y, v0 = blockIdx.z * 8 * W;
  const int tid = threadIdx.x, nthr = blockDim.x, warp = tid >> 5, lane = tid & 31;
  const int slot = p.seq_slot[b], pos0 = p.seq_pos0[b], len = p.seq_len[b], off = p.seq_off[b];
  if (len <= 0) return;
  const int c0 = v0 + warp * 8, d0 = lane * DR;
  const int ncol = max(0, min(8, V - c0));
  const T* proj = static_cast<const T*>(p.proj);
  const int ck = D / PER, cv = 8 * W / PER, cl = D / 4;
  const int n_pieces = 2 * ck + cv + cl;
  auto issue = [&](int i) {  // token i of this entry into slot i % kGlaRing
    const long long t = off + i;
    unsigned char* s = ring + (i % kGlaRing) * slot_bytes;
    const T* row = proj + t * p.row_stride;
    for (int e = tid; e < n_pieces; e += nthr) {
      if (e < ck) cp_async16(s + e * 16, row + p.k_off + head * D + e * PER);
      else if (e < 2 * ck) cp_async16(s + D * ES + (e - ck) * 16, row + p.q_off + head * D + (e - ck) * PER);
      else if (e < 2 * ck + cv) {
        const int c = e - 2 * ck, col = v0 + c * PER;
        if (col < V) cp_async16(s + 2 * D * ES + c * 16, row + p.v_off + head * V + col);
        else *reinterpret_cast<uint4*>(s + 2 * D * ES + c * 16) = make_uint4(0u, 0u, 0u, 0u);
      } else {
        const int c = e - 2 * ck - cv;
        cp_async16(s + (2 * D + 8 * W) * ES + c * 16, p.ld + t * (static_cast<long long>(H) * D) + head * D + c * 4);
      }
    }
  };
  for (int i = 0; i < kGlaAhead; ++i) {
    if (i < len) issue(i);
    cp_async_commit();
  }
  float* Sg = p.s_pool + (static_cast<long long>(slot) * H + head) * D * V;
  const bool fresh = pos0 == 0;
  float S[DR][8];
#pragma unroll
  for (int r = 0; r < DR; ++r) {
    const int d = d0 + r;
#pragma unroll
    for (int c = 0; c < 8; ++c) S[r][c] = (!fresh && d < D && c < ncol) ? Sg[static_cast<long long>(d) * V + c0 + c] : 0.f;
  }
  for (int i0 = 0; i0 < len; i0 += kGlaGroup) {
    cp_async_wait<kGlaAhead - kGlaGroup>();  // this thread's copies of tokens i0 .. i0 + 3 have landed ...
    __syncthreads();                         // ... and everybody's; the slots of the previous groups have been read by all warps
#pragma unroll
    for (int u = 0; u < kGlaGroup; ++u) {
      if (i0 + kGlaAhead + u < len) issue(i0 + kGlaAhead + u);
      cp_async_commit();
    }
#pragma unroll
    for (int u = 0; u < kGlaGroup; ++u) {
      const int i = i0 + u;
      if (i >= len) break;
      const long long t = off + i;
      const unsigned char* cur = ring + (i % kGlaRing) * slot_bytes;
      const T* kb = reinterpret_cast<const T*>(cur);
      const T* qb = kb + D;
      const T* vb = qb + D;
      const float* lb = reinterpret_cast<const float*>(cur + (2 * D + 8 * W) * ES);
      float kk[DR], qq[DR], aa[DR], vv[8];
#pragma unroll
      for (int r = 0; r < DR; ++r) {
        const bool ok = d0 + r < D;
        kk[r] = ok ? ldf(kb + d0 + r) : 0.f;
        qq[r] = ok ? ldf(qb + d0 + r) * p.q_scale : 0.f;
        aa[r] = ok ? expf(lb[d0 + r]) : 0.f;
      }
      ldv<8>(vb + warp * 8, vv);
      float num[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        float acc = 0.f;
#pragma unroll
        for (int r = 0; r < DR; ++r) {
          S[r][c] = fmaf(aa[r], S[r][c], kk[r] * vv[c]);
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
      if ((lane & 3) == 0 && col < ncol) p.o_raw[t * (static_cast<long long>(H) * V) + head * V + c0 + col] = x1;
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
}

// out[t, head, :] = o / rms(o) * norm_w * silu(g): one block of kOutThreads per (token, head); a thread's columns, their gates and
// norm weights are requested together before the reduction.
constexpr int kOutThreads = 128, kOutCols = 4;   // up to kOutThreads * kOutCols columns stay in registers
template <typename T>
__device__ __forceinline__ void gla_head_out(const float* __restrict__ o, const T* __restrict__ g, const T* __restrict__ nw, T* __restrict__ out, int V,
                                             float eps, float* red) {
  float ov[kOutCols], gv[kOutCols], wv[kOutCols];
  float ss = 0.f;
#pragma unroll
  for (int u = 0; u < kOutCols; ++u) {
    const int c = threadIdx.x + u * kOutThreads;
    ov[u] = c < V ? o[c] : 0.f;
    gv[u] = c < V ? ldf(g + c) : 0.f;
    wv[u] = c < V ? ldf(nw + c) : 0.f;
  }
#pragma unroll
  for (int u = 0; u < kOutCols; ++u) ss = fmaf(ov[u], ov[u], ss);
  for (int c = threadIdx.x + kOutCols * kOutThreads; c < V; c += kOutThreads) ss = fmaf(o[c], o[c], ss);
  ss = block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / static_cast<float>(V) + eps);
#pragma unroll
  for (int u = 0; u < kOutCols; ++u) {
    const int c = threadIdx.x + u * kOutThreads;
    if (c < V) stf(out + c, ov[u] * inv * wv[u] * (gv[u] * sigmoidf_(gv[u])));
  }
  for (int c = threadIdx.x + kOutCols * kOutThreads; c < V; c += kOutThreads) {
    const float x = ldf(g + c);
    stf(out + c, o[c] * inv * ldf(nw + c) * (x * sigmoidf_(x)));
  }
}

template <typename T>
__global__ void __launch_bounds__(kOutThreads) gla_out_kernel(const pcs_gla_params p) {
  __shared__ float red[33];
  const int V = p.vdim, H = p.heads, head = blockIdx.y;
  const long long t = blockIdx.x;
  gla_head_out<T>(p.o_raw + t * (static_cast<long long>(H) * V) + head * V, static_cast<const T*>(p.proj) + t * p.row_stride + p.g_off + head * V,
                  static_cast<const T*>(p.norm_w), static_cast<T*>(p.out) + t * (static_cast<long long>(H) * V) + head * V, V, p.eps, red);
}

// ---- the chunkwise form (prompts) -------------------------------------------------------------------------------------
// One block per (chunk, head).  q, k and the running sums of the log decays of the chunk sit in shared memory as 32-bit rows
// of dim + 1 numbers (a row per token: threads that walk the tokens at a fixed channel touch different banks).  The scores
// inside the chunk are formed pair by pair with the exact factor exp(B_i[d] - B_s[d]) <= 1 per channel, so no decay, however
// strong, overflows a factor; everything that crosses chunks is left to matrix products on exp(B_i) and exp(B_e - B_i) <= 1.
constexpr int kPrepThreads = 1024;
template <typename T>
__global__ void __launch_bounds__(kPrepThreads) gla_chunk_prep_kernel(const pcs_gla_chunk_params p) {
  extern __shared__ float sm[];
  const int D = p.dim, V = p.vdim, H = p.heads, C = p.chunk, DP = D + 1;
  float* qs = sm;              // [C][DP]
  float* ks = qs + C * DP;     // [C][DP]
  float* Bs = ks + C * DP;     // [C][DP]
  const int cn = blockIdx.x, head = blockIdx.y, tid = threadIdx.x;
  const int first = p.chunk_first[cn], n = p.chunk_len[cn];
  const T* proj = static_cast<const T*>(p.proj);
  for (int e = tid; e < C * D; e += kPrepThreads) {
    const int i = e / D, d = e - i * D;
    float qv = 0.f, kv = 0.f, lv = 0.f;
    if (i < n) {
      const T* row = proj + static_cast<long long>(first + i) * p.row_stride;
      qv = ldf(row + p.q_off + head * D + d) * p.q_scale;
      kv = ldf(row + p.k_off + head * D + d);
      lv = p.ld[static_cast<long long>(first + i) * (H * D) + head * D + d];
    }
    qs[i * DP + d] = qv;
    ks[i * DP + d] = kv;
    Bs[i * DP + d] = lv;
  }
  __syncthreads();
  for (int d = tid; d < D; d += kPrepThreads) {  // running sums over the chunk's tokens, per channel (rows past the chunk add nothing)
    float acc = 0.f;
    for (int i = 0; i < C; ++i) {
      acc += Bs[i * DP + d];
      Bs[i * DP + d] = acc;
    }
  }
  __syncthreads();
  const long long base = static_cast<long long>(cn) * H + head;
  float* qd = p.qd + base * C * D;
  float* kd = p.kd + base * C * D;
  const float* Be = Bs + (C - 1) * DP;
  for (int e = tid; e < C * D; e += kPrepThreads) {
    const int i = e / D, d = e - i * D;
    const float bi = Bs[i * DP + d];
    qd[e] = qs[i * DP + d] * expf(bi);
    kd[e] = ks[i * DP + d] * expf(Be[d] - bi);
  }
  for (int d = tid; d < D; d += kPrepThreads) p.g[base * D + d] = expf(Be[d]);
  float* vf = p.vf + base * C * V;
  for (int e = tid; e < C * V; e += kPrepThreads) {
    const int i = e / V, c = e - i * V;
    vf[e] = i < n ? ldf(proj + static_cast<long long>(first + i) * p.row_stride + p.v_off + head * V + c) : 0.f;
  }
  // scores inside the chunk.  Query rows i and C - 1 - i together have C + 1 visible keys, so the pairs are walked as C / 2 rows of
  // C + 1 places with every lane busy; lanes of a warp mostly walk the keys of one query (k and B rows in different banks, q and
  // B_i broadcast).  Pairs above the diagonal, and rows past the chunk's end, are zero.
  float* a = p.a + base * C * C;
  for (int e = tid; e < C * C; e += kPrepThreads) a[e] = 0.f;
  // bfloat16 projections: the pair factors go through the base-2 exponential unit (relative error 2^-22, far below the operands'
  // rounding), with the running sums rescaled once; float32 runs keep the library exponential
  constexpr bool kFast = sizeof(T) == 2;
  __syncthreads();
  if (kFast) {
    for (int e = tid; e < C * D; e += kPrepThreads) {
      const int i = e / D, d = e - i * D;
      Bs[i * DP + d] *= 1.4426950408889634f;
    }
  }
  __syncthreads();
  const int half = (C + 1) / 2;
  for (int e = tid; e < half * (C + 1); e += kPrepThreads) {
    const int r = e / (C + 1), j = e - r * (C + 1);
    int i, s_;
    if (j <= r) { i = r; s_ = j; } else { i = C - 1 - r; s_ = j - r - 1; }
    if (i >= n || s_ > i || (i == r && j > r)) continue;   // (an odd chunk's middle row is taken once)
    const float* qi = qs + i * DP;
    const float* bi = Bs + i * DP;
    const float* kk = ks + s_ * DP;
    const float* bs = Bs + s_ * DP;
    float a0 = 0.f, a1 = 0.f;
    int d = 0;
    for (; d + 1 < D; d += 2) {
      a0 = fmaf(qi[d] * kk[d], kFast ? ex2(bi[d] - bs[d]) : expf(bi[d] - bs[d]), a0);
      a1 = fmaf(qi[d + 1] * kk[d + 1], kFast ? ex2(bi[d + 1] - bs[d + 1]) : expf(bi[d + 1] - bs[d + 1]), a1);
    }
    if (d < D) a0 = fmaf(qi[d] * kk[d], kFast ? ex2(bi[d] - bs[d]) : expf(bi[d] - bs[d]), a0);
    a[i * C + s_] = a0 + a1;
  }
}

// One thread per VW neighbouring value columns of one state row: the entry's chunks in order.  The sums and decays of eight
// chunks are requested before the dependent chain S <- g S + u runs over them, so eight loads per thread are in flight.
template <int VW>
__global__ void __launch_bounds__(256) gla_chunk_scan_kernel(const pcs_gla_chunk_params p) {
  const int D = p.dim, V = p.vdim, H = p.heads;
  const int b = blockIdx.z, head = blockIdx.y;
  const int nchunks = p.seq_chunks[b];
  if (nchunks <= 0) return;
  const long long e = (static_cast<long long>(blockIdx.x) * 256 + threadIdx.x) * VW;
  if (e >= static_cast<long long>(D) * V) return;
  const int d = static_cast<int>(e / V);
  const int slot = p.seq_slot[b], c0 = p.seq_chunk0[b];
  float* Sg = p.s_pool + (static_cast<long long>(slot) * H + head) * D * V + e;
  float S[VW];
#pragma unroll
  for (int j = 0; j < VW; ++j) S[j] = p.seq_pos0[b] == 0 ? 0.f : Sg[j];
  const long long cstride = static_cast<long long>(H) * D * V;
  float* u0 = p.u + (static_cast<long long>(c0) * H + head) * D * V + e;
  const float* g0 = p.g + (static_cast<long long>(c0) * H + head) * D + d;
  constexpr int U = 8;
  for (int c = 0; c < nchunks; c += U) {
    float un[U][VW], gn[U];
#pragma unroll
    for (int k = 0; k < U; ++k) {
      if (c + k < nchunks) {
        gn[k] = g0[static_cast<long long>(c + k) * H * D];
        if (VW == 4) {
          const float4 v = *reinterpret_cast<const float4*>(u0 + (c + k) * cstride);
          un[k][0] = v.x; un[k][1 % VW] = v.y; un[k][2 % VW] = v.z; un[k][3 % VW] = v.w;
        } else {
          un[k][0] = u0[(c + k) * cstride];
        }
      }
    }
#pragma unroll
    for (int k = 0; k < U; ++k) {
      if (c + k < nchunks) {
        float* u = u0 + (c + k) * cstride;
        if (VW == 4) *reinterpret_cast<float4*>(u) = make_float4(S[0], S[1 % VW], S[2 % VW], S[3 % VW]);
        else u[0] = S[0];
#pragma unroll
        for (int j = 0; j < VW; ++j) S[j] = fmaf(gn[k], S[j], un[k][j]);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < VW; ++j) Sg[j] = S[j];
}

template <typename T>
__global__ void __launch_bounds__(kOutThreads) gla_chunk_out_kernel(const pcs_gla_chunk_params p) {
  __shared__ float red[33];
  const int V = p.vdim, H = p.heads, C = p.chunk, head = blockIdx.y;
  const long long t = blockIdx.x;
  const int row = p.tok_row[t];
  gla_head_out<T>(p.o + ((static_cast<long long>(row / C) * H + head) * C + row % C) * V, static_cast<const T*>(p.proj) + t * p.row_stride + p.g_off + head * V,
                  static_cast<const T*>(p.norm_w), static_cast<T*>(p.out) + t * (static_cast<long long>(H) * V) + head * V, V, p.eps, red);
}

}  // namespace pcs

PCS_API int pcs_gla_chunk_prep(const pcs_gla_chunk_params* p, void* stream) {
  PCS_REQUIRE(p, "pcs_gla_chunk_prep: null params");
  if (p->n_chunks == 0) return PCS_OK;
  PCS_REQUIRE(p->proj && p->ld && p->chunk_first && p->chunk_len && p->qd && p->kd && p->g && p->vf && p->a, "pcs_gla_chunk_prep: null tensor");
  PCS_REQUIRE(p->heads > 0 && p->heads <= 65535 && p->dim > 0 && p->vdim > 0 && p->chunk > 0, "pcs_gla_chunk_prep: bad sizes");
  const size_t smem = static_cast<size_t>(3) * p->chunk * (p->dim + 1) * sizeof(float);
  PCS_REQUIRE(smem <= 220 * 1024, "pcs_gla_chunk_prep: a chunk of %d tokens x %d channels exceeds shared memory", p->chunk, p->dim);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (smem > 48 * 1024)
    PCS_DISPATCH(p->dtype, PCS_CHECK_CUDA(cudaFuncSetAttribute(pcs::gla_chunk_prep_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024)));
  PCS_DISPATCH(p->dtype, pcs::gla_chunk_prep_kernel<T><<<dim3(p->n_chunks, p->heads), pcs::kPrepThreads, smem, st>>>(*p));
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}

PCS_API int pcs_gla_chunk_scan(const pcs_gla_chunk_params* p, void* stream) {
  PCS_REQUIRE(p, "pcs_gla_chunk_scan: null params");
  if (p->n_seqs == 0 || p->n_chunks == 0) return PCS_OK;
  PCS_REQUIRE(p->u && p->g && p->s_pool && p->seq_slot && p->seq_pos0 && p->seq_chunk0 && p->seq_chunks, "pcs_gla_chunk_scan: null tensor");
  PCS_REQUIRE(p->heads > 0 && p->heads <= 65535 && p->n_seqs <= 65535 && p->dim > 0 && p->vdim > 0, "pcs_gla_chunk_scan: bad sizes");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long elems = static_cast<long long>(p->dim) * p->vdim;
  if (p->vdim % 4 == 0 && ((reinterpret_cast<uintptr_t>(p->u) | reinterpret_cast<uintptr_t>(p->s_pool)) & 15) == 0)
    pcs::gla_chunk_scan_kernel<4><<<dim3(static_cast<unsigned>((elems / 4 + 255) / 256), p->heads, p->n_seqs), 256, 0, st>>>(*p);
  else
    pcs::gla_chunk_scan_kernel<1><<<dim3(static_cast<unsigned>((elems + 255) / 256), p->heads, p->n_seqs), 256, 0, st>>>(*p);
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}

PCS_API int pcs_gla_chunk_out(const pcs_gla_chunk_params* p, void* stream) {
  PCS_REQUIRE(p, "pcs_gla_chunk_out: null params");
  if (p->n_tokens == 0) return PCS_OK;
  PCS_REQUIRE(p->proj && p->o && p->tok_row && p->norm_w && p->out && p->chunk > 0 && p->heads > 0 && p->vdim > 0, "pcs_gla_chunk_out: bad arguments");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  PCS_DISPATCH(p->dtype, pcs::gla_chunk_out_kernel<T><<<dim3(p->n_tokens, p->heads), pcs::kOutThreads, 0, st>>>(*p));
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}

PCS_API int pcs_gla_decay(const void* a, int64_t a_stride, const void* a2, const float* a2_b, float* ld, int n_tokens, int n_channels, int rank,
                          float tau, int dtype, void* stream) {
  if (n_tokens == 0) return PCS_OK;
  PCS_REQUIRE(a && a2 && ld && n_channels > 0 && rank > 0 && rank <= 8192 && tau > 0.f, "pcs_gla_decay: bad arguments");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t tile_smem = static_cast<size_t>(rank) * (256 + pcs::kDecayTokens) * sizeof(float);
  if (n_tokens >= 2 * pcs::kDecayTokens && tile_smem <= 48 * 1024) {
    dim3 grid((n_channels + 255) / 256, (n_tokens + pcs::kDecayTokens - 1) / pcs::kDecayTokens);
    PCS_DISPATCH(dtype, pcs::gla_decay_tile_kernel<T><<<grid, 256, tile_smem, st>>>(static_cast<const T*>(a), a_stride, static_cast<const T*>(a2), a2_b, ld,
                                                                                   n_tokens, n_channels, rank, 1.f / tau));
  } else
  PCS_DISPATCH(dtype, pcs::gla_decay_kernel<T><<<dim3(n_tokens, (n_channels + 255) / 256 > 64 ? 64 : (n_channels + 255) / 256), 256, rank * sizeof(float), st>>>(static_cast<const T*>(a), a_stride, static_cast<const T*>(a2),
                                                                                           a2_b, ld, n_channels, rank, 1.f / tau));
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}

PCS_API int pcs_gla_scan(const pcs_gla_params* p, void* stream) {
  PCS_REQUIRE(p, "pcs_gla_scan: null params");
  if (p->n_seqs == 0 || p->n_tokens == 0) return PCS_OK;
  PCS_REQUIRE(p->proj && p->ld && p->norm_w && p->out && p->s_pool && p->seq_slot && p->seq_pos0 && p->seq_len && p->seq_off && p->o_raw,
              "pcs_gla_scan: null tensor");
  PCS_REQUIRE(p->heads > 0 && p->heads <= 65535 && p->dim > 0 && p->vdim > 0 && p->n_tokens > 0, "pcs_gla_scan: bad sizes");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int es = p->dtype == PCS_BF16 ? 2 : 4, per = 16 / es;
  const bool aligned = p->dim % per == 0 && p->dim % 4 == 0 && p->vdim % per == 0 && p->q_off % per == 0 && p->k_off % per == 0 && p->v_off % per == 0 &&
                       p->row_stride % per == 0 && reinterpret_cast<uintptr_t>(p->proj) % 16 == 0 && reinterpret_cast<uintptr_t>(p->ld) % 16 == 0;
  if (p->impl != 1 && p->dim <= 256 && aligned) {
    // register-resident state: warps per block halve until the launch has two blocks per SM (or 2 warps are left)
    int W = 16;
    while (W > 1 && 8 * (W / 2) >= p->vdim) W /= 2;
    auto blocks = [&](int w) { return static_cast<long long>(p->n_seqs) * p->heads * ((p->vdim + 8 * w - 1) / (8 * w)); };
    while (W > 2 && blocks(W) < 2 * 148) W /= 2;
    if (W < 2) W = 2;
    const int DR = p->dim <= 32 ? 1 : p->dim <= 64 ? 2 : p->dim <= 128 ? 4 : 8;
    const size_t smem = static_cast<size_t>(pcs::kGlaRing) * ((2 * p->dim + 8 * W) * es + p->dim * 4);
    if (smem > 48 * 1024) {
#define PCS_GLA_ATTR(DRV) PCS_DISPATCH(p->dtype, PCS_CHECK_CUDA(cudaFuncSetAttribute(pcs::gla_scan_reg_kernel<T, DRV>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024)))
      if (DR == 1) PCS_GLA_ATTR(1);
      else if (DR == 2) PCS_GLA_ATTR(2);
      else if (DR == 4) PCS_GLA_ATTR(4);
      else PCS_GLA_ATTR(8);
#undef PCS_GLA_ATTR
    }
    dim3 grid(p->n_seqs, p->heads, (p->vdim + 8 * W - 1) / (8 * W));
#define PCS_GLA_REG(DRV) PCS_DISPATCH(p->dtype, (pcs::gla_scan_reg_kernel<T, DRV><<<grid, 32 * W, smem, st>>>(*p, W)))
    if (DR == 1) PCS_GLA_REG(1);
    else if (DR == 2) PCS_GLA_REG(2);
    else if (DR == 4) PCS_GLA_REG(4);
    else PCS_GLA_REG(8);
#undef PCS_GLA_REG
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
    PCS_REQUIRE(smem <= 220 * 1024, "pcs_gla_scan: a state of %d rows exceeds shared memory", p->dim);
    if (smem > 48 * 1024)
      PCS_DISPATCH(p->dtype, PCS_CHECK_CUDA(cudaFuncSetAttribute(pcs::gla_scan_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024)));
    dim3 grid(p->n_seqs, p->heads, slices);
    PCS_DISPATCH(p->dtype, pcs::gla_scan_kernel<T><<<grid, threads, smem, st>>>(*p, VS, R));
    PCS_CHECK_CUDA(cudaGetLastError());
  }
  PCS_DISPATCH(p->dtype, pcs::gla_out_kernel<T><<<dim3(p->n_tokens, p->heads), pcs::kOutThreads, 0, st>>>(*p));
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch(2);
  return PCS_OK;
}
