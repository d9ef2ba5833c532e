// Attention over the slot pool: query / key preparation with append, and the plain attention kernel.
//
// pcs_qk_prep   one block per token: RMS norm over the WHOLE query projection (all heads at once) and over the whole key
//               projection, query temperature from the token's position, value mixing with the rows an earlier layer
//               appended for the same token, K / V rows written behind the slot's cached rows.
// pcs_attn      one block per (token, head, split of the keys): keys in tiles of 128, one key per thread for the score, online softmax in
//               32-bit, then one value column per thread.  Scores, weights and the accumulator are 32-bit in both types.
//               A sink is one more term exp(0 - m) of the denominator that has no value: the running maximum starts at 0
//               and the running sum at 1 instead of (-inf, 0).  A score may be capped (cap * tanh(score / cap)), and the keys may
//               be limited to a sliding window plus the first keys of the sequence: a query then walks a dense list of its
//               visible keys, so its work is bounded by window + keep_first whatever the sequence's length.
#include "seq_common.cuh"

namespace pcs {

template <typename T>
__global__ void __launch_bounds__(256) qk_prep_kernel(const pcs_qkprep_params p) {
  __shared__ float red[33];
  const int t = blockIdx.x;
  const int b = p.tok_seq[t], pos = p.tok_pos[t], slot = p.seq_slot[b];
  const T* row = static_cast<const T*>(p.qkv) + static_cast<long long>(t) * p.row_stride;
  const int nq = p.n_heads * p.dim, nk = p.n_kv_heads * p.dim, nv = p.n_kv_heads * p.vdim;
  // query
  {
    const T* q = row + p.q_off;
    float inv = 1.f;
    if (p.q_norm_w) {
      float ss = 0.f;
      for (int i = threadIdx.x; i < nq; i += blockDim.x) { const float v = ldf(q + i); ss = fmaf(v, v, ss); }
      ss = block_sum(ss, red);
      inv = 1.f / sqrtf(ss / static_cast<float>(nq) + p.eps);
    }
    float temp = 1.f;
    if (p.temp_every > 0) temp = 1.f + p.temp_coef * logf(static_cast<float>((pos + 1) / p.temp_every) + 1.f);
    const T* w = static_cast<const T*>(p.q_norm_w);
    T* qo = static_cast<T*>(p.q_out) + static_cast<long long>(t) * nq;
    for (int i = threadIdx.x; i < nq; i += blockDim.x) {
      float v = ldf(q + i) * inv;
      if (w) v *= ldf(w + i);
      stf(qo + i, v * temp);
    }
  }
  // key
  {
    const T* k = row + p.k_off;
    float inv = 1.f;
    if (p.k_norm_w) {
      float ss = 0.f;
      for (int i = threadIdx.x; i < nk; i += blockDim.x) { const float v = ldf(k + i); ss = fmaf(v, v, ss); }
      ss = block_sum(ss, red);
      inv = 1.f / sqrtf(ss / static_cast<float>(nk) + p.eps);
    }
    const T* w = static_cast<const T*>(p.k_norm_w);
    T* kp = static_cast<T*>(p.k_pool) + static_cast<long long>(slot) * p.n_kv_heads * p.cap * p.dim;
    for (int i = threadIdx.x; i < nk; i += blockDim.x) {
      float v = ldf(k + i) * inv;
      if (w) v *= ldf(w + i);
      const int g = i / p.dim, d = i - g * p.dim;
      stf(kp + (static_cast<long long>(g) * p.cap + pos) * p.dim + d, v);
    }
  }
  // value
  {
    const T* v = row + p.v_off;
    const long long base = static_cast<long long>(slot) * p.n_kv_heads * p.cap * p.vdim;
    T* vp = static_cast<T*>(p.v_pool) + base;
    const T* vf = p.v_first_pool ? static_cast<const T*>(p.v_first_pool) + base : nullptr;
    const float lam = vf ? ldf(static_cast<const T*>(p.v_lambda)) : 0.f;
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
      const int g = i / p.vdim, d = i - g * p.vdim;
      const long long o = (static_cast<long long>(g) * p.cap + pos) * p.vdim + d;
      float x = ldf(v + i);
      if (vf) x = (1.f - lam) * x + lam * ldf(vf + o);
      stf(vp + o, x);
    }
  }
}

// The same with 16-byte pieces (head sizes, offsets, the row stride and every pointer are multiples of a piece): the sums of
// squares of q and k share one reduction, a piece of a key or value row never straddles two heads.
template <typename T>
__global__ void __launch_bounds__(256) qk_prep_vec_kernel(const pcs_qkprep_params p) {
  constexpr int N = Vec<T>::n;
  __shared__ float red[2][9];
  const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int b = p.tok_seq[t], pos = p.tok_pos[t], slot = p.seq_slot[b];
  const T* row = static_cast<const T*>(p.qkv) + static_cast<long long>(t) * p.row_stride;
  const int nq = p.n_heads * p.dim, nk = p.n_kv_heads * p.dim, nv = p.n_kv_heads * p.vdim;
  const T* q = row + p.q_off;
  const T* k = row + p.k_off;
  float sq = 0.f, sk = 0.f;
  if (p.q_norm_w)
    for (int i = tid * N; i < nq; i += 256 * N) {
      float v[N];
      ld16(q + i, v);
#pragma unroll
      for (int e = 0; e < N; ++e) sq = fmaf(v[e], v[e], sq);
    }
  if (p.k_norm_w)
    for (int i = tid * N; i < nk; i += 256 * N) {
      float v[N];
      ld16(k + i, v);
#pragma unroll
      for (int e = 0; e < N; ++e) sk = fmaf(v[e], v[e], sk);
    }
  sq = warp_sum(sq);
  sk = warp_sum(sk);
  if (lane == 0) { red[0][warp] = sq; red[1][warp] = sk; }
  __syncthreads();
  if (warp == 0) {
    float a = lane < 8 ? red[0][lane] : 0.f, c = lane < 8 ? red[1][lane] : 0.f;
    a = warp_sum(a);
    c = warp_sum(c);
    if (lane == 0) { red[0][8] = a; red[1][8] = c; }
  }
  __syncthreads();
  const float inv_q = p.q_norm_w ? 1.f / sqrtf(red[0][8] / static_cast<float>(nq) + p.eps) : 1.f;
  const float inv_k = p.k_norm_w ? 1.f / sqrtf(red[1][8] / static_cast<float>(nk) + p.eps) : 1.f;
  float temp = 1.f;
  if (p.temp_every > 0) temp = 1.f + p.temp_coef * logf(static_cast<float>((pos + 1) / p.temp_every) + 1.f);
  {
    const T* w = static_cast<const T*>(p.q_norm_w);
    T* qo = static_cast<T*>(p.q_out) + static_cast<long long>(t) * nq;
    for (int i = tid * N; i < nq; i += 256 * N) {
      float v[N], wv[N];
      ld16(q + i, v);
      if (w) ld16(w + i, wv);
#pragma unroll
      for (int e = 0; e < N; ++e) {
        float x = v[e] * inv_q;
        if (w) x *= wv[e];
        v[e] = x * temp;
      }
      st16(qo + i, v);
    }
  }
  {
    const T* w = static_cast<const T*>(p.k_norm_w);
    T* kp = static_cast<T*>(p.k_pool) + static_cast<long long>(slot) * p.n_kv_heads * p.cap * p.dim;
    for (int i = tid * N; i < nk; i += 256 * N) {
      float v[N], wv[N];
      ld16(k + i, v);
      if (w) ld16(w + i, wv);
#pragma unroll
      for (int e = 0; e < N; ++e) {
        float x = v[e] * inv_k;
        if (w) x *= wv[e];
        v[e] = x;
      }
      const int g = i / p.dim, d = i - g * p.dim;
      st16(kp + (static_cast<long long>(g) * p.cap + pos) * p.dim + d, v);
    }
  }
  {
    const T* v = row + p.v_off;
    const long long base = static_cast<long long>(slot) * p.n_kv_heads * p.cap * p.vdim;
    T* vp = static_cast<T*>(p.v_pool) + base;
    const T* vf = p.v_first_pool ? static_cast<const T*>(p.v_first_pool) + base : nullptr;
    const float lam = vf ? ldf(static_cast<const T*>(p.v_lambda)) : 0.f;
    for (int i = tid * N; i < nv; i += 256 * N) {
      const int g = i / p.vdim, d = i - g * p.vdim;
      const long long o = (static_cast<long long>(g) * p.cap + pos) * p.vdim + d;
      float x[N];
      ld16(v + i, x);
      if (vf) {
        float f[N];
        ld16(vf + o, f);
#pragma unroll
        for (int e = 0; e < N; ++e) x[e] = (1.f - lam) * x[e] + lam * f[e];
      }
      st16(vp + o, x);
    }
  }
}

constexpr int kAttnThreads = 128;
constexpr int kAttnMaxVPT = 4;  // value columns per thread: vdim <= 512

// The keys a query at position `pos` sees, as one dense index range: with a window, the kept first keys [0, n_first) and
// then the window [lo, pos]; without one (or when the two touch), all of [0, pos].
struct VisibleKeys {
  int n_first, lo, count;
  __device__ __forceinline__ VisibleKeys(int pos, int window, int keep_first) {
    lo = window > 0 ? max(0, pos - window + 1) : 0;
    n_first = min(max(keep_first, 0), lo);
    count = n_first + (pos + 1 - lo);
  }
  __device__ __forceinline__ int key(int v) const { return v < n_first ? v : lo + (v - n_first); }
};

template <typename T>
__global__ void __launch_bounds__(kAttnThreads) attn_plain_kernel(const pcs_attn_params p) {
  extern __shared__ float sm[];  // q[dim], w[128]
  __shared__ float red[33];
  float* qs = sm;
  float* ws = sm + p.dim;
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int b = p.tok_seq[t], pos = p.tok_pos[t], slot = p.pool_slot ? p.pool_slot[b] : p.seq_slot[b];
  const int g = h / (p.n_heads / p.n_kv_heads);
  const int D = p.dim, V = p.vdim;
  const long long VS = p.v_row_stride > 0 ? p.v_row_stride : V;   // elements from one key's value row to the next
  const T* q = static_cast<const T*>(p.q) + (static_cast<long long>(t) * p.n_heads + h) * D;
  const T* K = static_cast<const T*>(p.k_pool) + (static_cast<long long>(slot) * p.n_kv_heads + g) * p.cap * D;
  const T* Vp = static_cast<const T*>(p.v_pool) + (static_cast<long long>(slot) * p.n_kv_heads + g) * p.cap * VS;
  for (int i = tid; i < D; i += kAttnThreads) qs[i] = ldf(q + i);
  const float r1 = p.bias_r1 ? p.bias_r1[h] : 0.f, r2 = p.bias_r1 ? p.bias_r2[h] : 0.f;
  // keys are cut into gridDim.z splits of whole tiles; the sink belongs to split 0
  const VisibleKeys vis(pos, p.window, p.keep_first);
  const int n_keys = vis.count, S = gridDim.z, sp = blockIdx.z;
  const int chunk = ((n_keys + S - 1) / S + kAttnThreads - 1) / kAttnThreads * kAttnThreads;
  const int k_begin = sp * chunk, k_end = min(n_keys, k_begin + chunk);
  const bool sink_here = p.sink && sp == 0;
  float m = sink_here ? (p.sink_logit ? p.sink_logit[h] : 0.f) : -INFINITY, l = sink_here ? 1.f : 0.f;
  float acc[kAttnMaxVPT] = {0.f, 0.f, 0.f, 0.f};
  const bool vec = (D % Vec<T>::n) == 0;
  __syncthreads();
  for (int j0 = k_begin; j0 < k_end; j0 += kAttnThreads) {
    const int j = vis.key(j0 + tid);
    float s = -INFINITY;
    if (j0 + tid < k_end) {
      const T* kr = K + static_cast<long long>(j) * D;
      float a = 0.f;
      if (vec) {
        for (int d = 0; d < D; d += Vec<T>::n) {
          float kv[Vec<T>::n];
          ld16(kr + d, kv);
#pragma unroll
          for (int e = 0; e < Vec<T>::n; ++e) a = fmaf(qs[d + e], kv[e], a);
        }
      } else {
        for (int d = 0; d < D; ++d) a = fmaf(qs[d], ldf(kr + d), a);
      }
      s = a * p.scale;
      if (p.softcap > 0.f) s = p.softcap * tanhf(s / p.softcap);
      if (p.bias_r1) s -= r1 * log1pf(r2 * static_cast<float>(pos - j));
    }
    const float tmax = block_max(s, red);
    const float m_new = fmaxf(m, tmax);
    const float f = (m == -INFINITY) ? 0.f : expf(m - m_new);
    const float w = (j0 + tid < k_end) ? expf(s - m_new) : 0.f;
    ws[tid] = w;
    const float tsum = block_sum(w, red);  // its barriers also publish ws
    l = l * f + tsum;
    m = m_new;
    const int nt = min(kAttnThreads, k_end - j0);
#pragma unroll
    for (int u = 0; u < kAttnMaxVPT; ++u) {
      const int c = tid + u * kAttnThreads;
      if (c < V) {
        float a = acc[u] * f;
        for (int jj = 0; jj < nt; ++jj) a = fmaf(ws[jj], ldf(Vp + static_cast<long long>(vis.key(j0 + jj)) * VS + c), a);
        acc[u] = a;
      }
    }
    __syncthreads();  // ws is rewritten by the next tile
  }
  if (S > 1) {  // partial (m, l, acc) of this split; attn_combine_kernel merges them
    float* part = p.workspace + ((static_cast<long long>(t) * p.n_heads + h) * S + sp) * (V + 2);
    if (tid == 0) { part[0] = m; part[1] = l; }
#pragma unroll
    for (int u = 0; u < kAttnMaxVPT; ++u) {
      const int c = tid + u * kAttnThreads;
      if (c < V) part[2 + c] = acc[u];
    }
    return;
  }
  T* o = static_cast<T*>(p.out) + (static_cast<long long>(t) * p.n_heads + h) * V;
  const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
  for (int u = 0; u < kAttnMaxVPT; ++u) {
    const int c = tid + u * kAttnThreads;
    if (c < V) stf(o + c, acc[u] * inv);
  }
}

// Few tokens over many keys (decoding).  One block per (token, head, split of the keys), tiles of 128 keys:
//   scores    one key per thread, its row read in 16-byte pieces with several loads in flight;
//   maximum   one barrier (warp maxima through shared memory), weights w = exp(s - m) into shared memory, one more barrier;
//   values    a thread owns one 16-byte piece of the value row and every R-th key of the tile (R = 128 / pieces per row),
//             so a warp reads whole rows; the denominator is summed the same way.  The R partial sums meet once, at the end.
// Needs dim and vdim to be multiples of a 16-byte piece and at most 128 pieces per value row; other shapes take the plain kernel.
template <typename T>
__global__ void __launch_bounds__(kAttnThreads) attn_decode_kernel(const pcs_attn_params p) {
  constexpr int N = Vec<T>::n;
  extern __shared__ float sm[];  // q[dim], w[128], partial sums [128 * N]
  __shared__ float red[kAttnThreads / 32];
  __shared__ float lred[kAttnThreads];
  float* qs = sm;
  float* ws = sm + p.dim;
  float* part_s = ws + kAttnThreads;
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int b = p.tok_seq[t], pos = p.tok_pos[t], slot = p.pool_slot ? p.pool_slot[b] : p.seq_slot[b];
  const int g = h / (p.n_heads / p.n_kv_heads);
  const int D = p.dim, V = p.vdim;
  const long long VS = p.v_row_stride > 0 ? p.v_row_stride : V;   // elements from one key's value row to the next
  const T* q = static_cast<const T*>(p.q) + (static_cast<long long>(t) * p.n_heads + h) * D;
  const T* K = static_cast<const T*>(p.k_pool) + (static_cast<long long>(slot) * p.n_kv_heads + g) * p.cap * D;
  const T* Vp = static_cast<const T*>(p.v_pool) + (static_cast<long long>(slot) * p.n_kv_heads + g) * p.cap * VS;
  for (int i = tid; i < D; i += kAttnThreads) qs[i] = ldf(q + i);
  const float r1 = p.bias_r1 ? p.bias_r1[h] : 0.f, r2 = p.bias_r1 ? p.bias_r2[h] : 0.f;
  const VisibleKeys vis(pos, p.window, p.keep_first);
  const int n_keys = vis.count, S = gridDim.z, sp = blockIdx.z;
  const int chunk = ((n_keys + S - 1) / S + kAttnThreads - 1) / kAttnThreads * kAttnThreads;
  const int k_begin = sp * chunk, k_end = min(n_keys, k_begin + chunk);
  const bool sink_here = p.sink && sp == 0;
  const int CH = V / N, R = kAttnThreads / CH;  // pieces per value row, keys handled side by side
  const int c = tid % CH, r = tid / CH;
  const bool active = r < R;
  float m = sink_here ? (p.sink_logit ? p.sink_logit[h] : 0.f) : -INFINITY;
  float lsum = (sink_here && tid == 0) ? 1.f : 0.f;
  float acc[N];
#pragma unroll
  for (int e = 0; e < N; ++e) acc[e] = 0.f;
  __syncthreads();
  for (int j0 = k_begin; j0 < k_end; j0 += kAttnThreads) {
    const int j = vis.key(j0 + tid);
    float s = -INFINITY;
    if (j0 + tid < k_end) {
      const T* kr = K + static_cast<long long>(j) * D;
      float a0 = 0.f, a1 = 0.f;
      int d = 0;
      for (; d + 4 * N <= D; d += 4 * N) {
        float k0[N], k1[N], k2[N], k3[N];
        ld16(kr + d, k0); ld16(kr + d + N, k1); ld16(kr + d + 2 * N, k2); ld16(kr + d + 3 * N, k3);
#pragma unroll
        for (int e = 0; e < N; ++e) {
          a0 = fmaf(qs[d + e], k0[e], a0);
          a1 = fmaf(qs[d + N + e], k1[e], a1);
        }
#pragma unroll
        for (int e = 0; e < N; ++e) {
          a0 = fmaf(qs[d + 2 * N + e], k2[e], a0);
          a1 = fmaf(qs[d + 3 * N + e], k3[e], a1);
        }
      }
      for (; d < D; d += N) {
        float k0[N];
        ld16(kr + d, k0);
#pragma unroll
        for (int e = 0; e < N; ++e) a0 = fmaf(qs[d + e], k0[e], a0);
      }
      s = (a0 + a1) * p.scale;
      if (p.softcap > 0.f) s = p.softcap * tanhf(s / p.softcap);
      if (p.bias_r1) s -= r1 * log1pf(r2 * static_cast<float>(pos - j));
    }
    const float wm = warp_max(s);
    if ((tid & 31) == 0) red[tid >> 5] = wm;
    __syncthreads();
    float tmax = red[0];
#pragma unroll
    for (int i = 1; i < kAttnThreads / 32; ++i) tmax = fmaxf(tmax, red[i]);
    const float m_new = fmaxf(m, tmax);  // finite: a tile has at least one key
    const float f = (m == -INFINITY) ? 0.f : expf(m - m_new);
    m = m_new;
    ws[tid] = (j0 + tid < k_end) ? expf(s - m_new) : 0.f;
    __syncthreads();
    if (active) {
      const int nt = min(kAttnThreads, k_end - j0);
      lsum *= f;
#pragma unroll
      for (int e = 0; e < N; ++e) acc[e] *= f;
      const T* vr = Vp + c * N;
      int jj = r;
      for (; jj + 3 * R < nt; jj += 4 * R) {
        float v0[N], v1[N], v2[N], v3[N];
        ld16(vr + static_cast<long long>(vis.key(j0 + jj)) * VS, v0);
        ld16(vr + static_cast<long long>(vis.key(j0 + jj + R)) * VS, v1);
        ld16(vr + static_cast<long long>(vis.key(j0 + jj + 2 * R)) * VS, v2);
        ld16(vr + static_cast<long long>(vis.key(j0 + jj + 3 * R)) * VS, v3);
        const float w0 = ws[jj], w1 = ws[jj + R], w2 = ws[jj + 2 * R], w3 = ws[jj + 3 * R];
#pragma unroll
        for (int e = 0; e < N; ++e) acc[e] = fmaf(w3, v3[e], fmaf(w2, v2[e], fmaf(w1, v1[e], fmaf(w0, v0[e], acc[e]))));
        lsum += (w0 + w1) + (w2 + w3);
      }
      for (; jj < nt; jj += R) {
        float v0[N];
        ld16(vr + static_cast<long long>(vis.key(j0 + jj)) * VS, v0);
        const float w0 = ws[jj];
#pragma unroll
        for (int e = 0; e < N; ++e) acc[e] = fmaf(w0, v0[e], acc[e]);
        lsum += w0;
      }
    }
    // the next tile writes `red` after this tile's second barrier and `ws` after its own first one: no barrier here
  }
  // the R partial sums of every column, and of the denominator (one per key group: the threads of piece 0)
  if (active) {
#pragma unroll
    for (int e = 0; e < N; ++e) part_s[r * V + c * N + e] = acc[e];
  }
  lred[tid] = (active && c == 0) ? lsum : 0.f;
  __syncthreads();
  float l = 0.f;
  for (int i = 0; i < kAttnThreads; ++i) l += lred[i];
  float* part = (S > 1) ? p.workspace + ((static_cast<long long>(t) * p.n_heads + h) * S + sp) * (V + 2) : nullptr;
  if (part && tid == 0) { part[0] = m; part[1] = l; }
  T* o = static_cast<T*>(p.out) + (static_cast<long long>(t) * p.n_heads + h) * V;
  const float inv = l > 0.f ? 1.f / l : 0.f;
  for (int col = tid; col < V; col += kAttnThreads) {
    float a = 0.f;
    for (int rr = 0; rr < R; ++rr) a += part_s[rr * V + col];
    if (part) part[2 + col] = a;
    else stf(o + col, a * inv);
  }
}

constexpr int kAttnMaxSplits = 64;

// Merge of the splits' partial results.  The splits' maxima and sums are read by one thread each, the common maximum, the total
// and every split's factor exp(m_s - M) are formed once in shared memory, and the columns then need independent loads only.
template <typename T>
__global__ void __launch_bounds__(kAttnThreads) attn_combine_kernel(const pcs_attn_params p, int S) {
  __shared__ float ms[kAttnMaxSplits], ls[kAttnMaxSplits], fs[kAttnMaxSplits];
  __shared__ float inv_s;
  const int t = blockIdx.x, h = blockIdx.y, V = p.vdim;
  const float* part = p.workspace + (static_cast<long long>(t) * p.n_heads + h) * S * (V + 2);
  if (threadIdx.x < S) {
    ms[threadIdx.x] = part[threadIdx.x * (V + 2)];
    ls[threadIdx.x] = part[threadIdx.x * (V + 2) + 1];
  }
  __syncthreads();
  if (threadIdx.x == 0) {  // the same order of sums as ever: s = 0, 1, ...
    float M = -INFINITY;
    for (int s = 0; s < S; ++s) M = fmaxf(M, ms[s]);
    float L = 0.f;
    for (int s = 0; s < S; ++s) {
      const float f = ms[s] != -INFINITY ? expf(ms[s] - M) : 0.f;
      fs[s] = f;
      if (ms[s] != -INFINITY) L += ls[s] * f;
    }
    inv_s = L > 0.f ? 1.f / L : 0.f;
  }
  __syncthreads();
  const float inv = inv_s;
  T* o = static_cast<T*>(p.out) + (static_cast<long long>(t) * p.n_heads + h) * V;
  // a block takes every gridDim.z-th group of 128 columns; a column's S values are requested together, then summed in order
  for (int c = blockIdx.z * blockDim.x + threadIdx.x; c < V; c += gridDim.z * blockDim.x) {
    float v[kAttnMaxSplits];
#pragma unroll
    for (int s = 0; s < kAttnMaxSplits; ++s) v[s] = s < S ? part[s * (V + 2) + 2 + c] : 0.f;
    float a = 0.f;
#pragma unroll
    for (int s = 0; s < kAttnMaxSplits; ++s)
      if (s < S) a = fmaf(v[s], fs[s], a);
    a *= inv;
    if (p.out_gate) a *= sigmoidf_(ldf(static_cast<const T*>(p.out_gate) + static_cast<long long>(t) * p.out_gate_stride + h * V + c));
    stf(o + c, a);
  }
}



}  // namespace pcs

PCS_API int64_t pcs_attn_workspace_floats(int n_tokens, int n_heads, int vdim) {
  if (n_tokens <= 0 || n_heads <= 0 || vdim <= 0) return 0;
  return static_cast<int64_t>(n_tokens) * n_heads * pcs::kAttnMaxSplits * (vdim + 2);
}

PCS_API int pcs_qk_prep(const pcs_qkprep_params* p, void* stream) {
  PCS_REQUIRE(p, "pcs_qk_prep: null params");
  if (p->n_tokens == 0) return PCS_OK;
  PCS_REQUIRE(p->qkv && p->q_out && p->k_pool && p->v_pool && p->tok_seq && p->tok_pos && p->seq_slot, "pcs_qk_prep: null tensor");
  PCS_REQUIRE(p->n_heads > 0 && p->n_kv_heads > 0 && p->n_heads % p->n_kv_heads == 0 && p->dim > 0 && p->vdim > 0 && p->cap > 0,
              "pcs_qk_prep: bad sizes H=%d Hkv=%d dim=%d vdim=%d cap=%d", p->n_heads, p->n_kv_heads, p->dim, p->vdim, p->cap);
  PCS_REQUIRE(p->v_first_pool == nullptr || p->v_lambda != nullptr, "pcs_qk_prep: value mixing needs lambda");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int piece = p->dtype == PCS_BF16 ? 8 : 4;
  auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  const bool vec = p->dim % piece == 0 && p->vdim % piece == 0 && p->q_off % piece == 0 && p->k_off % piece == 0 && p->v_off % piece == 0 &&
                   p->row_stride % piece == 0 && al(p->qkv) && al(p->q_out) && al(p->k_pool) && al(p->v_pool) && al(p->q_norm_w) &&
                   al(p->k_norm_w) && al(p->v_first_pool);
  if (vec) PCS_DISPATCH(p->dtype, pcs::qk_prep_vec_kernel<T><<<p->n_tokens, 256, 0, st>>>(*p));
  else PCS_DISPATCH(p->dtype, pcs::qk_prep_kernel<T><<<p->n_tokens, 256, 0, st>>>(*p));
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}

namespace pcs {
int launch_attn_tc(const pcs_attn_params& p, cudaStream_t st, bool* handled);
int launch_attn_latent(const pcs_attn_params& p, cudaStream_t st, int* splits_out);
int launch_attn_talk(const pcs_attn_params& p, cudaStream_t st, int* splits_out);
}

PCS_API int pcs_attn(const pcs_attn_params* p, void* stream) {
  PCS_REQUIRE(p, "pcs_attn: null params");
  if (p->n_tokens == 0) return PCS_OK;
  PCS_REQUIRE(p->q && p->k_pool && p->v_pool && p->out && p->tok_seq && p->tok_pos && p->seq_slot, "pcs_attn: null tensor");
  PCS_REQUIRE(p->n_heads > 0 && p->n_kv_heads > 0 && p->n_heads % p->n_kv_heads == 0 && p->dim > 0 && p->vdim > 0 && p->cap > 0,
              "pcs_attn: bad sizes H=%d Hkv=%d dim=%d vdim=%d cap=%d", p->n_heads, p->n_kv_heads, p->dim, p->vdim, p->cap);
  PCS_REQUIRE(p->vdim <= pcs::kAttnThreads * pcs::kAttnMaxVPT, "pcs_attn: vdim %d exceeds %d", p->vdim,
              pcs::kAttnThreads * pcs::kAttnMaxVPT);
  PCS_REQUIRE(p->n_heads <= 65535, "pcs_attn: too many heads");
  PCS_REQUIRE((p->bias_r1 == nullptr) == (p->bias_r2 == nullptr), "pcs_attn: the distance bias needs both r1 and r2");
  PCS_REQUIRE(p->v_row_stride == 0 || p->v_row_stride >= p->vdim, "pcs_attn: the value row stride %d is below vdim %d", p->v_row_stride, p->vdim);
  PCS_REQUIRE(p->out_gate == nullptr || p->talk != nullptr, "pcs_attn: the element-wise output gate comes with mixed head scores only");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (p->talk) {  // scores mixed across heads: kernels of their own (a block needs all heads of a pair), the same split merge
    int talk_splits = 1;
    if (int rc = pcs::launch_attn_talk(*p, st, &talk_splits)) return rc;
    if (talk_splits > 1) {
      PCS_DISPATCH(p->dtype, pcs::attn_combine_kernel<T><<<dim3(p->n_tokens, p->n_heads, (p->vdim + pcs::kAttnThreads - 1) / pcs::kAttnThreads), pcs::kAttnThreads, 0, st>>>(*p, talk_splits));
      PCS_CHECK_CUDA(cudaGetLastError());
      pcs::count_launch();
    }
    return PCS_OK;
  }
  if (p->impl == 0) {  // (impl 2: the plain kernels with the split of the keys, never a tensor-core kernel)
    bool handled = false;
    if (int rc = pcs::launch_attn_tc(*p, st, &handled)) return rc;
    if (handled) return PCS_OK;
    int latent_splits = 0;   // few tokens over rows that all heads share: the tensor-core kernel, then the merge of its partial results
    if (p->max_len <= 4 && p->n_tokens <= 64) {
      if (int rc = pcs::launch_attn_latent(*p, st, &latent_splits)) return rc;
    }
    if (latent_splits > 0) {
      PCS_DISPATCH(p->dtype, pcs::attn_combine_kernel<T><<<dim3(p->n_tokens, p->n_heads, (p->vdim + pcs::kAttnThreads - 1) / pcs::kAttnThreads), pcs::kAttnThreads, 0, st>>>(*p, latent_splits));
      PCS_CHECK_CUDA(cudaGetLastError());
      pcs::count_launch();
      return PCS_OK;
    }
  }
  const size_t smem = static_cast<size_t>(p->dim + pcs::kAttnThreads) * sizeof(float);
  PCS_REQUIRE(smem <= 48 * 1024, "pcs_attn: dim %d exceeds the shared-memory query row", p->dim);
  // few tokens over many keys (decoding): the keys are split so that the launch fills the GPU; each split has >= 128 keys
  const int piece = p->dtype == PCS_BF16 ? 8 : 4;
  const bool decode = (p->impl == 0 || p->impl == 2) && p->workspace != nullptr && p->dim % piece == 0 && p->vdim % piece == 0 &&
                      p->vdim / piece <= pcs::kAttnThreads && p->v_row_stride % piece == 0;
  int splits = 1;
  if (p->workspace != nullptr && p->max_keys > 512) {
    const long long blocks = static_cast<long long>(p->n_tokens) * p->n_heads;
    const int want = static_cast<int>((2 * 148 + blocks - 1) / blocks);
    splits = p->max_keys / (decode ? 128 : 256);
    if (splits > want) splits = want;
    if (splits > pcs::kAttnMaxSplits) splits = pcs::kAttnMaxSplits;
    if (splits < 1) splits = 1;
    PCS_REQUIRE(splits == 1 || p->workspace_floats >= static_cast<long long>(p->n_tokens) * p->n_heads * splits * (p->vdim + 2),
                "pcs_attn: workspace too small for %d splits", splits);
  }
  dim3 grid(p->n_tokens, p->n_heads, splits);
  if (decode) {
    const size_t smem_d = smem + static_cast<size_t>(pcs::kAttnThreads) * piece * sizeof(float);
    PCS_DISPATCH(p->dtype, pcs::attn_decode_kernel<T><<<grid, pcs::kAttnThreads, smem_d, st>>>(*p));
  } else {
    PCS_DISPATCH(p->dtype, pcs::attn_plain_kernel<T><<<grid, pcs::kAttnThreads, smem, st>>>(*p));
  }
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  if (splits > 1) {
    PCS_DISPATCH(p->dtype, pcs::attn_combine_kernel<T><<<dim3(p->n_tokens, p->n_heads, (p->vdim + pcs::kAttnThreads - 1) / pcs::kAttnThreads), pcs::kAttnThreads, 0, st>>>(*p, splits));
    PCS_CHECK_CUDA(cudaGetLastError());
    pcs::count_launch();
  }
  return PCS_OK;
}
