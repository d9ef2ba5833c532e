// Attention whose scores are mixed across heads before the softmax (pcs_attn with `talk`), plain kernel.
//
// For a (query, key) pair the H scaled scores s[g] = scale * q_g . k_g' become s'[h] = sum_g talk[h, g] s[g]; mask and softmax
// follow per head.  The mixing couples all heads of a pair, so one block takes ONE token with ALL its heads (and one split of
// its visible keys), walking the keys in tiles of 32:
//   scores    (head, key) items over the threads; the query rows of all heads sit in shared memory (32-bit), a key row is
//             read in 16-byte pieces where the sizes allow;
//   mix       (head, key) items again, H terms each, from the raw scores in shared memory;
//   softmax   one warp per head, a key per lane: running maximum and sum in 32-bit, the tile's weights back to shared memory;
//   values    (head, value column) items over the threads, each with its accumulator in a register; the tile's value rows were
//             asked for (L2 prefetch) before the scores, the next tile's key rows too.
// The visible keys are a dense list (a sliding window plus kept first keys, or everything up to the query), so the work is
// bounded by the window.  With several splits every block leaves (maximum, sum, accumulator) per head in the workspace, in the
// layout the split merge of pcs_attn reads.  Both compute types; scores, weights and sums are 32-bit.
#include "seq_common.cuh"
#include "seq_mma.cuh"

namespace pcs {

namespace {

constexpr int TK_THREADS = 256, TK_TILE = 32, TK_MAX_ACC = 32;   // heads x vdim <= 8192

struct VisibleKeysT {   // the same dense list of visible keys as the other attention kernels use
  int n_first, lo, count;
  __device__ __forceinline__ VisibleKeysT(int pos, int window, int keep_first) {
    lo = window > 0 ? max(0, pos - window + 1) : 0;
    n_first = min(max(keep_first, 0), lo);
    count = n_first + (pos + 1 - lo);
  }
  __device__ __forceinline__ int key(int v) const { return v < n_first ? v : lo + (v - n_first); }
};

// asks L2 for `nt` rows (keys j0 ... of the visible list) of `width` elements of every key/value head, 128 bytes per request
template <typename T>
__device__ __forceinline__ void prefetch_rows(const T* base, long long head_stride, long long row_stride, int n_kv_heads, const VisibleKeysT& vis, int j0,
                                              int nt, int width) {
  constexpr int PER = 128 / static_cast<int>(sizeof(T));
  const int lines = (width + PER - 1) / PER;
  for (int e = threadIdx.x; e < n_kv_heads * nt * lines; e += TK_THREADS) {
    const int line = e % lines, r = e / lines, jj = r % nt, g = r / nt;
    prefetch_l2(base + g * head_stride + static_cast<long long>(vis.key(j0 + jj)) * row_stride + line * PER);
  }
}

template <typename T>
__global__ void __launch_bounds__(TK_THREADS) attn_talk_kernel(const pcs_attn_params p) {
  extern __shared__ float sm[];
  const int H = p.n_heads, G = p.n_kv_heads, D = p.dim, V = p.vdim, rep = H / G;
  float* qs = sm;                       // [H, D]
  float* tk = qs + H * D;               // [H, H]
  float* sraw = tk + H * H;             // [H, TILE] raw scores
  float* sw = sraw + H * TK_TILE;       // [H, TILE] mixed scores, then weights
  float* mrun = sw + H * TK_TILE;       // [H]
  float* lrun = mrun + H;               // [H]
  float* fac = lrun + H;                // [H]
  const int t = blockIdx.x, sp = blockIdx.y, S = gridDim.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = p.tok_seq[t], pos = p.tok_pos[t], slot = p.pool_slot ? p.pool_slot[b] : p.seq_slot[b];
  const long long VS = p.v_row_stride > 0 ? p.v_row_stride : V;
  const T* q = static_cast<const T*>(p.q) + static_cast<long long>(t) * H * D;
  const T* K = static_cast<const T*>(p.k_pool) + static_cast<long long>(slot) * G * p.cap * D;
  const T* Vp = static_cast<const T*>(p.v_pool) + static_cast<long long>(slot) * G * p.cap * VS;
  for (int i = tid; i < H * D; i += TK_THREADS) qs[i] = ldf(q + i);
  for (int i = tid; i < H * H; i += TK_THREADS) tk[i] = p.talk[i];
  for (int i = tid; i < H; i += TK_THREADS) { mrun[i] = -INFINITY; lrun[i] = 0.f; }
  const VisibleKeysT vis(pos, p.window, p.keep_first);
  const int n_keys = vis.count;
  const int chunk = ((n_keys + S - 1) / S + TK_TILE - 1) / TK_TILE * TK_TILE;
  const int k_begin = sp * chunk, k_end = min(n_keys, k_begin + chunk);
  float acc[TK_MAX_ACC];
#pragma unroll
  for (int u = 0; u < TK_MAX_ACC; ++u) acc[u] = 0.f;
  constexpr int N = Vec<T>::n;
  const bool vec = (D % N) == 0 && (reinterpret_cast<uintptr_t>(K) & 15) == 0;
  const bool vecv = (V % N) == 0 && (VS % N) == 0 && (reinterpret_cast<uintptr_t>(Vp) & 15) == 0;
  __syncthreads();
  for (int j0 = k_begin; j0 < k_end; j0 += TK_TILE) {
    const int nt = min(TK_TILE, k_end - j0);
    // the tile's value rows, and the next tile's key rows, are on their way while the scores are formed
    prefetch_rows(Vp, static_cast<long long>(p.cap) * VS, VS, G, vis, j0, nt, V);
    if (j0 + TK_TILE < k_end) prefetch_rows(K, static_cast<long long>(p.cap) * D, D, G, vis, j0 + TK_TILE, min(TK_TILE, k_end - j0 - TK_TILE), D);
    // raw scores
    for (int e = tid; e < H * TK_TILE; e += TK_THREADS) {
      const int h = e / TK_TILE, jj = e - h * TK_TILE;
      float a = 0.f;
      if (jj < nt) {
        const T* kr = K + (static_cast<long long>(h / rep) * p.cap + vis.key(j0 + jj)) * D;
        const float* qh = qs + h * D;
        if (vec) {
          float a1 = 0.f;
          int d = 0;
          for (; d + 2 * Vec<T>::n <= D; d += 2 * Vec<T>::n) {
            float k0[Vec<T>::n], k1[Vec<T>::n];
            ld16(kr + d, k0);
            ld16(kr + d + Vec<T>::n, k1);
#pragma unroll
            for (int i = 0; i < Vec<T>::n; ++i) { a = fmaf(qh[d + i], k0[i], a); a1 = fmaf(qh[d + Vec<T>::n + i], k1[i], a1); }
          }
          for (; d < D; d += Vec<T>::n) {
            float k0[Vec<T>::n];
            ld16(kr + d, k0);
#pragma unroll
            for (int i = 0; i < Vec<T>::n; ++i) a = fmaf(qh[d + i], k0[i], a);
          }
          a += a1;
        } else {
          for (int d = 0; d < D; ++d) a = fmaf(qh[d], ldf(kr + d), a);
        }
        a *= p.scale;
      }
      sraw[e] = a;
    }
    __syncthreads();
    // mixed across heads; keys past the tile's end are masked
    for (int e = tid; e < H * TK_TILE; e += TK_THREADS) {
      const int h = e / TK_TILE, jj = e - h * TK_TILE;
      float a = 0.f;
      const float* tr = tk + h * H;
      for (int g = 0; g < H; ++g) a = fmaf(tr[g], sraw[g * TK_TILE + jj], a);
      sw[e] = jj < nt ? a : -INFINITY;
    }
    __syncthreads();
    // per head: running maximum and sum, the tile's weights
    for (int h = warp; h < H; h += TK_THREADS / 32) {
      const float s = sw[h * TK_TILE + lane];
      const float m_old = mrun[h];
      const float m_new = fmaxf(m_old, warp_max(s));
      const float w = expf(s - m_new);          // exp(-inf) = 0 for masked keys; every tile holds at least one key
      const float f = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
      const float ts = warp_sum(w);
      sw[h * TK_TILE + lane] = w;
      if (lane == 0) { mrun[h] = m_new; lrun[h] = lrun[h] * f + ts; fac[h] = f; }
    }
    __syncthreads();
    // values: a thread owns whole 16-byte pieces of a head's value row where the sizes allow (accumulator k of a thread belongs
    // to the flat output column out_col(k)), else single columns
    if (vecv) {
#pragma unroll
      for (int u = 0; u < TK_MAX_ACC / N; ++u) {
        const int e = tid + u * TK_THREADS;
        if (e < H * V / N) {
          const int h = e / (V / N), c = (e - h * (V / N)) * N;
          const T* vr = Vp + static_cast<long long>(h / rep) * p.cap * VS + c;
          const float* wh = sw + h * TK_TILE;
          const float f = fac[h];
#pragma unroll
          for (int i = 0; i < N; ++i) acc[u * N + i] *= f;
          for (int jj = 0; jj < nt; ++jj) {
            float vv[N];
            ld16(vr + static_cast<long long>(vis.key(j0 + jj)) * VS, vv);
            const float w = wh[jj];
#pragma unroll
            for (int i = 0; i < N; ++i) acc[u * N + i] = fmaf(w, vv[i], acc[u * N + i]);
          }
        }
      }
    } else {
#pragma unroll
      for (int u = 0; u < TK_MAX_ACC; ++u) {
        const int e = tid + u * TK_THREADS;
        if (e < H * V) {
          const int h = e / V, c = e - h * V;
          const T* vr = Vp + static_cast<long long>(h / rep) * p.cap * VS + c;
          const float* wh = sw + h * TK_TILE;
          float a = acc[u] * fac[h];
          for (int jj = 0; jj < nt; ++jj) a = fmaf(wh[jj], ldf(vr + static_cast<long long>(vis.key(j0 + jj)) * VS), a);
          acc[u] = a;
        }
      }
    }
    __syncthreads();
  }
  // accumulator k of this thread -> flat output column
  auto out_col = [&](int k) { return vecv ? (tid + (k / N) * TK_THREADS) * N + (k % N) : tid + k * TK_THREADS; };
  if (S > 1) {
    if (tid < H) {
      float* part = p.workspace + ((static_cast<long long>(t) * H + tid) * S + sp) * (V + 2);
      part[0] = mrun[tid];
      part[1] = lrun[tid];
    }
#pragma unroll
    for (int u = 0; u < TK_MAX_ACC; ++u) {
      const int e = out_col(u);
      if (e < H * V) {
        const int h = e / V, c = e - h * V;
        p.workspace[((static_cast<long long>(t) * H + h) * S + sp) * (V + 2) + 2 + c] = acc[u];
      }
    }
    return;
  }
  T* o = static_cast<T*>(p.out) + static_cast<long long>(t) * H * V;
#pragma unroll
  for (int u = 0; u < TK_MAX_ACC; ++u) {
    const int e = out_col(u);
    if (e < H * V) {
      const float l = lrun[e / V];
      float a = l > 0.f ? acc[u] / l : 0.f;
      if (p.out_gate) a *= sigmoidf_(ldf(static_cast<const T*>(p.out_gate) + static_cast<long long>(t) * p.out_gate_stride + e));
      stf(o + e, a);
    }
  }
}

}  // namespace

int launch_attn_talk_tc(const pcs_attn_params& p, cudaStream_t st, bool* handled);

// *splits_out: the number of key splits the launch used (> 1: the caller runs the split merge)
int launch_attn_talk(const pcs_attn_params& p, cudaStream_t st, int* splits_out) {
  const int H = p.n_heads;
  PCS_REQUIRE(p.bias_r1 == nullptr && p.softcap == 0.f && !p.sink, "pcs_attn: mixed head scores do not combine with a distance bias, a cap or a sink");
  PCS_REQUIRE(H <= TK_THREADS, "pcs_attn: mixed head scores serve at most %d heads", TK_THREADS);
  if (p.impl == 0) {
    bool handled = false;
    if (int rc = launch_attn_talk_tc(p, st, &handled)) return rc;
    if (handled) { *splits_out = 1; return PCS_OK; }
  }
  PCS_REQUIRE(static_cast<long long>(H) * p.vdim <= TK_THREADS * TK_MAX_ACC, "pcs_attn: mixed head scores: heads x vdim = %lld exceeds %d",
              static_cast<long long>(H) * p.vdim, TK_THREADS * TK_MAX_ACC);
  const size_t smem = (static_cast<size_t>(H) * p.dim + static_cast<size_t>(H) * H + 2 * static_cast<size_t>(H) * TK_TILE + 3 * static_cast<size_t>(H)) * sizeof(float);
  PCS_REQUIRE(smem <= 200 * 1024, "pcs_attn: mixed head scores: %zu bytes of shared memory per token exceed the limit", smem);
  int splits = 1;
  if (p.workspace != nullptr && p.max_keys > 2 * TK_TILE) {   // few tokens: the keys are split so that the launch fills more of the GPU
    const int want = (2 * 148 + p.n_tokens - 1) / p.n_tokens;
    splits = p.max_keys / TK_TILE;   // down to one tile per block: the tiles of a block run one after the other
    if (splits > want) splits = want;
    if (splits > 64) splits = 64;
    if (splits < 1) splits = 1;
    if (p.workspace_floats < static_cast<long long>(p.n_tokens) * H * splits * (p.vdim + 2)) splits = 1;
  }
  if (smem > 48 * 1024)
    PCS_DISPATCH(p.dtype, PCS_CHECK_CUDA(cudaFuncSetAttribute(attn_talk_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)));
  dim3 grid(p.n_tokens, splits);
  PCS_DISPATCH(p.dtype, attn_talk_kernel<T><<<grid, TK_THREADS, smem, st>>>(p));
  PCS_CHECK_CUDA(cudaGetLastError());
  count_launch();
  *splits_out = splits;
  return PCS_OK;
}

}  // namespace pcs
