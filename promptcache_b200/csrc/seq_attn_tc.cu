// Tensor-core attention over the slot pool for prompts (bfloat16 storage).
//
// One block = 64 consecutive new tokens of one sequence and one head, 4 warps of 16 query rows each; keys in tiles of 64.
// Q, K and V tiles are staged in shared memory (rows padded by 16 bytes; K in two cp.async stages, the next tile travels
// while the current one is multiplied; V in one, loaded during the score phase), fragments come from ldmatrix, products are
// m16n8k16 bfloat16 tensor-core operations with 32-bit accumulators held in registers:
//     S = Q K^T           32-bit scores; scale, distance bias r1 ln(1 + r2 (i - j)) and the causal mask applied per score
//                         (a cap cap * tanh(s / cap) before the bias; a sliding window with kept first keys: key tiles that
//                         no row of the block sees are skipped)
//     online softmax      running maximum / sum per query row in 32-bit; a sink starts them at (0, 1) instead of (-inf, 0)
//     O += P V            the 32-bit weights enter the tensor cores as TWO bfloat16 operands, P = hi + lo with
//                         hi = bf16(P), lo = bf16(P - hi), so that the product keeps ~16 bits of every weight instead of 8
// Key / value widths are padded in shared memory to 64, 128 or 256 (zero fill); every width that is a multiple of 8 up to
// 256 is served.  Other types and shapes fall to the plain kernel (seq_attn.cu).
#include "seq_common.cuh"
#include "seq_mma.cuh"

namespace pcs {

namespace {

constexpr int BM = 64, BN = 64, TC_THREADS = 128, PAD = 8;
constexpr int kSMs = 148;  // B200: blocks are handed to the SMs in index order, one per SM and round

// rows [row0, row0 + 64) x `width` of a [*, src_stride] bfloat16 matrix into a [64][WP + PAD] tile; rows >= n_rows and
// columns >= width are zero
template <int WP>
__device__ __forceinline__ void load_tile(__nv_bfloat16* dst, const __nv_bfloat16* src, long long src_stride, int row0, int n_rows,
                                          int width) {
  constexpr int CH = WP / 8;
  for (int e = threadIdx.x; e < BM * CH; e += TC_THREADS) {
    const int r = e / CH, c = (e - r * CH) * 8;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (row0 + r < n_rows && c < width) v = *reinterpret_cast<const uint4*>(src + static_cast<long long>(row0 + r) * src_stride + c);
    *reinterpret_cast<uint4*>(dst + r * (WP + PAD) + c) = v;
  }
}

// the same through cp.async (the caller commits and waits)
template <int WP>
__device__ __forceinline__ void load_tile_async(__nv_bfloat16* dst, const __nv_bfloat16* src, long long src_stride, int row0, int n_rows,
                                                int width) {
  constexpr int CH = WP / 8;
  for (int e = threadIdx.x; e < BM * CH; e += TC_THREADS) {
    const int r = e / CH, c = (e - r * CH) * 8;
    __nv_bfloat16* d = dst + r * (WP + PAD) + c;
    if (row0 + r < n_rows && c < width) cp_async16(d, src + static_cast<long long>(row0 + r) * src_stride + c);
    else *reinterpret_cast<uint4*>(d) = make_uint4(0u, 0u, 0u, 0u);
  }
}

template <int DP, int VP>
__global__ void __launch_bounds__(TC_THREADS, (DP <= 128 && VP <= 128) ? 3 : 1) attn_tc_kernel(const pcs_attn_params p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* Kbuf = Qs + BM * (DP + PAD);       // two stages of K, then one of V
  __nv_bfloat16* Vbuf = Kbuf + 2 * BN * (DP + PAD);
  // one-dimensional grid in the order (query tile, sequence, head), the LAST query tiles first: blocks are handed out in
  // index order, so every head's longest blocks (most key tiles) start in the first wave and the tail is made of short ones
  const int per_tile = p.n_seqs * p.n_heads, n_qtiles = (p.max_len + BM - 1) / BM;
  // every second group of 148 blocks (one per SM) runs backwards, so that an SM's first block, one of the longest, shares
  // the SM with one of the shortest of the next group rather than with another long one
  int idx = blockIdx.x;
  {
    const int wave = idx / kSMs, first = wave * kSMs, last = min(first + kSMs, static_cast<int>(gridDim.x)) - 1;
    if (wave & 1) idx = first + (last - idx);
  }
  const int qt = idx / per_tile, rem = idx - qt * per_tile;
  const int b = rem / p.n_heads, h = rem - b * p.n_heads, q0 = (n_qtiles - 1 - qt) * BM;
  const int len = p.seq_len[b];
  if (q0 >= len) return;
  const int pos0 = p.seq_pos0[b], off = p.seq_off[b], slot = p.pool_slot ? p.pool_slot[b] : p.seq_slot[b];
  const int g = h / (p.n_heads / p.n_kv_heads), D = p.dim, V = p.vdim;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, grp = lane >> 2, qd = lane & 3;
  const __nv_bfloat16* Kg = static_cast<const __nv_bfloat16*>(p.k_pool) + (static_cast<long long>(slot) * p.n_kv_heads + g) * p.cap * D;
  const __nv_bfloat16* Vg = static_cast<const __nv_bfloat16*>(p.v_pool) + (static_cast<long long>(slot) * p.n_kv_heads + g) * p.cap * V;
  const __nv_bfloat16* Qg = static_cast<const __nv_bfloat16*>(p.q) + static_cast<long long>(off) * p.n_heads * D + h * D;
  load_tile<DP>(Qs, Qg, static_cast<long long>(p.n_heads) * D, q0, len, D);
  const int total_keys = pos0 + len;
  const int n_keys = min(total_keys, pos0 + q0 + BM);  // the last row of this tile sees keys below this bound
  const float r1 = p.bias_r1 ? p.bias_r1[h] : 0.f, r2 = p.bias_r1 ? p.bias_r2[h] : 0.f;
  const bool bias = p.bias_r1 != nullptr;
  // this thread's two query rows (grp, grp + 8 of the warp's 16) and their positions
  const int row_a = warp * 16 + grp, row_b = row_a + 8;
  const int pq_a = pos0 + q0 + row_a, pq_b = pos0 + q0 + row_b;
  // the bias r1 ln(1 + r2 d) depends on the distance d = i - j alone: 127 distances per tile, computed once per tile into
  // shared memory in the base-2 domain (r1 log2(1 + r2 d)).  A thread's two scores of an 8-key group are neighbours in
  // the table; two copies, one shifted by an entry, keep every thread's float2 read aligned whatever its row's parity.
  float* T0 = reinterpret_cast<float*>(Vbuf + BN * (VP + PAD));
  float* T1 = T0 + 144;  // 16 banks away from T0: the odd and the even rows of a warp read different banks
  const float* tp_a = (row_a & 1) ? T0 + (63 - row_a + qd * 2) : T1 + (62 - row_a + qd * 2);
  const float scale2 = p.scale * 1.4426950408889634f;
  float m_a = p.sink ? (p.sink_logit ? p.sink_logit[h] * 1.4426950408889634f : 0.f) : -INFINITY, m_b = m_a;  // base-2 domain
  float l_a = (p.sink && qd == 0) ? 1.f : 0.f, l_b = l_a;  // per-thread share of the row sums; the sink's 1 sits in one lane
  float o[VP / 8][4];
#pragma unroll
  for (int i = 0; i < VP / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  const uint32_t q_base = static_cast<uint32_t>(__cvta_generic_to_shared(Qs)) +
                          ((warp * 16 + (lane & 15)) * (DP + PAD) + (lane >> 4) * 8) * 2;
  const uint32_t k_base0 = static_cast<uint32_t>(__cvta_generic_to_shared(Kbuf)) + (((lane & 7)) * (DP + PAD) + (lane >> 3) * 8) * 2;
  const uint32_t v_base0 = static_cast<uint32_t>(__cvta_generic_to_shared(Vbuf)) + ((lane & 15) * (VP + PAD) + (lane >> 4) * 8) * 2;
  // With a window the key tiles a block walks are the tiles of the kept first keys and then the tiles from the one that holds
  // the lowest key its first row sees; when the two parts touch, all tiles from 0.  Tile `it` of the walk starts at key
  // (it < n_first ? it : lo_tile + it - n_first) * 64.
  const bool windowed = p.window > 0;
  int lo_tile = 0, n_first = 0;
  if (windowed) {
    lo_tile = max(0, pos0 + q0 - p.window + 1) / BN;
    n_first = (min(max(p.keep_first, 0), total_keys) + BN - 1) / BN;
    if (n_first >= lo_tile) { n_first = 0; lo_tile = 0; }
  }
  const int n_it = n_first + (n_keys + BN - 1) / BN - lo_tile;
  const float cap_in = p.softcap > 0.f ? p.scale / p.softcap * 2.885390081777927f : 0.f;  // 2 log2(e) scale / cap
  const float cap_out = p.softcap * 1.4426950408889634f;
  load_tile_async<DP>(Kbuf, Kg, D, (n_first > 0 ? 0 : lo_tile) * BN, total_keys, D);
  cp_async_commit();

  // K in two stages, V in one (three blocks of 4 warps fit an SM at widths up to 128): per tile the copies are committed in
  // the order V_t, K_{t+1}; K_t is complete when at most those two groups are pending, V_t when at most one is
  for (int it = 0; it < n_it; ++it) {
    const int st = it & 1;
    const int k0 = (it < n_first ? it : lo_tile + it - n_first) * BN;
    load_tile_async<VP>(Vbuf, Vg, V, k0, total_keys, V);  // has the score phase to arrive
    cp_async_commit();
    if (it + 1 < n_it)
      load_tile_async<DP>(Kbuf + (st ^ 1) * BN * (DP + PAD), Kg, D, (it + 1 < n_first ? it + 1 : lo_tile + it + 1 - n_first) * BN, total_keys, D);
    cp_async_commit();  // (an empty group after the last tile keeps the counts the same)
    if (bias) {  // this tile's distance biases, one per thread: entry y belongs to distance (q0 - k0) + 63 - y
      const int y = threadIdx.x, d = pos0 + q0 - k0 + 63 - y;
      const float v = d >= 0 ? r1 * __log2f(fmaf(r2, static_cast<float>(d), 1.f)) : 0.f;
      T0[y] = v;
      if (y > 0) T1[y - 1] = v;
    }
    cp_async_wait<2>();
    __syncthreads();  // this K tile (and Q on the first pass), and its bias table, are complete for every warp
    const uint32_t k_base = k_base0 + st * BN * (DP + PAD) * 2, v_base = v_base0;
    // ---- S = Q K^T: 16 rows x 64 keys per warp; eight independent accumulators between two products into the same one ----
    float s[BN / 8][4];
#pragma unroll
    for (int i = 0; i < BN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < DP / 16; kk += 2) {
      uint32_t a0, a1, a2, a3, c0, c1, c2, c3;
      ldsm_x4(q_base + kk * 32, a0, a1, a2, a3);
      ldsm_x4(q_base + (kk + 1) * 32, c0, c1, c2, c3);
      {
        uint32_t kf[BN / 8][4];  // keys u*8.., dims kk*16.. ([0],[1]) and (kk+1)*16.. ([2],[3])
#pragma unroll
        for (int u = 0; u < BN / 8; ++u) ldsm_x4(k_base + (u * 8 * (DP + PAD) + kk * 16) * 2, kf[u][0], kf[u][1], kf[u][2], kf[u][3]);
#pragma unroll
        for (int u = 0; u < BN / 8; ++u) mma_bf16(s[u], a0, a1, a2, a3, kf[u][0], kf[u][1]);
#pragma unroll
        for (int u = 0; u < BN / 8; ++u) mma_bf16(s[u], c0, c1, c2, c3, kf[u][2], kf[u][3]);
      }
    }
    // ---- scores in the base-2 domain: s * scale * log2(e) - bias (from the tile's table); causal mask only where a tile
    //      reaches past the warp's first row or the last key; row maxima ----
    const bool need_mask = (k0 + BN - 1 > pos0 + q0 + warp * 16) || (k0 + BN > total_keys) ||
                           (windowed && pos0 + q0 + warp * 16 + 15 - k0 >= p.window);
    float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < BN / 8; ++nt) {
      float2 ba = make_float2(0.f, 0.f), bb = ba;
      if (bias) {
        ba = *reinterpret_cast<const float2*>(tp_a + nt * 8);
        bb = *reinterpret_cast<const float2*>(tp_a + nt * 8 - 8);
      }
      if (p.softcap > 0.f) {  // cap tanh(s scale / cap) as 1 - 2 / (1 + e^(2x)), then to the base-2 domain
#pragma unroll
        for (int c = 0; c < 4; ++c) s[nt][c] = (1.f - __fdividef(2.f, 1.f + ex2(s[nt][c] * cap_in))) * cap_out;
        s[nt][0] -= ba.x; s[nt][1] -= ba.y; s[nt][2] -= bb.x; s[nt][3] -= bb.y;
      } else {
        s[nt][0] = fmaf(s[nt][0], scale2, -ba.x);
        s[nt][1] = fmaf(s[nt][1], scale2, -ba.y);
        s[nt][2] = fmaf(s[nt][2], scale2, -bb.x);
        s[nt][3] = fmaf(s[nt][3], scale2, -bb.y);
      }
      if (need_mask) {
        const int pk = k0 + nt * 8 + qd * 2;
        if (pk > pq_a || pk >= total_keys) s[nt][0] = -INFINITY;
        if (pk + 1 > pq_a || pk + 1 >= total_keys) s[nt][1] = -INFINITY;
        if (pk > pq_b || pk >= total_keys) s[nt][2] = -INFINITY;
        if (pk + 1 > pq_b || pk + 1 >= total_keys) s[nt][3] = -INFINITY;
        if (windowed) {
          if (pq_a - pk >= p.window && pk >= p.keep_first) s[nt][0] = -INFINITY;
          if (pq_a - pk - 1 >= p.window && pk + 1 >= p.keep_first) s[nt][1] = -INFINITY;
          if (pq_b - pk >= p.window && pk >= p.keep_first) s[nt][2] = -INFINITY;
          if (pq_b - pk - 1 >= p.window && pk + 1 >= p.keep_first) s[nt][3] = -INFINITY;
        }
      }
      mx_a = fmaxf(mx_a, fmaxf(s[nt][0], s[nt][1]));
      mx_b = fmaxf(mx_b, fmaxf(s[nt][2], s[nt][3]));
    }
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
    // a masked score gives 2^-inf = 0; a row that has seen no key yet (under a window the first tile of the walk may hold
    // none of a later row's keys) keeps its maximum at minus infinity and subtracts 0 instead
    const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
    const float f_a = (m_a == -INFINITY) ? 0.f : ex2(m_a - mn_a), f_b = (m_b == -INFINITY) ? 0.f : ex2(m_b - mn_b);
    m_a = mn_a;
    m_b = mn_b;
    const float sub_a = mn_a == -INFINITY ? 0.f : mn_a, sub_b = mn_b == -INFINITY ? 0.f : mn_b;
    float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
    for (int nt = 0; nt < BN / 8; ++nt) {
      s[nt][0] = ex2(s[nt][0] - sub_a);
      s[nt][1] = ex2(s[nt][1] - sub_a);
      s[nt][2] = ex2(s[nt][2] - sub_b);
      s[nt][3] = ex2(s[nt][3] - sub_b);
      sum_a += s[nt][0] + s[nt][1];
      sum_b += s[nt][2] + s[nt][3];
    }
    l_a = l_a * f_a + sum_a;
    l_b = l_b * f_b + sum_b;
#pragma unroll
    for (int i = 0; i < VP / 8; ++i) {
      o[i][0] *= f_a; o[i][1] *= f_a; o[i][2] *= f_b; o[i][3] *= f_b;
    }
    cp_async_wait<1>();
    __syncthreads();  // the V tile is complete for every warp
    // ---- O += P V, P as hi + lo; eight value-column tiles between the hi and the lo product of one accumulator ----
#pragma unroll
    for (int j = 0; j < BN / 16; ++j) {
      uint32_t lo0, lo1, lo2, lo3;
      const uint32_t hi0 = split_pair(s[2 * j][0], s[2 * j][1], lo0);
      const uint32_t hi1 = split_pair(s[2 * j][2], s[2 * j][3], lo1);
      const uint32_t hi2 = split_pair(s[2 * j + 1][0], s[2 * j + 1][1], lo2);
      const uint32_t hi3 = split_pair(s[2 * j + 1][2], s[2 * j + 1][3], lo3);
#pragma unroll
      for (int vn = 0; vn < VP / 8; vn += 8) {
        uint32_t vf[4][4];  // keys j*16.., value columns (vn + 2u)*8.. ([0],[1]) and (vn + 2u + 1)*8.. ([2],[3])
#pragma unroll
        for (int u = 0; u < 4; ++u) ldsm_x4_t(v_base + (j * 16 * (VP + PAD) + (vn + 2 * u) * 8) * 2, vf[u][0], vf[u][1], vf[u][2], vf[u][3]);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          mma_bf16(o[vn + 2 * u], hi0, hi1, hi2, hi3, vf[u][0], vf[u][1]);
          mma_bf16(o[vn + 2 * u + 1], hi0, hi1, hi2, hi3, vf[u][2], vf[u][3]);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          mma_bf16(o[vn + 2 * u], lo0, lo1, lo2, lo3, vf[u][0], vf[u][1]);
          mma_bf16(o[vn + 2 * u + 1], lo0, lo1, lo2, lo3, vf[u][2], vf[u][3]);
        }
      }
    }
    __syncthreads();  // every warp has read V and this K stage: the next tiles may overwrite them
  }
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
  const float inv_a = l_a > 0.f ? 1.f / l_a : 0.f, inv_b = l_b > 0.f ? 1.f / l_b : 0.f;
  __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out) + static_cast<long long>(off) * p.n_heads * V + h * V;
#pragma unroll
  for (int vn = 0; vn < VP / 8; ++vn) {
    const int c = vn * 8 + qd * 2;
    if (c < V) {
      if (q0 + row_a < len)
        *reinterpret_cast<uint32_t*>(out + static_cast<long long>(q0 + row_a) * p.n_heads * V + c) = pack_bf16(o[vn][0] * inv_a, o[vn][1] * inv_a);
      if (q0 + row_b < len)
        *reinterpret_cast<uint32_t*>(out + static_cast<long long>(q0 + row_b) * p.n_heads * V + c) = pack_bf16(o[vn][2] * inv_b, o[vn][3] * inv_b);
    }
  }
}

template <int DP, int VP>
int launch(const pcs_attn_params& p, cudaStream_t st) {
  const size_t smem = (static_cast<size_t>(BM + 2 * BN) * (DP + PAD) + static_cast<size_t>(BN) * (VP + PAD)) * sizeof(__nv_bfloat16) +
                      272 * sizeof(float);
  static bool configured = false;
  if (!configured) {
    PCS_CHECK_CUDA(cudaFuncSetAttribute(attn_tc_kernel<DP, VP>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    configured = true;
  }
  dim3 grid(static_cast<unsigned>((p.max_len + BM - 1) / BM) * p.n_seqs * p.n_heads);
  attn_tc_kernel<DP, VP><<<grid, TC_THREADS, smem, st>>>(p);
  PCS_CHECK_CUDA(cudaGetLastError());
  count_launch();
  return PCS_OK;
}

template <int DP>
int launch_v(const pcs_attn_params& p, cudaStream_t st) {
  if (p.vdim <= 64) return launch<DP, 64>(p, st);
  if (p.vdim <= 128) return launch<DP, 128>(p, st);
  return launch<DP, 256>(p, st);
}

}  // namespace

int launch_attn_tc(const pcs_attn_params& p, cudaStream_t st, bool* handled) {
  *handled = false;
  if (p.dtype != PCS_BF16 || p.max_len < 16 || (p.v_row_stride != 0 && p.v_row_stride != p.vdim) || p.dim % 8 != 0 || p.vdim % 8 != 0 || p.dim > 256 || p.vdim > 256) return PCS_OK;
  if (!p.seq_pos0 || !p.seq_len || !p.seq_off) return PCS_OK;
  if (static_cast<long long>((p.max_len + BM - 1) / BM) * p.n_seqs * p.n_heads > 0x7fffffffLL) return PCS_OK;
  *handled = true;
  if (p.dim <= 64) return launch_v<64>(p, st);
  if (p.dim <= 128) return launch_v<128>(p, st);
  return launch_v<256>(p, st);
}

}  // namespace pcs
