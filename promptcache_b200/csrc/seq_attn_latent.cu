// Decoding attention over rows that all heads share (the latent form of low-rank attention): one cached row per key serves as
// the key of every head, and its leading vdim numbers as the value of every head.
//
// One block = one token, a group of 16 heads and a split of the keys; 4 warps; keys in tiles of 64 rows, staged once in shared
// memory (two cp.async stages) and used by all 16 heads, so a row crosses from L2 once per 16 heads instead of once per head.
//     S = Q K^T      the 16 heads are the rows of the m16n8k16 bfloat16 products; every warp forms all 16 x 64 scores (the
//                    softmax statistics then need no exchange between warps)
//     online softmax base 2, 32-bit; a sink starts split 0 at (sink, 1)
//     O += P V       P enters as hi + lo bfloat16 operands; V is the same tile read transposed; a warp owns a quarter of the
//                    value columns
// Every block writes its partial (maximum, sum, unnormalised result) per head; the merge kernel of the plain path finishes.
#include "seq_common.cuh"
#include "seq_mma.cuh"

namespace pcs {

namespace {

constexpr int LB_N = 64, LB_THREADS = 128, LB_PAD = 8, LB_HEADS = 16;
constexpr int kLatentMaxSplits = 64;  // what the merge kernel and the workspace size of pcs_attn_workspace_floats allow

template <int NT>  // n8 tiles of value columns per warp: the kernel serves vdim <= 4 * NT * 8
__global__ void __launch_bounds__(LB_THREADS) attn_latent_kernel(const pcs_attn_params p, int DKP) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int ROW = DKP + LB_PAD;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [16][ROW]
  __nv_bfloat16* Kbuf = Qs + LB_HEADS * ROW;                        // [2][64][ROW]
  const int t = blockIdx.x, h0 = blockIdx.y * LB_HEADS, sp = blockIdx.z, S = gridDim.z;
  const int b = p.tok_seq[t], pos = p.tok_pos[t], slot = p.pool_slot ? p.pool_slot[b] : p.seq_slot[b];
  const int D = p.dim, V = p.vdim, H = p.n_heads;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, grp = lane >> 2, qd = lane & 3;
  const int n_keys = pos + 1;
  const int chunk = ((n_keys + S - 1) / S + LB_N - 1) / LB_N * LB_N;
  const int k_begin = sp * chunk, k_end = min(n_keys, k_begin + chunk);
  const __nv_bfloat16* Kg = static_cast<const __nv_bfloat16*>(p.k_pool) + static_cast<long long>(slot) * p.cap * D;
  const __nv_bfloat16* Qg = static_cast<const __nv_bfloat16*>(p.q) + (static_cast<long long>(t) * H + h0) * D;
  const int pieces = DKP / 8;
  auto load_tile = [&](int stage, int k0) {
    __nv_bfloat16* dst = Kbuf + stage * LB_N * ROW;
    for (int e = tid; e < LB_N * pieces; e += LB_THREADS) {
      const int r = e / pieces, c = (e - r * pieces) * 8;
      __nv_bfloat16* d = dst + r * ROW + c;
      if (k0 + r < k_end && c < D) cp_async16(d, Kg + static_cast<long long>(k0 + r) * D + c);
      else *reinterpret_cast<uint4*>(d) = make_uint4(0u, 0u, 0u, 0u);
    }
  };
  const int n_tiles = k_begin < k_end ? (k_end - k_begin + LB_N - 1) / LB_N : 0;
  if (n_tiles > 0) load_tile(0, k_begin);
  cp_async_commit();
  for (int e = tid; e < LB_HEADS * pieces; e += LB_THREADS) {
    const int r = e / pieces, c = (e - r * pieces) * 8;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (h0 + r < H && c < D) v = *reinterpret_cast<const uint4*>(Qg + static_cast<long long>(r) * D + c);
    *reinterpret_cast<uint4*>(Qs + r * ROW + c) = v;
  }
  // this thread's two heads (rows grp and grp + 8 of the group)
  const int h_a = h0 + grp, h_b = h_a + 8;
  const bool sink_here = p.sink && sp == 0;
  const float LOG2E = 1.4426950408889634f;
  float m_a = (sink_here && h_a < H) ? (p.sink_logit ? p.sink_logit[h_a] * LOG2E : 0.f) : -INFINITY;
  float m_b = (sink_here && h_b < H) ? (p.sink_logit ? p.sink_logit[h_b] * LOG2E : 0.f) : -INFINITY;
  float l_a = (sink_here && qd == 0 && h_a < H) ? 1.f : 0.f, l_b = (sink_here && qd == 0 && h_b < H) ? 1.f : 0.f;
  float o[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  const float scale2 = p.scale * LOG2E;
  const uint32_t q_base = static_cast<uint32_t>(__cvta_generic_to_shared(Qs)) + ((lane & 15) * ROW + (lane >> 4) * 8) * 2;
  const uint32_t kb = static_cast<uint32_t>(__cvta_generic_to_shared(Kbuf));
  const uint32_t k_off = ((lane & 7) * ROW + (lane >> 3) * 8) * 2;
  const uint32_t v_off = ((lane & 15) * ROW + (lane >> 4) * 8) * 2;
  for (int it = 0; it < n_tiles; ++it) {
    const int st = it & 1, k0 = k_begin + it * LB_N;
    if (it + 1 < n_tiles) load_tile(st ^ 1, k0 + LB_N);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();  // this tile (and the queries on the first pass) is complete for every warp
    const uint32_t k_base = kb + st * LB_N * ROW * 2 + k_off, v_base = kb + st * LB_N * ROW * 2 + v_off;
    float s[LB_N / 8][4];
#pragma unroll
    for (int i = 0; i < LB_N / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
    for (int kk = 0; kk < DKP / 16; kk += 2) {
      uint32_t a0, a1, a2, a3, c0, c1, c2, c3;
      ldsm_x4(q_base + kk * 32, a0, a1, a2, a3);
      ldsm_x4(q_base + (kk + 1) * 32, c0, c1, c2, c3);
      uint32_t kf[LB_N / 8][4];
#pragma unroll
      for (int u = 0; u < LB_N / 8; ++u) ldsm_x4(k_base + (u * 8 * ROW + kk * 16) * 2, kf[u][0], kf[u][1], kf[u][2], kf[u][3]);
#pragma unroll
      for (int u = 0; u < LB_N / 8; ++u) mma_bf16(s[u], a0, a1, a2, a3, kf[u][0], kf[u][1]);
#pragma unroll
      for (int u = 0; u < LB_N / 8; ++u) mma_bf16(s[u], c0, c1, c2, c3, kf[u][2], kf[u][3]);
    }
    const bool need_mask = k0 + LB_N > k_end;
    float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < LB_N / 8; ++nt) {
#pragma unroll
      for (int c = 0; c < 4; ++c) s[nt][c] *= scale2;
      if (need_mask) {
        const int pk = k0 + nt * 8 + qd * 2;
        if (pk >= k_end) s[nt][0] = s[nt][2] = -INFINITY;
        if (pk + 1 >= k_end) s[nt][1] = s[nt][3] = -INFINITY;
      }
      mx_a = fmaxf(mx_a, fmaxf(s[nt][0], s[nt][1]));
      mx_b = fmaxf(mx_b, fmaxf(s[nt][2], s[nt][3]));
    }
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
    const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);   // finite: a tile has at least one key
    const float f_a = (m_a == -INFINITY) ? 0.f : ex2(m_a - mn_a), f_b = (m_b == -INFINITY) ? 0.f : ex2(m_b - mn_b);
    m_a = mn_a;
    m_b = mn_b;
    float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
    for (int nt = 0; nt < LB_N / 8; ++nt) {
      s[nt][0] = ex2(s[nt][0] - mn_a);
      s[nt][1] = ex2(s[nt][1] - mn_a);
      s[nt][2] = ex2(s[nt][2] - mn_b);
      s[nt][3] = ex2(s[nt][3] - mn_b);
      sum_a += s[nt][0] + s[nt][1];
      sum_b += s[nt][2] + s[nt][3];
    }
    l_a = l_a * f_a + sum_a;
    l_b = l_b * f_b + sum_b;
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      o[i][0] *= f_a; o[i][1] *= f_a; o[i][2] *= f_b; o[i][3] *= f_b;
    }
    // O += P V over this warp's value columns: n8 tiles warp * NT .. warp * NT + NT - 1 (tiles past the padded row are skipped)
#pragma unroll
    for (int j = 0; j < LB_N / 16; ++j) {
      uint32_t lo0, lo1, lo2, lo3;
      const uint32_t hi0 = split_pair(s[2 * j][0], s[2 * j][1], lo0);
      const uint32_t hi1 = split_pair(s[2 * j][2], s[2 * j][3], lo1);
      const uint32_t hi2 = split_pair(s[2 * j + 1][0], s[2 * j + 1][1], lo2);
      const uint32_t hi3 = split_pair(s[2 * j + 1][2], s[2 * j + 1][3], lo3);
#pragma unroll
      for (int u = 0; u < NT; u += 2) {
        const int col = (warp * NT + u) * 8;
        if (col + 16 <= DKP) {
          uint32_t v0, v1, v2, v3;
          ldsm_x4_t(v_base + (j * 16 * ROW + col) * 2, v0, v1, v2, v3);
          mma_bf16(o[u], hi0, hi1, hi2, hi3, v0, v1);
          mma_bf16(o[u + 1], hi0, hi1, hi2, hi3, v2, v3);
          mma_bf16(o[u], lo0, lo1, lo2, lo3, v0, v1);
          mma_bf16(o[u + 1], lo0, lo1, lo2, lo3, v2, v3);
        }
      }
    }
    __syncthreads();  // every warp has read this stage: the tile after next may overwrite it
  }
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
  // partial (m in natural units, l, unnormalised o) per head for the merge
  const float LN2 = 0.6931471805599453f;
  if (h_a < H) {
    float* part = p.workspace + ((static_cast<long long>(t) * H + h_a) * S + sp) * (V + 2);
    if (warp == 0 && qd == 0) { part[0] = m_a * LN2; part[1] = l_a; }
#pragma unroll
    for (int u = 0; u < NT; ++u) {
      const int c = (warp * NT + u) * 8 + qd * 2;
      if (c < V) { part[2 + c] = o[u][0]; part[3 + c] = o[u][1]; }
    }
  }
  if (h_b < H) {
    float* part = p.workspace + ((static_cast<long long>(t) * H + h_b) * S + sp) * (V + 2);
    if (warp == 0 && qd == 0) { part[0] = m_b * LN2; part[1] = l_b; }
#pragma unroll
    for (int u = 0; u < NT; ++u) {
      const int c = (warp * NT + u) * 8 + qd * 2;
      if (c < V) { part[2 + c] = o[u][2]; part[3 + c] = o[u][3]; }
    }
  }
}

template <int NT>
int launch_nt(const pcs_attn_params& p, cudaStream_t st, int DKP, int splits, size_t smem) {
  static bool configured = false;
  if (!configured) {
    PCS_CHECK_CUDA(cudaFuncSetAttribute(attn_latent_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    configured = true;
  }
  dim3 grid(p.n_tokens, (p.n_heads + LB_HEADS - 1) / LB_HEADS, splits);
  attn_latent_kernel<NT><<<grid, LB_THREADS, smem, st>>>(p, DKP);
  PCS_CHECK_CUDA(cudaGetLastError());
  count_launch();
  return PCS_OK;
}

}  // namespace

// Serves bfloat16 rows shared by all heads whose values are the rows' leading numbers, without bias, cap or window, when a
// workspace for the partial results is given; `splits_out` tells the caller how many partial results the merge reads.
int launch_attn_latent(const pcs_attn_params& p, cudaStream_t st, int* splits_out) {
  *splits_out = 0;
  if (p.dtype != PCS_BF16 || p.n_kv_heads != 1 || p.v_pool != p.k_pool || p.v_row_stride != p.dim || p.workspace == nullptr) return PCS_OK;
  if (p.bias_r1 || p.softcap > 0.f || p.window > 0 || p.dim % 8 != 0 || p.vdim % 8 != 0 || p.vdim > 512 || p.vdim > p.dim) return PCS_OK;
  if ((reinterpret_cast<uintptr_t>(p.k_pool) | reinterpret_cast<uintptr_t>(p.q)) & 15) return PCS_OK;
  const int DKP = (p.dim + 31) / 32 * 32;
  const size_t smem = static_cast<size_t>(LB_HEADS + 2 * LB_N) * (DKP + LB_PAD) * sizeof(__nv_bfloat16);
  if (smem > 220 * 1024) return PCS_OK;
  const int groups = (p.n_heads + LB_HEADS - 1) / LB_HEADS;
  const int max_keys = p.max_keys > 0 ? p.max_keys : p.cap;
  int splits = (max_keys + LB_N - 1) / LB_N;
  const long long blocks = static_cast<long long>(p.n_tokens) * groups;
  const int want = static_cast<int>((2 * 148 + blocks - 1) / blocks);
  if (splits > want) splits = want;
  if (splits > kLatentMaxSplits) splits = kLatentMaxSplits;
  if (splits < 1) splits = 1;
  if (p.workspace_floats < static_cast<long long>(p.n_tokens) * p.n_heads * splits * (p.vdim + 2)) return PCS_OK;
  *splits_out = splits;
  if (p.vdim <= 128) return launch_nt<4>(p, st, DKP, splits, smem);
  if (p.vdim <= 256) return launch_nt<8>(p, st, DKP, splits, smem);
  return launch_nt<16>(p, st, DKP, splits, smem);
}

}  // namespace pcs
