// Tensor-core attention with scores mixed across heads, for prompts (bfloat16 storage).
//
// The mixing s'[h] = sum_g talk[h, g] s[g] couples all heads of a (query, key) pair, so a block takes 16 consecutive new tokens
// of one sequence with ALL heads; its 8 warps share the heads (warp w owns heads w * HPW ... w * HPW + HPW - 1).  Keys go in
// tiles of BN; the K and V rows of all key/value heads of a tile are staged in shared memory by cp.async (K of the next tile
// travels during the softmax and P V of the current one, V of the next during the next Q K^T).  Per tile:
//     S_g = scale * Q_g K^T   m16n8k16 bfloat16 products of the warp's own heads (query rows of all heads sit in shared memory;
//                             an A fragment is loaded once per 16 coordinates and meets all key columns of the tile), the 32-bit
//                             raw scores of ALL heads go to shared memory
//     mix                     every thread reads, for the score positions of its accumulator fragment, the H raw scores (once for
//                             all heads of its warp) and forms its own heads' mixed scores in 32-bit, two multiply-adds per
//                             instruction; then the causal / window mask
//     online softmax          running maximum / sum per query row and head in 32-bit
//     O_h += P_h V            the 32-bit weights enter the tensor cores as TWO bfloat16 operands (hi + lo), V through ldmatrix.trans
// and at the end O / l, times the element-wise sigmoid gate when one is given.  Head widths are padded in shared memory to 64
// or 128 (zero fill); at most 16 heads.  Other types and shapes take the plain kernel (seq_attn_talk.cu).
#include "seq_common.cuh"
#include "seq_mma.cuh"

namespace pcs {

namespace {

constexpr int TT_BM = 16, TT_PAD = 8;

__device__ __forceinline__ uint32_t lds32(const __nv_bfloat16* p) { return *reinterpret_cast<const uint32_t*>(p); }

// rows [row0, row0 + n_rows_tile) x `width` of `heads` matrices (head hd at src + hd * head_stride, rows `row_stride` apart) into
// dst[(hd * n_rows_tile + r)][WP + PAD]; rows >= n_rows and columns >= width are zero
template <int WP, int THREADS>
__device__ __forceinline__ void load_rows_async(__nv_bfloat16* dst, const __nv_bfloat16* src, long long head_stride, long long row_stride, int heads,
                                                int n_rows_tile, int row0, int n_rows, int width) {
  constexpr int CH = WP / 8;
  const int total = heads * n_rows_tile * CH;
  for (int e = threadIdx.x; e < total; e += THREADS) {
    const int c = (e % CH) * 8, hr = e / CH, r = hr % n_rows_tile, hd = hr / n_rows_tile;
    __nv_bfloat16* d = dst + static_cast<long long>(hr) * (WP + TT_PAD) + c;
    if (row0 + r < n_rows && c < width) cp_async16(d, src + hd * head_stride + static_cast<long long>(row0 + r) * row_stride + c);
    else *reinterpret_cast<uint4*>(d) = make_uint4(0u, 0u, 0u, 0u);
  }
}

template <int WP, int HPW, int BN, int NW, int MINB>
__global__ void __launch_bounds__(NW * 32, MINB) attn_talk_tc_kernel(const pcs_attn_params p) {
  constexpr int LD = WP + TT_PAD, NT = BN / 8, LDS_S = BN + 8, TT_THREADS = NW * 32;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int H = p.n_heads, G = p.n_kv_heads, D = p.dim, V = p.vdim, rep = H / G;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);            // [H][16][LD]
  __nv_bfloat16* Ks = Qs + H * TT_BM * LD;                                    // [G][BN][LD]
  __nv_bfloat16* Vs = Ks + G * BN * LD;                                       // [G][BN][LD]
  float* Ss = reinterpret_cast<float*>(Vs + G * BN * LD);                     // [H][16][BN + 8] raw scores
  float* Tk = Ss + H * TT_BM * LDS_S;                                         // [warps * HPW][H]
  const int n_qtiles = (p.max_len + TT_BM - 1) / TT_BM;
  const int b = blockIdx.x / n_qtiles, qt = n_qtiles - 1 - blockIdx.x % n_qtiles;   // long tiles first
  const int len = p.seq_len[b], q0 = qt * TT_BM;
  if (q0 >= len) return;
  const int pos0 = p.seq_pos0[b], off = p.seq_off[b], slot = p.pool_slot ? p.pool_slot[b] : p.seq_slot[b];
  const int rows = min(TT_BM, len - q0);                 // valid query rows
  const int qp0 = pos0 + q0, n_ctx = qp0 + rows;         // first query's position; keys [0, n_ctx) exist for this block
  const int lo = p.window > 0 ? max(0, qp0 - p.window + 1) : 0;
  const int n_tiles = (n_ctx - lo + BN - 1) / BN;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, tq = lane & 3;
  const __nv_bfloat16* Q = static_cast<const __nv_bfloat16*>(p.q) + static_cast<long long>(off + q0) * H * D;
  const __nv_bfloat16* K = static_cast<const __nv_bfloat16*>(p.k_pool) + static_cast<long long>(slot) * G * p.cap * D;
  const long long VS = p.v_row_stride > 0 ? p.v_row_stride : V;
  const __nv_bfloat16* Vg = static_cast<const __nv_bfloat16*>(p.v_pool) + static_cast<long long>(slot) * G * p.cap * VS;
  // queries of all heads: head hd's rows are H * D apart
  load_rows_async<WP, TT_THREADS>(Qs, Q, D, static_cast<long long>(H) * D, H, TT_BM, 0, rows, D);
  load_rows_async<WP, TT_THREADS>(Ks, K, static_cast<long long>(p.cap) * D, D, G, BN, lo, n_ctx, D);
  cp_async_commit();
  load_rows_async<WP, TT_THREADS>(Vs, Vg, static_cast<long long>(p.cap) * VS, VS, G, BN, lo, n_ctx, V);
  cp_async_commit();
  float oacc[HPW][WP / 8][4];
  float mrow[HPW][2], lrow[HPW][2];
#pragma unroll
  for (int i = 0; i < HPW; ++i) {
    mrow[i][0] = mrow[i][1] = -INFINITY;
    lrow[i][0] = lrow[i][1] = 0.f;
#pragma unroll
    for (int n = 0; n < WP / 8; ++n) oacc[i][n][0] = oacc[i][n][1] = oacc[i][n][2] = oacc[i][n][3] = 0.f;
  }
  const int pos_a = qp0 + gq, pos_b = qp0 + gq + 8;      // positions of the thread's two query rows
  // the rows of the mixing matrix of this warp's heads (zero for heads past H); the score scale rides in them
  float* Tw = Tk + warp * HPW * H;
  for (int e = lane; e < HPW * H; e += 32) Tw[e] = warp * HPW + e / H < H ? p.talk[(warp * HPW + e / H) * H + e % H] * p.scale : 0.f;
  __syncwarp();
  for (int jt = 0; jt < n_tiles; ++jt) {
    const int j0 = lo + jt * BN;
    // all keys of the tile at or before the first query and inside the last valid row's window: nothing to mask
    const bool full_tile = j0 + BN - 1 <= qp0 && (p.window <= 0 || (qp0 + TT_BM - 1) - j0 < p.window);
    cp_async_wait<1>();      // K of this tile (and, on the first tile, Q)
    __syncthreads();
    // ---- raw scores of the warp's own heads -> shared memory
#pragma unroll
    for (int i = 0; i < HPW; ++i) {
      const int h = warp * HPW + i;
      if (h < H) {
        float sacc[NT][4];
#pragma unroll
        for (int n = 0; n < NT; ++n) sacc[n][0] = sacc[n][1] = sacc[n][2] = sacc[n][3] = 0.f;
        const __nv_bfloat16* qh = Qs + static_cast<long long>(h) * TT_BM * LD;
        const __nv_bfloat16* kh = Ks + static_cast<long long>(h / rep) * BN * LD;
#pragma unroll
        for (int ks = 0; ks < WP / 16; ++ks) {
          const uint32_t a0 = lds32(qh + gq * LD + ks * 16 + 2 * tq), a1 = lds32(qh + (gq + 8) * LD + ks * 16 + 2 * tq);
          const uint32_t a2 = lds32(qh + gq * LD + ks * 16 + 8 + 2 * tq), a3 = lds32(qh + (gq + 8) * LD + ks * 16 + 8 + 2 * tq);
#pragma unroll
          for (int n = 0; n < NT; ++n) {
            const __nv_bfloat16* kr = kh + (n * 8 + gq) * LD + ks * 16 + 2 * tq;
            mma_bf16(sacc[n], a0, a1, a2, a3, lds32(kr), lds32(kr + 8));
          }
        }
        float* sh = Ss + static_cast<long long>(h) * TT_BM * LDS_S;
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          *reinterpret_cast<float2*>(sh + gq * LDS_S + n * 8 + 2 * tq) = make_float2(sacc[n][0], sacc[n][1]);
          *reinterpret_cast<float2*>(sh + (gq + 8) * LDS_S + n * 8 + 2 * tq) = make_float2(sacc[n][2], sacc[n][3]);
        }
      }
    }
    cp_async_wait<0>();      // V of this tile
    __syncthreads();         // all heads' raw scores are there; K's buffer is free
    if (jt + 1 < n_tiles) load_rows_async<WP, TT_THREADS>(Ks, K, static_cast<long long>(p.cap) * D, D, G, BN, j0 + BN, n_ctx, D);
    cp_async_commit();
    // ---- own heads: mix (every raw score is read once for all heads of the warp), mask, softmax, P V
    float sm_[HPW][NT][4];
#pragma unroll
    for (int i = 0; i < HPW; ++i)
#pragma unroll
      for (int n = 0; n < NT; ++n) sm_[i][n][0] = sm_[i][n][1] = sm_[i][n][2] = sm_[i][n][3] = 0.f;
    for (int g2 = 0; g2 < H; ++g2) {
      float w[HPW];
#pragma unroll
      for (int i = 0; i < HPW; ++i) w[i] = Tw[i * H + g2];
      const float* sg = Ss + static_cast<long long>(g2) * TT_BM * LDS_S;
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const float2 u = *reinterpret_cast<const float2*>(sg + gq * LDS_S + n * 8 + 2 * tq);
        const float2 v = *reinterpret_cast<const float2*>(sg + (gq + 8) * LDS_S + n * 8 + 2 * tq);
#pragma unroll
        for (int i = 0; i < HPW; ++i) {   // two 32-bit multiply-adds per instruction (fma.rn.f32x2)
          const float2 ww = make_float2(w[i], w[i]);
          const float2 a = __ffma2_rn(ww, u, make_float2(sm_[i][n][0], sm_[i][n][1]));
          const float2 c = __ffma2_rn(ww, v, make_float2(sm_[i][n][2], sm_[i][n][3]));
          sm_[i][n][0] = a.x;
          sm_[i][n][1] = a.y;
          sm_[i][n][2] = c.x;
          sm_[i][n][3] = c.y;
        }
      }
    }
#pragma unroll
    for (int i = 0; i < HPW; ++i) {
      const int h = warp * HPW + i;
      if (h < H) {
        float (&s)[NT][4] = sm_[i];
        float mx_a = -INFINITY, mx_b = -INFINITY;
        if (full_tile) {   // every key of the tile is seen by every row of the block: no mask
#pragma unroll
          for (int n = 0; n < NT; ++n) {
            mx_a = fmaxf(mx_a, fmaxf(s[n][0], s[n][1]));
            mx_b = fmaxf(mx_b, fmaxf(s[n][2], s[n][3]));
          }
        } else {
#pragma unroll
          for (int n = 0; n < NT; ++n) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
              const int j = j0 + n * 8 + 2 * tq + c;
              const bool ok_a = j <= pos_a && (p.window <= 0 || pos_a - j < p.window);
              const bool ok_b = j <= pos_b && (p.window <= 0 || pos_b - j < p.window);
              if (!ok_a) s[n][c] = -INFINITY;
              if (!ok_b) s[n][2 + c] = -INFINITY;
              mx_a = fmaxf(mx_a, s[n][c]);
              mx_b = fmaxf(mx_b, s[n][2 + c]);
            }
          }
        }
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
        mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
        mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
        const float mn_a = fmaxf(mrow[i][0], mx_a), mn_b = fmaxf(mrow[i][1], mx_b);
        const float use_a = mn_a == -INFINITY ? 0.f : mn_a, use_b = mn_b == -INFINITY ? 0.f : mn_b;   // a row that has seen no key yet
        // exponentials through the base-2 unit (relative error 2^-22, far below the operands' rounding): exp(x) = 2^(x log2 e)
        constexpr float kLog2e = 1.4426950408889634f;
        const float ua = use_a * kLog2e, ub = use_b * kLog2e;
        const float f_a = mrow[i][0] == -INFINITY ? 0.f : ex2(mrow[i][0] * kLog2e - ua), f_b = mrow[i][1] == -INFINITY ? 0.f : ex2(mrow[i][1] * kLog2e - ub);
        float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          s[n][0] = ex2(fmaf(s[n][0], kLog2e, -ua));
          s[n][1] = ex2(fmaf(s[n][1], kLog2e, -ua));
          s[n][2] = ex2(fmaf(s[n][2], kLog2e, -ub));
          s[n][3] = ex2(fmaf(s[n][3], kLog2e, -ub));
          sum_a += s[n][0] + s[n][1];
          sum_b += s[n][2] + s[n][3];
        }
        sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 1);
        sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 2);
        sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 1);
        sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 2);
        mrow[i][0] = mn_a;
        mrow[i][1] = mn_b;
        lrow[i][0] = lrow[i][0] * f_a + sum_a;
        lrow[i][1] = lrow[i][1] * f_b + sum_b;
        if (__any_sync(0xffffffffu, f_a != 1.f || f_b != 1.f)) {   // (after the first tiles the maxima rarely move)
#pragma unroll
          for (int n = 0; n < WP / 8; ++n) {
            oacc[i][n][0] *= f_a;
            oacc[i][n][1] *= f_a;
            oacc[i][n][2] *= f_b;
            oacc[i][n][3] *= f_b;
          }
        }
        const __nv_bfloat16* vh = Vs + static_cast<long long>(h / rep) * BN * LD;
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          uint32_t l0, l1, l2, l3;
          const uint32_t h0 = split_pair(s[2 * kk][0], s[2 * kk][1], l0), h1 = split_pair(s[2 * kk][2], s[2 * kk][3], l1);
          const uint32_t h2 = split_pair(s[2 * kk + 1][0], s[2 * kk + 1][1], l2), h3 = split_pair(s[2 * kk + 1][2], s[2 * kk + 1][3], l3);
          // four 8 x 8 pieces of V per ldmatrix: keys kk * 16 + (0..7 | 8..15) x value columns n * 16 + (0..7 | 8..15)
          const int key = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, colo = (lane >> 4) * 8;
#pragma unroll
          for (int n = 0; n < WP / 16; ++n) {
            uint32_t b0, b1, b2, b3;
            ldsm_x4_t(static_cast<uint32_t>(__cvta_generic_to_shared(vh + key * LD + n * 16 + colo)), b0, b1, b2, b3);
            mma_bf16(oacc[i][2 * n], h0, h1, h2, h3, b0, b1);
            mma_bf16(oacc[i][2 * n], l0, l1, l2, l3, b0, b1);
            mma_bf16(oacc[i][2 * n + 1], h0, h1, h2, h3, b2, b3);
            mma_bf16(oacc[i][2 * n + 1], l0, l1, l2, l3, b2, b3);
          }
        }
      }
    }
    __syncthreads();         // V's buffer and the raw scores are free
    if (jt + 1 < n_tiles) load_rows_async<WP, TT_THREADS>(Vs, Vg, static_cast<long long>(p.cap) * VS, VS, G, BN, j0 + BN, n_ctx, V);
    cp_async_commit();
  }
  cp_async_wait<0>();
  // ---- O / l, the element-wise gate, store
  __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out) + static_cast<long long>(off + q0) * H * V;
  const __nv_bfloat16* gate = p.out_gate ? static_cast<const __nv_bfloat16*>(p.out_gate) + static_cast<long long>(off + q0) * p.out_gate_stride : nullptr;
#pragma unroll
  for (int i = 0; i < HPW; ++i) {
    const int h = warp * HPW + i;
    if (h < H) {
      const float inv_a = lrow[i][0] > 0.f ? 1.f / lrow[i][0] : 0.f, inv_b = lrow[i][1] > 0.f ? 1.f / lrow[i][1] : 0.f;
#pragma unroll
      for (int n = 0; n < WP / 8; ++n) {
        const int c = n * 8 + 2 * tq;
        if (c < V) {   // V is a multiple of 8: the pair (c, c + 1) lies inside
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int r = gq + half * 8;
            if (r < rows) {
              float v0 = oacc[i][n][2 * half] * (half ? inv_b : inv_a), v1 = oacc[i][n][2 * half + 1] * (half ? inv_b : inv_a);
              const long long o = static_cast<long long>(r) * H * V + h * V + c;
              if (gate) {
                const __nv_bfloat162 gv = *reinterpret_cast<const __nv_bfloat162*>(gate + static_cast<long long>(r) * p.out_gate_stride + h * V + c);
                v0 *= sigmoidf_(__bfloat162float(gv.x));
                v1 *= sigmoidf_(__bfloat162float(gv.y));
              }
              *reinterpret_cast<__nv_bfloat162*>(out + o) = __floats2bfloat162_rn(v0, v1);
            }
          }
        }
      }
    }
  }
}

template <int WP, int HPW, int BN, int NW, int MINB>
int launch_one(const pcs_attn_params& p, cudaStream_t st, size_t smem) {
  static bool configured = false;
  if (!configured) {
    PCS_CHECK_CUDA(cudaFuncSetAttribute(attn_talk_tc_kernel<WP, HPW, BN, NW, MINB>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    configured = true;
  }
  const int n_qtiles = (p.max_len + TT_BM - 1) / TT_BM;
  attn_talk_tc_kernel<WP, HPW, BN, NW, MINB><<<p.n_seqs * n_qtiles, NW * 32, smem, st>>>(p);
  PCS_CHECK_CUDA(cudaGetLastError());
  count_launch();
  return PCS_OK;
}

size_t talk_tc_smem(int H, int G, int WP, int BN) {
  const size_t LD = WP + TT_PAD;
  return (static_cast<size_t>(H) * TT_BM + 2 * static_cast<size_t>(G) * BN) * LD * 2 + static_cast<size_t>(H) * TT_BM * (BN + 8) * 4 + static_cast<size_t>(16) * H * 4;
}

}  // namespace

int launch_attn_talk_tc(const pcs_attn_params& p, cudaStream_t st, bool* handled) {
  *handled = false;
  auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  const int wmax = p.dim > p.vdim ? p.dim : p.vdim;
  const bool fits = p.dtype == PCS_BF16 && p.max_len >= 16 && p.n_heads <= 16 && p.dim % 8 == 0 && p.vdim % 8 == 0 && wmax <= 128 && p.keep_first == 0 &&
                    p.seq_len && p.seq_off && p.seq_pos0 && p.n_seqs > 0 && al(p.q) && al(p.k_pool) && al(p.v_pool) && al(p.out) &&
                    (p.v_row_stride == 0 || p.v_row_stride % 8 == 0) &&
                    (p.out_gate == nullptr || ((reinterpret_cast<uintptr_t>(p.out_gate) & 3) == 0 && p.out_gate_stride % 2 == 0));
  if (!fits) return PCS_OK;
  // 8 warps; up to 8 heads one head per warp, up to 16 two; tiles of 64 keys where the shared memory allows, else 32.  (Measured
  // alternatives that were not faster at 8 / 16 heads of 128, also with thousands of blocks: two blocks per SM at 128 registers and
  // 32-key tiles, 16 warps with one head each.)
  const int WP = wmax <= 64 ? 64 : 128, HPW = p.n_heads <= 8 ? 1 : 2;
  const size_t limit = 220 * 1024;
  int BN = 64;
  if (talk_tc_smem(p.n_heads, p.n_kv_heads, WP, 64) > limit) BN = 32;
  const size_t smem = talk_tc_smem(p.n_heads, p.n_kv_heads, WP, BN);
  if (smem > limit) return PCS_OK;
  *handled = true;
#define PCS_TT(W_, H_, B_) if (WP == W_ && HPW == H_ && BN == B_) return launch_one<W_, H_, B_, 8, 1>(p, st, smem)
  PCS_TT(64, 1, 64); PCS_TT(64, 2, 64); PCS_TT(128, 1, 64); PCS_TT(128, 2, 64);
  PCS_TT(64, 1, 32); PCS_TT(64, 2, 32); PCS_TT(128, 1, 32); PCS_TT(128, 2, 32);
#undef PCS_TT
  *handled = false;
  return PCS_OK;
}

}  // namespace pcs
