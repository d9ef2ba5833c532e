// Mixture of experts for many rows (prompts, bfloat16): rows sorted by expert, then two grouped tensor-core products.
//
// pcs_moe_plan   one block: counts the (token, choice) pairs of every expert, lays the experts' rows out one after the other,
//                cuts them into tiles of 128 rows that never straddle two experts, and writes the experts' cumulative row
//                ends, the sorted pair list and every pair's sorted row.  Pairs whose choice is a pass-through output take no row.
// pcs_moe_gather copies the rows the sorted pairs read into one matrix, for a library's grouped product.  Everything stays on the device: the products below
//                are launched for the largest possible number of tiles and blocks past the real number return at once.
// pcs_moe_gemm   block = (row tile of 128, 128 rows of the expert's matrix), 8 warps of 32 x 64, K in steps of 32 through four
//                cp.async stages (one barrier per step), ldmatrix + m16n8k16 bfloat16 products with 32-bit accumulators.
//                  stage 0: rows gathered from h by pair; 64 gate and the 64 matching up features of the tile's expert side by
//                           side, so that a thread holds both halves of its outputs and the epilogue writes silu(gate) * up
//                           in the sorted order (bfloat16);
//                  stage 1: rows of that matrix times the expert's down matrix, written 32-bit to the PAIR's row, so the
//                           weighted sum afterwards runs in the order of the choices whatever the sort did.
//                A row's sums depend on K alone, not on where the sort placed it or on what else is in the batch.
#include "seq_common.cuh"
#include "seq_mma.cuh"

namespace pcs {

namespace {

constexpr int GM = 128, GN = 128, GK = 32, GPAD = 8, G_THREADS = 256, G_STAGES = 4;
constexpr size_t G_SMEM = static_cast<size_t>(G_STAGES) * 2 * GM * (GK + GPAD) * sizeof(__nv_bfloat16);
constexpr int kPlanMaxExperts = 1024;

__host__ __device__ inline int plan_max_tiles(int n_pairs, int n_experts) { return (n_pairs + GM - 1) / GM + n_experts; }
// the plan's parts (int32 offsets): [0] tiles in use; the experts' cumulative row ends; the tiles; the sorted pairs; the
// pairs' sorted rows
__host__ __device__ inline int plan_ends(int, int) { return 4; }
__host__ __device__ inline int plan_tiles(int, int E) { return 4 + (E + 3) / 4 * 4; }
__host__ __device__ inline int plan_sorted(int P, int E) { return plan_tiles(P, E) + 3 * plan_max_tiles(P, E); }
__host__ __device__ inline int plan_rows(int P, int E) { return plan_sorted(P, E) + P; }
__host__ __device__ inline int plan_total(int P, int E) { return plan_rows(P, E) + P; }

__global__ void __launch_bounds__(1024) moe_plan_kernel(const int32_t* __restrict__ idx, int n_pairs, int E, int32_t* __restrict__ plan) {
  __shared__ int cnt[kPlanMaxExperts];
  __shared__ int cur[kPlanMaxExperts];
  int32_t* ends = plan + plan_ends(n_pairs, E);
  int32_t* tiles = plan + plan_tiles(n_pairs, E);
  int32_t* sorted = plan + plan_sorted(n_pairs, E);
  int32_t* row_of = plan + plan_rows(n_pairs, E);
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = idx[p];
    if (e >= 0 && e < E) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0, nt = 0;
    for (int e = 0; e < E; ++e) {
      cur[e] = off;
      for (int r0 = 0; r0 < cnt[e]; r0 += GM) {
        tiles[3 * nt] = e;
        tiles[3 * nt + 1] = off + r0;
        tiles[3 * nt + 2] = min(GM, cnt[e] - r0);
        ++nt;
      }
      off += cnt[e];
      ends[e] = off;
    }
    plan[0] = nt;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = idx[p];
    int r = -1;
    if (e >= 0 && e < E) {
      r = atomicAdd(&cur[e], 1);
      sorted[r] = p;
    }
    row_of[p] = r;
  }
}

// sorted row r of `out` = the row of h that pair sorted[r] reads (16-byte pieces); rows past the last expert's end are left alone
__global__ void __launch_bounds__(128) moe_gather_kernel(const uint4* __restrict__ h, long long h_stride16, const int32_t* __restrict__ plan,
                                                         uint4* __restrict__ out, int n_pairs, int top, int E, int pieces) {
  const int r = blockIdx.x;
  if (r >= plan[plan_ends(n_pairs, E) + E - 1]) return;
  const int pr = plan[plan_sorted(n_pairs, E) + r];
  const uint4* src = h + static_cast<long long>(pr / top) * h_stride16;
  uint4* dst = out + static_cast<long long>(r) * pieces;
  for (int i = threadIdx.x; i < pieces; i += 128) dst[i] = src[i];
}

// STAGE 0: A = h rows gathered by pair, B = 64 gate | 64 up rows of w_gu[e]; STAGE 1: A = act rows, B = 128 rows of w_down[e]
template <int STAGE>
__global__ void __launch_bounds__(G_THREADS, 2) moe_gemm_kernel(const __nv_bfloat16* __restrict__ a, long long a_stride, const __nv_bfloat16* __restrict__ w,
                                                                const int32_t* __restrict__ plan, void* __restrict__ out, int n_pairs, int top, int E,
                                                                int ff, int W, const GluAct glu) {
  constexpr int LD = GK + GPAD;                         // row length in shared memory
  constexpr int TILE = GM * LD;                         // elements of one A (or B) tile
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* sm = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // per stage: A tile, then B tile
  __shared__ int row_src[GM];
  const int tile = blockIdx.x;
  if (tile >= plan[0]) return;
  const int32_t* tl = plan + plan_tiles(n_pairs, E) + 3 * tile;
  const int e = tl[0], row0 = tl[1], rows = tl[2];
  const int32_t* sorted = plan + plan_sorted(n_pairs, E);
  const int K = STAGE == 0 ? W : ff, N = STAGE == 0 ? ff : W;
  const int n0 = blockIdx.y * (STAGE == 0 ? GN / 2 : GN);
  const __nv_bfloat16* wb = STAGE == 0 ? w + static_cast<long long>(e) * 2 * ff * W : w + static_cast<long long>(e) * W * ff;
  for (int r = threadIdx.x; r < GM; r += G_THREADS) row_src[r] = r < rows ? sorted[row0 + r] : -1;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wm = warp >> 1, wn = warp & 1, grp = lane >> 2, qd = lane & 3;

  // a thread copies the same pieces of the A tile and of the B tile at every K step (four neighbouring threads share a row's
  // 64 bytes): their sources are fixed
  constexpr int CH = GK / 8, PER = GM * CH / G_THREADS;
  const __nv_bfloat16* a_src[PER];
  const __nv_bfloat16* b_src[PER];
  int dst_off[PER], kc_of[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int c = threadIdx.x + i * G_THREADS, r = c / CH, kc = (c - r * CH) * 8;
    dst_off[i] = r * LD + kc;
    kc_of[i] = kc;
    const int pr = row_src[r];
    a_src[i] = pr < 0 ? nullptr : (STAGE == 0 ? a + static_cast<long long>(pr / top) * a_stride : a + static_cast<long long>(row0 + r) * a_stride) + kc;
    int n, wrow;
    if (STAGE == 0) { n = n0 + (r & 63); wrow = (r >> 6) * ff + n; } else { n = n0 + r; wrow = n; }
    b_src[i] = n < N ? wb + static_cast<long long>(wrow) * K + kc : nullptr;
  }
  auto load = [&](int st, int k0) {
    __nv_bfloat16* As = sm + st * 2 * TILE;
    __nv_bfloat16* Bs = As + TILE;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const bool in_k = k0 + kc_of[i] < K;
      if (a_src[i] && in_k) cp_async16(As + dst_off[i], a_src[i] + k0);
      else *reinterpret_cast<uint4*>(As + dst_off[i]) = make_uint4(0u, 0u, 0u, 0u);
      if (b_src[i] && in_k) cp_async16(Bs + dst_off[i], b_src[i] + k0);
      else *reinterpret_cast<uint4*>(Bs + dst_off[i]) = make_uint4(0u, 0u, 0u, 0u);
    }
  };

  float acc[2][8][4];  // [m tile][n tile]; stage 0: n tiles 0..3 gate, 4..7 up of the same 32 features
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;

  const int steps = (K + GK - 1) / GK;
#pragma unroll
  for (int s = 0; s < G_STAGES - 1; ++s) {
    if (s < steps) load(s, s * GK);
    cp_async_commit();
  }
  const uint32_t sm_base = static_cast<uint32_t>(__cvta_generic_to_shared(sm));
  const uint32_t a_off = ((wm * 32 + (lane & 15)) * LD + (lane >> 4) * 8) * 2;
  uint32_t b_off[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int brow = STAGE == 0 ? (j >> 2) * 64 + wn * 32 + (j & 3) * 8 : wn * 64 + j * 8;
    b_off[j] = (TILE + (brow + (lane & 7)) * LD + (lane >> 3) * 8) * 2;
  }
  for (int s = 0; s < steps; ++s) {
    cp_async_wait<G_STAGES - 2>();
    __syncthreads();  // step s has landed for every thread, and every warp is done with the stage that is refilled next
    if (s + G_STAGES - 1 < steps) load((s + G_STAGES - 1) % G_STAGES, (s + G_STAGES - 1) * GK);
    cp_async_commit();
    const uint32_t base = sm_base + (s % G_STAGES) * 2 * TILE * 2;
#pragma unroll
    for (int kp = 0; kp < GK / 32; ++kp) {  // 32 of the step's K at a time
      uint32_t af[2][2][4];  // [m tile][k16 step]
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int kk = 0; kk < 2; ++kk)
          ldsm_x4(base + a_off + (i * 16 * LD + kp * 32 + kk * 16) * 2, af[i][kk][0], af[i][kk][1], af[i][kk][2], af[i][kk][3]);
#pragma unroll
      for (int jh = 0; jh < 2; ++jh) {
        uint32_t bf[4][4];  // four n tiles: k 0..15 in [0],[1], k 16..31 in [2],[3]
#pragma unroll
        for (int j = 0; j < 4; ++j) ldsm_x4(base + b_off[jh * 4 + j] + kp * 64, bf[j][0], bf[j][1], bf[j][2], bf[j][3]);
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) mma_bf16(acc[i][jh * 4 + j], af[i][0][0], af[i][0][1], af[i][0][2], af[i][0][3], bf[j][0], bf[j][1]);
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) mma_bf16(acc[i][jh * 4 + j], af[i][1][0], af[i][1][1], af[i][1][2], af[i][1][3], bf[j][2], bf[j][3]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = wm * 32 + i * 16 + grp + half * 8;
      if (r >= rows) continue;
      if (STAGE == 0) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int n = n0 + wn * 32 + j * 8 + qd * 2;
          if (n >= N) continue;
          const float g0 = acc[i][j][half * 2], g1 = acc[i][j][half * 2 + 1];
          const float u0 = acc[i][4 + j][half * 2], u1 = acc[i][4 + j][half * 2 + 1];
          __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out) + static_cast<long long>(row0 + r) * ff + n;
          *reinterpret_cast<uint32_t*>(o) = pack_bf16(glu(g0, u0), glu(g1, u1));
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int n = n0 + wn * 64 + j * 8 + qd * 2;
          if (n >= N) continue;
          float* o = static_cast<float*>(out) + static_cast<long long>(row_src[r]) * W + n;
          *reinterpret_cast<float2*>(o) = make_float2(acc[i][j][half * 2], acc[i][j][half * 2 + 1]);
        }
      }
    }
}

}  // namespace
}  // namespace pcs

PCS_API int64_t pcs_moe_plan_ints(int n_pairs, int n_experts) {
  if (n_pairs <= 0 || n_experts <= 0) return 4;
  return pcs::plan_total(n_pairs, n_experts);
}

PCS_API int pcs_moe_plan(const int32_t* idx, int n_pairs, int n_experts, int32_t* plan, void* stream) {
  if (n_pairs == 0 || n_experts == 0) return PCS_OK;
  PCS_REQUIRE(idx && plan && n_pairs > 0 && n_experts > 0 && n_experts <= pcs::kPlanMaxExperts, "pcs_moe_plan: bad arguments (at most %d experts)",
              pcs::kPlanMaxExperts);
  pcs::moe_plan_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(idx, n_pairs, n_experts, plan);
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}

PCS_API int pcs_moe_plan_part(int part, int n_pairs, int n_experts) {
  switch (part) {
    case 0: return pcs::plan_ends(n_pairs, n_experts);
    case 1: return pcs::plan_tiles(n_pairs, n_experts);
    case 2: return pcs::plan_sorted(n_pairs, n_experts);
    case 3: return pcs::plan_rows(n_pairs, n_experts);
    default: return -1;
  }
}

PCS_API int pcs_moe_gather(const void* h, int64_t h_stride, const int32_t* plan, void* out, int n_pairs, int top, int n_experts, int width,
                           void* stream) {
  if (n_pairs == 0 || n_experts == 0) return PCS_OK;
  PCS_REQUIRE(h && plan && out && n_pairs > 0 && top > 0 && width > 0, "pcs_moe_gather: bad arguments");
  PCS_REQUIRE(width % 8 == 0 && h_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(h) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0,
              "pcs_moe_gather: bfloat16 rows in 16-byte pieces");
  pcs::moe_gather_kernel<<<n_pairs, 128, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint4*>(h), h_stride / 8, plan,
                                                                                static_cast<uint4*>(out), n_pairs, top, n_experts, width / 8);
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}

PCS_API int pcs_moe_gemm(int stage, const void* a, int64_t a_stride, const void* w, const int32_t* plan, void* out, int n_pairs, int top,
                         int n_experts, int ff, int width, const pcs_glu_act* glu, void* stream) {
  if (n_pairs == 0 || n_experts == 0) return PCS_OK;
  PCS_REQUIRE(a && w && plan && out && n_pairs > 0 && top > 0 && ff > 0 && width > 0 && (stage == 0 || stage == 1), "pcs_moe_gemm: bad arguments");
  PCS_REQUIRE(ff % 8 == 0 && width % 8 == 0 && a_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(a) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0,
              "pcs_moe_gemm: sizes, the row stride and the pointers must be multiples of 16 bytes");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int per_block = stage == 0 ? pcs::GN / 2 : pcs::GN;  // output features of one block
  dim3 grid(pcs::plan_max_tiles(n_pairs, n_experts), ((stage == 0 ? ff : width) + per_block - 1) / per_block);
  static bool configured = false;
  if (!configured) {
    PCS_CHECK_CUDA(cudaFuncSetAttribute(pcs::moe_gemm_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(pcs::G_SMEM)));
    PCS_CHECK_CUDA(cudaFuncSetAttribute(pcs::moe_gemm_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(pcs::G_SMEM)));
    configured = true;
  }
  PCS_REQUIRE(grid.y <= 65535, "pcs_moe_gemm: too many output features");
  const pcs::GluAct act(glu);
  if (!act.gated()) return pcs::set_error(PCS_ERR_UNSUPPORTED, "pcs_moe_gemm: experts without a gate branch (activation %d) take the row kernels or the library's grouped product", act.kind);
  const __nv_bfloat16* ap = static_cast<const __nv_bfloat16*>(a);
  const __nv_bfloat16* wp = static_cast<const __nv_bfloat16*>(w);
  if (stage == 0) pcs::moe_gemm_kernel<0><<<grid, pcs::G_THREADS, pcs::G_SMEM, st>>>(ap, a_stride, wp, plan, out, n_pairs, top, n_experts, ff, width, act);
  else pcs::moe_gemm_kernel<1><<<grid, pcs::G_THREADS, pcs::G_SMEM, st>>>(ap, a_stride, wp, plan, out, n_pairs, top, n_experts, ff, width, act);
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}
