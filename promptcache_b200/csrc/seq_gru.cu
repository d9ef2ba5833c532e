// Element-wise gated recurrence whose gates read only the current token (a "minimal" gated recurrent unit):
//     z_t = sigmoid(pz_t),  c_t = u_t >= 0 ? u_t + 1/2 : sigmoid(u_t),  S_t = (1 - z_t) S_(t-1) + z_t c_t,  out_t = S_t * silu(g_t)
// where pz, u and g are projections of the layer's input (biases already added).  Because neither z nor c depends on the state,
// every step is an affine map S -> a S + b with a = 1 - z, b = z c, and maps compose: a stretch of tokens is one pair (A, B).
//
// One block = a few neighbouring channels of one batch entry x up to 64 segments of the entry's tokens; a thread owns one channel
// of one segment, at most 32 tokens at a time (a longer entry is walked in stretches of segments x 32 tokens, the state carried
// from stretch to stretch).
//   fold     a thread reads its tokens' gate and candidate inputs ONCE (sixteen tokens' loads are issued together) and keeps, for
//            every token i of its segment, the composed map of the segment up to and including i, (A_i, B_i), in registers;
//   join     the segments' whole maps meet in shared memory; every thread carries the state at the stretch's start through the
//            segments in order, notes the state at its own segment's start, and ends with the state after the stretch;
//   write    S_i = A_i S_start + B_i for every token: no chain is left, only the gate input is read.
// A prompt of 2048 tokens is 32 dependent steps and one read of its inputs.  A decoding step is the case of one token and one
// segment.  State, gates and candidates are 32-bit in both types; neighbouring threads load neighbouring elements.
#include <type_traits>

#include "seq_common.cuh"

namespace pcs {

constexpr int kGruMaxSegs = 64, kGruPer = 32, kGruUnroll = 16, kGruThreads = 512, kGruSMs = 148;

// float32 runs take the library's exponential and a true division; bfloat16 runs the hardware's base-2 exponential and
// reciprocal (a relative error near 2^-22, in 32-bit all the same): the scan is bound by instruction issue, not by bytes
template <bool kFast>
__device__ __forceinline__ float gru_sigmoid(float z) {
  if constexpr (kFast) return __fdividef(1.f, 1.f + __expf(-z));
  else return sigmoidf_(z);
}

template <bool kFast>
__device__ __forceinline__ void gru_step(float pz, float u, float& a, float& b) {
  const float z = gru_sigmoid<kFast>(pz);
  const float c = u >= 0.f ? u + 0.5f : gru_sigmoid<kFast>(u);
  a = 1.f - z;
  b = z * c;
}

template <typename T>
__global__ void __launch_bounds__(kGruThreads) gru_scan_kernel(const pcs_gru_params p) {
  __shared__ float As[kGruThreads], Bs[kGruThreads];
  constexpr bool kFast = !std::is_same<T, float>::value;
  const int lane = threadIdx.x, ch = blockDim.x, seg = threadIdx.y, n_segs = blockDim.y, b = blockIdx.y;
  const int c = blockIdx.x * ch + lane;
  const int len = p.seq_len[b], off = p.seq_off[b], pos0 = p.seq_pos0[b], slot = p.seq_slot[b];
  int per = (len + n_segs - 1) / n_segs;   // tokens of a segment in one stretch; stretches of equal size
  if (per > kGruPer) per = (per + (per + kGruPer - 1) / kGruPer - 1) / ((per + kGruPer - 1) / kGruPer);
  const int stretch = per * n_segs;
  const bool live = c < p.width;
  const long long rs = p.row_stride;
  const T* base = static_cast<const T*>(p.proj) + static_cast<long long>(off) * rs + (live ? c : 0);
  T* out = static_cast<T*>(p.out) + static_cast<long long>(off) * p.width + (live ? c : 0);
  float* state = p.s_pool + static_cast<long long>(slot) * p.width + (live ? c : 0);
  float S = (live && pos0 > 0) ? *state : 0.f;   // the state at the start of the stretch
  for (int s0 = 0; s0 < len; s0 += stretch) {
    const int t0 = min(len, s0 + seg * per), n = min(len, t0 + per) - t0;
    float Ap[kGruPer], Bp[kGruPer];
    float A = 1.f, B = 0.f;
#pragma unroll
    for (int j = 0; j < kGruPer; j += kGruUnroll) {
      if (j < n) {
        float pz[kGruUnroll], u[kGruUnroll];
#pragma unroll
        for (int i = 0; i < kGruUnroll; ++i) {
          const T* row = base + static_cast<long long>(t0 + min(j + i, n - 1)) * rs;
          pz[i] = ldf(row + p.z_off);
          u[i] = ldf(row + p.x_off);
        }
#pragma unroll
        for (int i = 0; i < kGruUnroll; ++i) {
          if (j + i < n) {
            float a, bb;
            gru_step<kFast>(pz[i], u[i], a, bb);
            A *= a;
            B = fmaf(a, B, bb);
            Ap[j + i] = A;
            Bp[j + i] = B;
          }
        }
      }
    }
    As[seg * ch + lane] = A;
    Bs[seg * ch + lane] = B;
    __syncthreads();
    float mine = S;
    for (int s = 0; s < n_segs; ++s) {
      if (s == seg) mine = S;
      S = fmaf(As[s * ch + lane], S, Bs[s * ch + lane]);
    }
    if (live) {
#pragma unroll
      for (int j = 0; j < kGruPer; j += kGruUnroll) {
        if (j < n) {
          float g[kGruUnroll];
#pragma unroll
          for (int i = 0; i < kGruUnroll; ++i) g[i] = ldf(base + static_cast<long long>(t0 + min(j + i, n - 1)) * rs + p.g_off);
#pragma unroll
          for (int i = 0; i < kGruUnroll; ++i)
            if (j + i < n) stf(out + static_cast<long long>(t0 + j + i) * p.width, fmaf(Ap[j + i], mine, Bp[j + i]) * (g[i] * gru_sigmoid<kFast>(g[i])));
        }
      }
    }
    __syncthreads();   // the next stretch overwrites the segments' maps
  }
  if (live && seg == 0 && len > 0) *state = S;
}

}  // namespace pcs

PCS_API int pcs_gru_scan(const pcs_gru_params* p, void* stream) {
  PCS_REQUIRE(p, "pcs_gru_scan: null params");
  if (p->n_seqs == 0 || p->n_tokens == 0) return PCS_OK;
  PCS_REQUIRE(p->proj && p->out && p->s_pool && p->seq_slot && p->seq_pos0 && p->seq_len && p->seq_off, "pcs_gru_scan: null tensor");
  PCS_REQUIRE(p->width > 0 && p->z_off >= 0 && p->x_off >= 0 && p->g_off >= 0 && p->n_seqs <= 65535, "pcs_gru_scan: bad sizes");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int segs = 1;   // a segment holds at least 16 tokens of the longest entry
  while (segs < pcs::kGruMaxSegs && p->max_len >= 32 * segs) segs *= 2;
  int ch = pcs::kGruThreads / segs;   // channels of a block: a warp's worth for short steps
  if (ch > 32) ch = 32;
  if (segs == pcs::kGruMaxSegs) {
    // long prompts: the launch is bound by instruction issue, so what counts is how evenly the blocks (one resident per SM) fill
    // the SMs: the channel count with the fewest rounds of blocks x channels per block; more channels mean fewer segments and
    // more stretches, which costs little beside that
    long long best = -1;
    for (int c = 6; c <= 32; ++c) {
      const long long blocks = static_cast<long long>((p->width + c - 1) / c) * p->n_seqs;
      const long long cost = ((blocks + pcs::kGruSMs - 1) / pcs::kGruSMs) * c;
      if (best < 0 || cost <= best) { best = cost; ch = c; }
    }
    segs = pcs::kGruThreads / ch;
    if (segs > pcs::kGruMaxSegs) segs = pcs::kGruMaxSegs;
  }
  dim3 grid((p->width + ch - 1) / ch, p->n_seqs), block(ch, segs);
  PCS_DISPATCH(p->dtype, pcs::gru_scan_kernel<T><<<grid, block, 0, st>>>(*p));
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}
