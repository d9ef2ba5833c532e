// Element-wise gated recurrence whose gates read only the current token (a "minimal" gated recurrent unit):
//     z_t = sigmoid(pz_t),  c_t = u_t >= 0 ? u_t + 1/2 : sigmoid(u_t),  S_t = (1 - z_t) S_(t-1) + z_t c_t,  out_t = S_t * silu(g_t)
// where pz, u and g are projections of the layer's input (biases already added).  Because neither z nor c depends on the state,
// every step is an affine map S -> a S + b with a = 1 - z, b = z c, and maps compose: a stretch of tokens is one pair (A, B).
//
// One block = 16 neighbouring channels of one batch entry x up to 64 segments of the entry's tokens (16 x segments threads;
// the launch picks the number of segments from the longest entry, so that a segment holds at least 16 tokens).
//   pass 1   every thread folds its segment into (A, B), starting from the identity;
//   join     the segments' pairs meet in shared memory; a thread's true start state is the entry's state (the slot pool's, or
//            zero for an entry whose slot holds no tokens) carried through the segments before its own, in order;
//   pass 2   the segment is walked again from that state and the gated result is written (its inputs come from L1 / L2).
// Both passes take eight tokens at a time: their loads are issued together, then the eight dependent updates follow.  The first
// segment's threads carry the state through all segments and store it for the next step.  A decoding step is the case of one
// token and one segment.  State, gates and candidates are 32-bit in both types; a channel's loads of neighbouring threads are
// neighbouring elements.
#include "seq_common.cuh"

namespace pcs {

constexpr int kGruMaxSegs = 64, kGruChannels = 16, kGruUnroll = 8;

__device__ __forceinline__ void gru_step(float pz, float u, float& a, float& b) {
  const float z = sigmoidf_(pz);
  const float c = u >= 0.f ? u + 0.5f : sigmoidf_(u);
  a = 1.f - z;
  b = z * c;
}

template <typename T>
__global__ void __launch_bounds__(kGruChannels * kGruMaxSegs) gru_scan_kernel(const pcs_gru_params p) {
  __shared__ float As[kGruMaxSegs][kGruChannels], Bs[kGruMaxSegs][kGruChannels];
  const int lane = threadIdx.x, seg = threadIdx.y, n_segs = blockDim.y, b = blockIdx.y;
  const int c = blockIdx.x * kGruChannels + lane;
  const int len = p.seq_len[b], off = p.seq_off[b], pos0 = p.seq_pos0[b], slot = p.seq_slot[b];
  const int per = (len + n_segs - 1) / n_segs;
  const int t0 = min(len, seg * per), t1 = min(len, t0 + per);
  const bool live = c < p.width;
  const long long rs = p.row_stride;
  const T* base = static_cast<const T*>(p.proj) + static_cast<long long>(off) * rs + (live ? c : 0);
  float A = 1.f, B = 0.f;
  if (live && n_segs > 1) {   // (one segment: nothing to fold ahead of pass 2)
    int t = t0;
    for (; t + kGruUnroll <= t1; t += kGruUnroll) {
      float pz[kGruUnroll], u[kGruUnroll];
#pragma unroll
      for (int i = 0; i < kGruUnroll; ++i) {
        const T* row = base + static_cast<long long>(t + i) * rs;
        pz[i] = ldf(row + p.z_off);
        u[i] = ldf(row + p.x_off);
      }
#pragma unroll
      for (int i = 0; i < kGruUnroll; ++i) {
        float a, bb;
        gru_step(pz[i], u[i], a, bb);
        A *= a;
        B = fmaf(a, B, bb);
      }
    }
    for (; t < t1; ++t) {
      const T* row = base + static_cast<long long>(t) * rs;
      float a, bb;
      gru_step(ldf(row + p.z_off), ldf(row + p.x_off), a, bb);
      A *= a;
      B = fmaf(a, B, bb);
    }
  }
  As[seg][lane] = A;
  Bs[seg][lane] = B;
  __syncthreads();
  if (!live) return;
  float* state = p.s_pool + static_cast<long long>(slot) * p.width + c;
  float S = pos0 > 0 ? *state : 0.f;
  for (int s = 0; s < seg; ++s) S = fmaf(As[s][lane], S, Bs[s][lane]);
  T* out = static_cast<T*>(p.out) + static_cast<long long>(off) * p.width + c;
  int t = t0;
  for (; t + kGruUnroll <= t1; t += kGruUnroll) {
    float pz[kGruUnroll], u[kGruUnroll], g[kGruUnroll];
#pragma unroll
    for (int i = 0; i < kGruUnroll; ++i) {
      const T* row = base + static_cast<long long>(t + i) * rs;
      pz[i] = ldf(row + p.z_off);
      u[i] = ldf(row + p.x_off);
      g[i] = ldf(row + p.g_off);
    }
#pragma unroll
    for (int i = 0; i < kGruUnroll; ++i) {
      float a, bb;
      gru_step(pz[i], u[i], a, bb);
      S = fmaf(a, S, bb);
      stf(out + static_cast<long long>(t + i) * p.width, S * (g[i] * sigmoidf_(g[i])));
    }
  }
  for (; t < t1; ++t) {
    const T* row = base + static_cast<long long>(t) * rs;
    float a, bb;
    gru_step(ldf(row + p.z_off), ldf(row + p.x_off), a, bb);
    S = fmaf(a, S, bb);
    const float g = ldf(row + p.g_off);
    stf(out + static_cast<long long>(t) * p.width, S * (g * sigmoidf_(g)));
  }
  if (seg == 0) {   // the state after the entry's last token: through the other segments' pairs
    for (int s = 1; s < n_segs; ++s) S = fmaf(As[s][lane], S, Bs[s][lane]);
    *state = S;
  }
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
  dim3 grid((p->width + pcs::kGruChannels - 1) / pcs::kGruChannels, p->n_seqs), block(pcs::kGruChannels, segs);
  PCS_DISPATCH(p->dtype, pcs::gru_scan_kernel<T><<<grid, block, 0, st>>>(*p));
  PCS_CHECK_CUDA(cudaGetLastError());
  pcs::count_launch();
  return PCS_OK;
}
