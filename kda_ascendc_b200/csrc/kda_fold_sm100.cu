// Fold of per-segment affine state transforms: the exchange step of the sequence split.  sm_100a.
//
// A contiguous segment of chunks maps the state that enters it to the state that leaves it as
//   S_out = S_in * M_seg + Q_seg          S: [V=128][K=128] fp32,  M_seg: [K][K],  Q_seg: [V][K]
// (the reference only analyses this route: tools/probe_segment_affine.py:100-125 of the reference
// project; M_seg and Q_seg come from two state-only K2 passes over the segment's records).  With the
// transforms of all segments of a chain in local memory this kernel walks them in order,
//   S = h0;  for j = 0 .. n_seg-1:  s_in[j] = S;  S = S * M_j + Q_j;      s_in[n_seg] = S
// and leaves the entry state of every segment plus the state after the last one.
//
// The rows of S are independent (row v of S_out needs row v of S_in only), so a CTA owns four rows
// of one chain for the whole walk: thread t owns column t of those rows, the rows sit in shared
// memory (double-buffered, one barrier per segment), and M_j streams through L2 as 128 coalesced
// 512-byte row reads per warp with sixteen loads in flight.  Plain fp32 FMAs: the entry states feed
// a recurrence whose parity bound is 2e-3 absolute, so no reduced-precision tensor-core path here.
// 32 CTAs per chain; the walk is latency-bound (one pass over 64 KiB of M_j per segment and CTA).
#include "../../include/kda_b200.h"
#include "kda_common.cuh"
#include "kda_kernels.h"

namespace kda {

constexpr int FOLD_ROWS = 4;

__global__ void __launch_bounds__(D, 4)
kda_state_fold_kernel(const float* __restrict__ mq, long long seg_stride, long long chain_stride,
                      const float* __restrict__ h0, float* __restrict__ s_in, int n_chains, int n_seg) {
  __shared__ __align__(16) float sS[2][FOLD_ROWS][D];
  const int t = threadIdx.x;
  const int chain = blockIdx.x / (D / FOLD_ROWS);
  const int r0 = (blockIdx.x % (D / FOLD_ROWS)) * FOLD_ROWS;
  const size_t state_elems = static_cast<size_t>(D) * D;
  float s[FOLD_ROWS];
#pragma unroll
  for (int r = 0; r < FOLD_ROWS; ++r)
    s[r] = (h0 != nullptr) ? h0[chain * state_elems + static_cast<size_t>(r0 + r) * D + t] : 0.f;

  int buf = 0;
  for (int j = 0; j < n_seg; ++j) {
    float* out = s_in + (static_cast<size_t>(j) * n_chains + chain) * state_elems;
#pragma unroll
    for (int r = 0; r < FOLD_ROWS; ++r) {
      out[static_cast<size_t>(r0 + r) * D + t] = s[r];
      sS[buf][r][t] = s[r];
    }
    __syncthreads();   // the rows of S are complete; the other buffer is free for the next segment
    const float* M = mq + static_cast<size_t>(j) * seg_stride + static_cast<size_t>(chain) * chain_stride;
    const float* Q = M + state_elems;
    float acc[FOLD_ROWS];
#pragma unroll
    for (int r = 0; r < FOLD_ROWS; ++r) acc[r] = __ldg(Q + static_cast<size_t>(r0 + r) * D + t);
#pragma unroll 4
    for (int k0 = 0; k0 < D; k0 += 16) {
      float m[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) m[i] = __ldg(M + static_cast<size_t>(k0 + i) * D + t);
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
#pragma unroll
        for (int r = 0; r < FOLD_ROWS; ++r) {
          const float4 sv = *reinterpret_cast<const float4*>(&sS[buf][r][k0 + q4 * 4]);
          acc[r] = fmaf(sv.x, m[q4 * 4 + 0], acc[r]);
          acc[r] = fmaf(sv.y, m[q4 * 4 + 1], acc[r]);
          acc[r] = fmaf(sv.z, m[q4 * 4 + 2], acc[r]);
          acc[r] = fmaf(sv.w, m[q4 * 4 + 3], acc[r]);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < FOLD_ROWS; ++r) s[r] = acc[r];
    buf ^= 1;
  }
  float* out = s_in + (static_cast<size_t>(n_seg) * n_chains + chain) * state_elems;
#pragma unroll
  for (int r = 0; r < FOLD_ROWS; ++r) out[static_cast<size_t>(r0 + r) * D + t] = s[r];
}

cudaError_t launch_state_fold(const float* mq, long long seg_stride, long long chain_stride, const float* h0,
                              float* s_in, int n_chains, int n_seg, cudaStream_t stream) {
  kda_state_fold_kernel<<<n_chains * (D / FOLD_ROWS), D, 0, stream>>>(mq, seg_stride, chain_stride, h0, s_in, n_chains,
                                                                      n_seg);
  return cudaGetLastError();
}

}  // namespace kda
