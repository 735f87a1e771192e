// Peer-memory pieces of the sequence split's exchange.  sm_100a.
//
// The reference only analyses the segment route (tools/probe_segment_affine.py:100-125,
// docs/SEGMENT_SCAN_ROUTE_A_EVAL.md:92-118 of the reference project); there is no kernel to
// replace.  With the ranks of a box mapped into each other's address space, the all-to-all of
// the per-segment transforms is one copy kernel per rank -- slice d of the local transforms goes
// into rank d's receive buffer with plain 16-byte stores over NVLink, and a per-source flag in
// rank d's memory tells its fold kernel that the slice is complete -- and the way back (entry
// states) is written by the fold kernel itself (kda_fold_sm100.cu).  No multicast, no TMA on
// peer memory; received data lands in the receiver's own memory before anything reads it.
#include "kda_common.cuh"
#include "kda_kernels.h"

namespace kda {

namespace {
constexpr int PUSH_THREADS = 256;
constexpr int PUSH_CTAS_PER_DST = 16;

__global__ void __launch_bounds__(PUSH_THREADS) kda_peer_push_kernel(const PeerPushParams p) {
  const int d = blockIdx.x / PUSH_CTAS_PER_DST, part = blockIdx.x % PUSH_CTAS_PER_DST;
  const float4* __restrict__ src = p.src + static_cast<long long>(d) * p.slice;
  float4* __restrict__ dst = p.dst[d] + p.dst_offset;
  const long long step = static_cast<long long>(PUSH_CTAS_PER_DST) * PUSH_THREADS;
  long long i = static_cast<long long>(part) * PUSH_THREADS + threadIdx.x;
  for (; i + 3 * step < p.slice; i += 4 * step) {   // four independent 16-byte copies in flight per thread
    const float4 a = src[i], b = src[i + step], c = src[i + 2 * step], e = src[i + 3 * step];
    dst[i] = a; dst[i + step] = b; dst[i + 2 * step] = c; dst[i + 3 * step] = e;
  }
  for (; i < p.slice; i += step) dst[i] = src[i];
  // the slice is complete once every CTA that copies part of it has fenced its stores
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int done = atomicAdd(p.counter + d, 1);
    __threadfence();
    if (done == PUSH_CTAS_PER_DST - 1) {
      p.counter[d] = 0;
      __threadfence_system();
      st_release_sys(p.flag[d], p.epoch);
    }
  }
}

__global__ void kda_flag_wait_kernel(const int* flags, int n, int epoch, int* status) {
  const int i = threadIdx.x;
  if (i < n && !flag_wait_bounded(flags + i, epoch) && status != nullptr) atomicExch(status, ST_PEER_TIMEOUT);
}
}  // namespace

cudaError_t launch_peer_push(const PeerPushParams& p, cudaStream_t stream) {
  kda_peer_push_kernel<<<p.world * PUSH_CTAS_PER_DST, PUSH_THREADS, 0, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_flag_wait(const int* flags, int n, int epoch, int* status, cudaStream_t stream) {
  kda_flag_wait_kernel<<<1, 32, 0, stream>>>(flags, n, epoch, status);
  return cudaGetLastError();
}

}  // namespace kda
