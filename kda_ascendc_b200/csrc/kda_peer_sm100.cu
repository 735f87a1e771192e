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
constexpr int PUSH_THREADS = 512;
constexpr int PUSH_UNROLL = 8;   // independent 16-byte copies in flight per thread

// grid = world x ctas_per_dst: CTA (d, part) copies a contiguous part of slice d
__global__ void __launch_bounds__(PUSH_THREADS) kda_peer_push_kernel(const PeerPushParams p) {
  const int cpd = p.ctas_per_dst;
  const int d = blockIdx.x / cpd, part = blockIdx.x % cpd;
  const float4* __restrict__ src = p.src + static_cast<long long>(d) * p.slice;
  float4* __restrict__ dst = p.dst[d] + p.dst_offset;
  const long long per = (p.slice + cpd - 1) / cpd;
  const long long begin = per * part, end = (begin + per < p.slice) ? begin + per : p.slice;
  for (long long i = begin + threadIdx.x; i < end; i += static_cast<long long>(PUSH_UNROLL) * PUSH_THREADS) {
    float4 v[PUSH_UNROLL];
#pragma unroll
    for (int u = 0; u < PUSH_UNROLL; ++u)
      if (i + static_cast<long long>(u) * PUSH_THREADS < end) v[u] = src[i + static_cast<long long>(u) * PUSH_THREADS];
#pragma unroll
    for (int u = 0; u < PUSH_UNROLL; ++u)
      if (i + static_cast<long long>(u) * PUSH_THREADS < end) dst[i + static_cast<long long>(u) * PUSH_THREADS] = v[u];
  }
  // The slice is complete once every CTA that copies part of it has counted itself.  Ordering: the CTA
  // barrier puts every thread's stores before thread 0's device-scope fence and count; the CTA that counts
  // last has thereby observed all of them and raises the flag behind ONE system-scope fence (a system-scope
  // fence costs microseconds: with one in every CTA a 16-byte push measured 16 us against 9 us for an empty
  // launch between the same two events).
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const int done = atomicAdd(p.counter + d, 1);
    __threadfence();
    if (done == cpd - 1) {
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

cudaError_t launch_peer_push(const PeerPushParams& p0, cudaStream_t stream) {
  // Stores over NVLink are limited per SM, not per link: spread every slice over as many CTAs as fill the GPU
  // about twice (measured at four ranks x 1 MB per slice: 64 CTAs of 256 threads 24 us; see the header comment)
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  PeerPushParams p = p0;
  long long cpd = (2LL * sms) / p.world;
  const long long most = (p.slice + PUSH_THREADS - 1) / PUSH_THREADS;   // at least one 16-byte unit per thread
  if (cpd > most) cpd = most;
  if (cpd < 1) cpd = 1;
  if (cpd > 128) cpd = 128;
  p.ctas_per_dst = static_cast<int>(cpd);
  kda_peer_push_kernel<<<p.world * p.ctas_per_dst, PUSH_THREADS, 0, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_flag_wait(const int* flags, int n, int epoch, int* status, cudaStream_t stream) {
  kda_flag_wait_kernel<<<1, 32, 0, stream>>>(flags, n, epoch, status);
  return cudaGetLastError();
}

}  // namespace kda
