// Fold of per-segment affine state transforms: the exchange step of the sequence split.  sm_100a.
//
// A contiguous segment of chunks maps the state that enters it to the state that leaves it as
//   S_out = S_in * M_seg + Q_seg          S: [V=128][K=128] fp32,  M_seg: [K][K],  Q_seg: [V][K]
// (the reference only analyses this route: tools/probe_segment_affine.py:100-125 of the reference
// project; M_seg and Q_seg come from a state-only K2 pass over the segment's records).  With the
// transforms of all segments of a chain in local memory this kernel walks them in order,
//   S = h0;  for j = 0 .. n_seg-1:  s_in[j] = S;  S = S * M_j + Q_j;      s_in[n_seg] = S
// and leaves the entry state of every segment plus the state after the last one.
//
// The rows of S are independent (row v of S_out needs row v of S_in only), so a CTA owns ROWS rows
// of one chain for the whole walk: thread t owns column t of those rows and the rows sit in shared
// memory.  M_j (64 KiB) arrives by bulk (TMA) copies into a two-deep ring, so the copy of M_{j+1}
// runs under the products with M_j and the walk costs about one L2-to-shared copy per segment
// instead of 128 dependent global reads.  Plain fp32 FMAs: the entry states feed a recurrence whose
// parity bound is 2e-3 absolute, so there is no reduced-precision tensor-core path here.  ROWS is the
// smallest of 4, 8, 16 with which the CTAs (chains * 128 / ROWS, one per SM: the ring takes 128 KiB) fit one wave.
// Every wait is bounded and reports through the status word.
//
// Exchange over peer memory (FoldParams::wait_flags / s_in_seg / signal): when the transforms are
// stored into mq by the other GPUs of a sequence split, the walk first waits (bounded) for their
// flags, writes the entry state of segment j straight into rank j's buffer, and the last CTA to
// finish raises the flags that tell those ranks their entry states have arrived.
#include "../../include/kda_b200.h"
#include "kda_common.cuh"
#include "kda_kernels.h"

namespace kda {

constexpr int ST_FOLD_TIMEOUT = 5;
constexpr int FOLD_M_BYTES = D * D * 4;          // 65,536
constexpr int FOLD_PIECE = 16384;                // one bulk copy

template <int ROWS>
struct FoldSmem {
  static constexpr int M0 = 0;                               // two M buffers
  static constexpr int S = 2 * FOLD_M_BYTES;                 // fp32 [2][ROWS][128]: the CTA's rows of S
  static constexpr int BARS = S + 2 * ROWS * D * 4;          // full[2]
  static constexpr int FLAG = BARS + 16;
  static constexpr int TOTAL = FLAG + 16;
};

template <int ROWS>
__global__ void __launch_bounds__(D, 1)
kda_state_fold_kernel(const FoldParams p) {
  const float* __restrict__ mq = p.mq;
  const float* __restrict__ h0 = p.h0;
  float* __restrict__ s_in = p.s_in;
  const long long seg_stride = p.seg_stride, chain_stride = p.chain_stride;
  const int n_chains = p.n_chains, n_seg = p.n_seg;
  int* status = p.status;
  extern __shared__ __align__(1024) uint8_t smem[];
  using SM = FoldSmem<ROWS>;
  const int t = threadIdx.x;
  const int chain = blockIdx.x / (D / ROWS);
  const int r0 = (blockIdx.x % (D / ROWS)) * ROWS;
  const size_t state_elems = static_cast<size_t>(D) * D;
  const uint32_t sbase = smem_u32(smem);
  const uint32_t full0 = sbase + SM::BARS;
  volatile int* sAbort = reinterpret_cast<volatile int*>(smem + SM::FLAG);
  float (*sS)[ROWS][D] = reinterpret_cast<float (*)[ROWS][D]>(smem + SM::S);

  auto m_ptr = [&](int j) {
    return mq + static_cast<size_t>(j) * seg_stride + static_cast<size_t>(chain) * chain_stride;
  };
  auto issue = [&](int j) {   // thread 0: M_j into ring slot j & 1
    const uint32_t bar = full0 + (j & 1) * 8;
    mbar_arrive_expect_tx(bar, FOLD_M_BYTES);
    const uint8_t* src = reinterpret_cast<const uint8_t*>(m_ptr(j));
#pragma unroll
    for (int i = 0; i < FOLD_M_BYTES / FOLD_PIECE; ++i)
      bulk_g2s(sbase + SM::M0 + (j & 1) * FOLD_M_BYTES + i * FOLD_PIECE, src + i * FOLD_PIECE, FOLD_PIECE, bar);
  };

  if (t == 0) {
    mbar_init(full0, 1);
    mbar_init(full0 + 8, 1);
    *sAbort = 0;
    fence_mbar_init();
    // transforms stored by peers: wait for every source's flag before the first copy reads them
    for (int i = 0; i < p.n_wait; ++i)
      if (!flag_wait_bounded(p.wait_flags + i, p.epoch)) { *sAbort = 2; break; }
    if (*sAbort == 0) {
      if (p.n_wait > 0) fence_proxy_async();
      if (n_seg > 0) issue(0);
      if (n_seg > 1) issue(1);
    }
  }

  float s[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r)
    s[r] = (h0 != nullptr) ? h0[static_cast<size_t>(chain) * p.h0_stride + static_cast<size_t>(r0 + r) * D + t] : 0.f;
  __syncthreads();   // barriers initialised
  if (*sAbort == 2) {   // a peer's flag never came: nothing has been issued, report and leave
    if (t == 0 && status != nullptr) atomicExch(status, ST_PEER_TIMEOUT);
    return;
  }
  // where the state before segment j (j = n_seg: after the last one) of this chain goes, or null
  auto s_in_at = [&](int j) -> float* {
    if (p.s_in_seg_on) return p.s_in_seg[j] != nullptr ? p.s_in_seg[j] + static_cast<size_t>(chain) * state_elems : nullptr;
    return s_in != nullptr ? s_in + (static_cast<size_t>(j) * n_chains + chain) * state_elems : nullptr;
  };

  int issued = n_seg < 2 ? n_seg : 2;
  for (int j = 0; j < n_seg; ++j) {
    const float* Q = m_ptr(j) + state_elems;
    float* const sj = s_in_at(j);
    float acc[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      if (sj != nullptr) sj[static_cast<size_t>(r0 + r) * D + t] = s[r];
      sS[j & 1][r][t] = s[r];
      acc[r] = p.use_q ? __ldg(Q + static_cast<size_t>(r0 + r) * D + t) : 0.f;
    }
    const bool ok = mbar_wait_bounded(full0 + (j & 1) * 8, (j >> 1) & 1, sAbort);
    if (!ok) *sAbort = 1;
    __syncthreads();   // the rows of S are complete and M_j has landed (or the walk is given up)
    if (*sAbort != 0) break;
    const float* M = reinterpret_cast<const float*>(smem + SM::M0 + (j & 1) * FOLD_M_BYTES);
#pragma unroll 2
    for (int k0 = 0; k0 < D; k0 += 4) {
      const float m0 = M[(k0 + 0) * D + t], m1 = M[(k0 + 1) * D + t], m2 = M[(k0 + 2) * D + t], m3 = M[(k0 + 3) * D + t];
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        const float4 sv = *reinterpret_cast<const float4*>(&sS[j & 1][r][k0]);
        acc[r] = fmaf(sv.x, m0, acc[r]);
        acc[r] = fmaf(sv.y, m1, acc[r]);
        acc[r] = fmaf(sv.z, m2, acc[r]);
        acc[r] = fmaf(sv.w, m3, acc[r]);
      }
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) s[r] = acc[r];
    if (j + 2 < n_seg) {
      __syncthreads();   // every thread has read M_j: its slot takes M_{j+2}
      if (t == 0) {
        fence_proxy_async();
        issue(j + 2);
      }
      issued = j + 3;
    }
  }

  if (*sAbort != 0) {
    // a copy never completed: report, give the copies in flight one more bounded wait, leave
    if (t == 0) {
      if (status != nullptr) atomicExch(status, ST_FOLD_TIMEOUT);
      for (int j = (issued >= 2 ? issued - 2 : 0); j < issued; ++j) mbar_wait_bounded(full0 + (j & 1) * 8, (j >> 1) & 1, nullptr);
    }
    __syncthreads();
    return;
  }
  float* const s_last = s_in_at(n_seg);
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    if (s_last != nullptr) s_last[static_cast<size_t>(r0 + r) * D + t] = s[r];
    if (p.final_out != nullptr) p.final_out[static_cast<size_t>(chain) * p.final_stride + static_cast<size_t>(r0 + r) * D + t] = s[r];
  }
  if (p.n_signal > 0) {
    // the stores to the peers are ordered before the flags: CTA barrier, device-scope fence and count per
    // CTA; the CTA that counts last has observed them all and raises the flags behind one system-scope fence
    __syncthreads();
    if (t == 0) {
      __threadfence();
      const int done = atomicAdd(p.counter, 1);
      __threadfence();
      if (done == static_cast<int>(gridDim.x) - 1) {
        *p.counter = 0;
        __threadfence_system();
        for (int i = 0; i < p.n_signal; ++i) st_release_sys(p.signal[i], p.epoch);
      }
    }
  }
}

template <int ROWS>
static cudaError_t launch_fold_t(const FoldParams& p, cudaStream_t stream) {
  constexpr int smem_bytes = FoldSmem<ROWS>::TOTAL;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kda_state_fold_kernel<ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  kda_state_fold_kernel<ROWS><<<p.n_chains * (D / ROWS), D, smem_bytes, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_state_fold(const FoldParams& p, cudaStream_t stream) {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  // Measured on B200 (8 segments): the walk is bound by the L2-to-shared copies of M_j (every CTA of a
  // chain pulls all 64 KiB of it), so few rows per CTA only pay while the CTAs fit one wave:
  // 4 chains 23 us with 4 rows per CTA against 35 us with 16; 32 chains 100 us against 65 us; in between
  // 8 rows per CTA (8 chains x 4 segments 19.9 us against 24.1 us with 16 rows, x 8 segments 28.5 against 38.9).
  if (p.n_chains * (D / 4) <= sms) return launch_fold_t<4>(p, stream);
  if (p.n_chains * (D / 8) <= sms) return launch_fold_t<8>(p, stream);
  return launch_fold_t<16>(p, stream);
}

}  // namespace kda
