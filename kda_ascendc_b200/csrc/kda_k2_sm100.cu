// K2: delta-rule state recurrence and output of the KDA forward.  sm_100a.
//
// Replaces kda_bt16_kernel_k2 of the reference (src/kda_bt16/kernels.py:187-302); the
// arithmetic is the recurrence of the reference's torch chunk implementation
// (tests/test_torch_reference.py:175-194), V-first state h[V][K]:
//   v_new = u - w h^T ;  o = scale (qg h^T) + Aqk v_new ;  h = h diag(dec) + v_new^T kg
// evaluated in the transposed form so that the 128-wide state dimension V is the MMA
// row dimension:
//   P1: [v_new^T | o^T]  = h [w^T | qg^T]       (M = V rows, N = 16+16 tokens, K = 128)
//   P2: h               += v_new^T kg            (M = V rows, N = 128,          K = 16 tokens)
//   P3: o^T             += v_new^T Aqk^T         (M = V rows, N = 16,           K = 16)
//
// One warp owns 16 rows of the state for the whole sequence and keeps them in
// registers (fp32, 64 per thread) in the m16n8 accumulator layout.  That layout is also
// the A-operand layout of the next product, so the chain
//   bf16(h) -> P1 -> v_new -> P2 -> h
// never leaves the register file: no shared-memory or tensor-memory round trip sits on
// the serial path, which is what bounds this kernel (NT dependent steps per head).
// P2 uses a hi/lo bf16 split of both v_new and kg (three MMAs) because the state must
// stay within 2e-3 of an fp32 implementation; P3 does the same with v_new and Aqk (the
// intra-chunk term dominates o); P1 uses plain bf16 operands.
//
// A CTA = VW consumer warps (a slice of VW*16 state rows of one (batch, head)) plus one
// producer warp that streams the chunk records through a ring of shared-memory stages
// with bulk (TMA) copies: full/empty mbarriers, every wait bounded.
#include "kda_common.cuh"
#include "kda_kernels.h"

namespace kda {

constexpr int K2_STAGES = 4;

template <int VW>
struct K2Smem {
  static constexpr int STAGE = REC_SHARED_BYTES + VW * REC_U_TILE_BYTES;
  static constexpr int BARS = K2_STAGES * STAGE;            // full[S], empty[S]
  static constexpr int FLAG = BARS + 2 * K2_STAGES * 8;     // abort flag, issued count
  static constexpr int TOTAL = FLAG + 16;
};

template <int VW, bool STATE_ONLY>
__global__ void __launch_bounds__((VW + 1) * 32, 1) kda_k2_kernel(const K2Params p) {
  extern __shared__ __align__(128) uint8_t smem[];
  using SM = K2Smem<VW>;
  constexpr int NV = 8 / VW;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int bh = blockIdx.x / NV;
  const int vs = blockIdx.x % NV;
  const int b = bh / p.H, h = bh % p.H;
  const int NT = p.NT;

  const uint32_t sbase = smem_u32(smem);
  const uint32_t full0 = sbase + SM::BARS;
  const uint32_t empty0 = full0 + K2_STAGES * 8;
  volatile int* sAbort = reinterpret_cast<volatile int*>(smem + SM::FLAG);
  volatile int* sIssued = sAbort + 1;

  if (tid == 0) {
    for (int s = 0; s < K2_STAGES; ++s) {
      mbar_init(full0 + s * 8, 1);
      mbar_init(empty0 + s * 8, VW);
    }
    *sAbort = 0;
    *sIssued = 0;
    fence_mbar_init();
  }
  __syncthreads();

  const uint8_t* rec_bh = p.rec + static_cast<size_t>(bh) * NT * REC_BYTES;

  if (warp == VW) {
    // ------------------------------ producer -------------------------------
    if (lane == 0) {
      for (int n = 0; n < NT; ++n) {
        const int s = n % K2_STAGES;
        if (n >= K2_STAGES) {
          if (!mbar_wait_bounded(empty0 + s * 8, ((n / K2_STAGES) - 1) & 1, sAbort)) {
            if (*sAbort == 0) { *sAbort = 1; atomicExch(p.status, ST_K2_EMPTY_TIMEOUT); }
            break;
          }
        }
        const uint8_t* rec = rec_bh + static_cast<size_t>(n) * REC_BYTES;
        const uint32_t dst = sbase + s * SM::STAGE;
        mbar_arrive_expect_tx(full0 + s * 8, SM::STAGE);
        bulk_g2s(dst, rec, REC_SHARED_BYTES, full0 + s * 8);
        bulk_g2s(dst + REC_SHARED_BYTES, rec + REC_U + vs * VW * REC_U_TILE_BYTES, VW * REC_U_TILE_BYTES,
                 full0 + s * 8);
        *sIssued = n + 1;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ consumers ------------------------------
    const int gq = lane >> 2, tq = lane & 3;
    const int vrow0 = (vs * VW + warp) * 16;
    float hs[16][4];
    if (p.h0 != nullptr) {
      const float* h0 = p.h0 + static_cast<size_t>(bh) * D * D;
#pragma unroll
      for (int nt = 0; nt < 16; ++nt) {
        const float2 a = *reinterpret_cast<const float2*>(h0 + (vrow0 + gq) * D + nt * 8 + tq * 2);
        const float2 c = *reinterpret_cast<const float2*>(h0 + (vrow0 + gq + 8) * D + nt * 8 + tq * 2);
        hs[nt][0] = a.x; hs[nt][1] = a.y; hs[nt][2] = c.x; hs[nt][3] = c.y;
      }
    } else {
#pragma unroll
      for (int nt = 0; nt < 16; ++nt) hs[nt][0] = hs[nt][1] = hs[nt][2] = hs[nt][3] = 0.f;
    }

    // per-lane ldmatrix address components (constant across steps)
    const int p1_row = (lane & 7) + (lane >> 4) * 8, p1_col = ((lane >> 3) & 1) * 8;   // [N=tok][K=k]
    const int p2_row = (lane & 7) + ((lane >> 3) & 1) * 8, p2_col = (lane >> 4) * 8;   // [K=tok][N=k], .trans
    const uint32_t p3_off = REC_AQK + (((lane & 7) + (lane >> 4) * 8) * 16 + ((lane >> 3) & 1) * 8) * 2;

    bool failed = false;
    for (int n = 0; n < NT; ++n) {
      const int s = n % K2_STAGES;
      // the verdict is made warp-uniform: the MMAs below need all 32 lanes
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(full0 + s * 8, (n / K2_STAGES) & 1, sAbort))) {
        if (*sAbort == 0) { *sAbort = 1; atomicExch(p.status, ST_K2_FULL_TIMEOUT); }
        failed = true;
        break;
      }
      const uint32_t sp = sbase + s * SM::STAGE;
      const uint8_t* spg = smem + s * SM::STAGE;

      // A fragments of bf16(h) (pre-chunk state), then the decay on the fp32 copy
      uint32_t ah[8][4];
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        ah[ks][0] = pack_bf16(hs[2 * ks][0], hs[2 * ks][1]);
        ah[ks][1] = pack_bf16(hs[2 * ks][2], hs[2 * ks][3]);
        ah[ks][2] = pack_bf16(hs[2 * ks + 1][0], hs[2 * ks + 1][1]);
        ah[ks][3] = pack_bf16(hs[2 * ks + 1][2], hs[2 * ks + 1][3]);
      }
#pragma unroll
      for (int nt = 0; nt < 16; ++nt) {
        const float2 d = *reinterpret_cast<const float2*>(spg + REC_DEC + (nt * 8 + tq * 2) * 4);
        hs[nt][0] *= d.x; hs[nt][1] *= d.y; hs[nt][2] *= d.x; hs[nt][3] *= d.y;
      }

      // P1: two accumulator sets (even / odd k-steps) to halve the dependent MMA chain
      float pw[2][2][4] = {}, pq[2][2][4] = {};
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        uint32_t bw[4];
        ldsm_x4(sp + REC_W + swz_off(p1_row, ks * 16 + p1_col), bw[0], bw[1], bw[2], bw[3]);
        mma_bf16(pw[ks & 1][0], ah[ks], bw[0], bw[1]);
        mma_bf16(pw[ks & 1][1], ah[ks], bw[2], bw[3]);
        if (!STATE_ONLY) {
          uint32_t bq[4];
          ldsm_x4(sp + REC_QG + swz_off(p1_row, ks * 16 + p1_col), bq[0], bq[1], bq[2], bq[3]);
          mma_bf16(pq[ks & 1][0], ah[ks], bq[0], bq[1]);
          mma_bf16(pq[ks & 1][1], ah[ks], bq[2], bq[3]);
        }
      }

      // v_new^T (fp32, C layout: rows v, cols tok) and its hi/lo A fragments
      float vn[2][4];
      {
        float4 u0 = make_float4(0, 0, 0, 0), u1 = u0;
        if (!(STATE_ONLY && p.zero_u)) {
          u0 = *reinterpret_cast<const float4*>(spg + REC_SHARED_BYTES + warp * REC_U_TILE_BYTES + lane * 16);
          u1 = *reinterpret_cast<const float4*>(spg + REC_SHARED_BYTES + warp * REC_U_TILE_BYTES + (32 + lane) * 16);
        }
        vn[0][0] = u0.x - (pw[0][0][0] + pw[1][0][0]); vn[0][1] = u0.y - (pw[0][0][1] + pw[1][0][1]);
        vn[0][2] = u0.z - (pw[0][0][2] + pw[1][0][2]); vn[0][3] = u0.w - (pw[0][0][3] + pw[1][0][3]);
        vn[1][0] = u1.x - (pw[0][1][0] + pw[1][1][0]); vn[1][1] = u1.y - (pw[0][1][1] + pw[1][1][1]);
        vn[1][2] = u1.z - (pw[0][1][2] + pw[1][1][2]); vn[1][3] = u1.w - (pw[0][1][3] + pw[1][1][3]);
      }
      uint32_t avh[4], avl[4];
      split_pack(vn[0][0], vn[0][1], avh[0], avl[0]);
      split_pack(vn[0][2], vn[0][3], avh[1], avl[1]);
      split_pack(vn[1][0], vn[1][1], avh[2], avl[2]);
      split_pack(vn[1][2], vn[1][3], avh[3], avl[3]);

      // P2: h += v_new^T kg  (hi*hi + lo*hi + hi*lo)
#pragma unroll
      for (int np = 0; np < 8; ++np) {
        uint32_t kh[4], kl[4];
        ldsm_x4_t(sp + REC_KGH + swz_off(p2_row, np * 16 + p2_col), kh[0], kh[1], kh[2], kh[3]);
        ldsm_x4_t(sp + REC_KGL + swz_off(p2_row, np * 16 + p2_col), kl[0], kl[1], kl[2], kl[3]);
        mma_bf16(hs[2 * np], avh, kh[0], kh[1]);
        mma_bf16(hs[2 * np + 1], avh, kh[2], kh[3]);
        mma_bf16(hs[2 * np], avl, kh[0], kh[1]);
        mma_bf16(hs[2 * np + 1], avl, kh[2], kh[3]);
        mma_bf16(hs[2 * np], avh, kl[0], kl[1]);
        mma_bf16(hs[2 * np + 1], avh, kl[2], kl[3]);
      }

      if (!STATE_ONLY) {
        // P3 and the output: o^T = scale * (h qg^T) + v_new^T Aqk^T
        float oa[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e) oa[j][e] = p.scale * (pq[0][j][e] + pq[1][j][e]);
        uint32_t ba[4], bl[4];
        ldsm_x4(sp + p3_off, ba[0], ba[1], ba[2], ba[3]);
        ldsm_x4(sp + p3_off + (REC_AQL - REC_AQK), bl[0], bl[1], bl[2], bl[3]);
        mma_bf16(oa[0], avh, ba[0], ba[1]);
        mma_bf16(oa[1], avh, ba[2], ba[3]);
        mma_bf16(oa[0], avl, ba[0], ba[1]);
        mma_bf16(oa[1], avl, ba[2], ba[3]);
        mma_bf16(oa[0], avh, bl[0], bl[1]);
        mma_bf16(oa[1], avh, bl[2], bl[3]);
        const int t0 = n * BT;
        __nv_bfloat16* ob = p.o + b * p.o_s[0] + h * p.o_s[2] + vrow0 + gq;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int tok = t0 + j * 8 + tq * 2;
          if (tok < p.T) {
            ob[tok * p.o_s[1]] = __float2bfloat16_rn(oa[j][0]);
            ob[tok * p.o_s[1] + 8] = __float2bfloat16_rn(oa[j][2]);
          }
          if (tok + 1 < p.T) {
            ob[(tok + 1) * p.o_s[1]] = __float2bfloat16_rn(oa[j][1]);
            ob[(tok + 1) * p.o_s[1] + 8] = __float2bfloat16_rn(oa[j][3]);
          }
        }
      }

      // release the stage
      __syncwarp();
      if (lane == 0) mbar_arrive(empty0 + s * 8);
    }

    if (!failed && p.ht != nullptr) {
      float* ht = p.ht + static_cast<size_t>(bh) * D * D;
#pragma unroll
      for (int nt = 0; nt < 16; ++nt) {
        *reinterpret_cast<float2*>(ht + (vrow0 + gq) * D + nt * 8 + tq * 2) = make_float2(hs[nt][0], hs[nt][1]);
        *reinterpret_cast<float2*>(ht + (vrow0 + gq + 8) * D + nt * 8 + tq * 2) = make_float2(hs[nt][2], hs[nt][3]);
      }
    }
  }

  __syncthreads();
  if (*sAbort != 0 && tid == 0) {
    // give copies that are still in flight a bounded chance to land before the CTA's
    // shared memory is released
    const int issued = *sIssued;
    for (int n = max(0, issued - K2_STAGES); n < issued; ++n)
      mbar_wait_bounded(full0 + (n % K2_STAGES) * 8, (n / K2_STAGES) & 1, nullptr);
  }
}

template <int VW, bool STATE_ONLY>
static cudaError_t launch_k2_t(const K2Params& p, cudaStream_t stream) {
  constexpr int smem_bytes = K2Smem<VW>::TOTAL;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kda_k2_kernel<VW, STATE_ONLY>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         smem_bytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const int nblocks = p.B * p.H * (8 / VW);
  kda_k2_kernel<VW, STATE_ONLY><<<nblocks, (VW + 1) * 32, smem_bytes, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_k2(const K2Params& p, int vsplit, bool state_only, cudaStream_t stream) {
#define KDA_K2_CASE(NVV, VWW)                                                    \
  case NVV:                                                                      \
    return state_only ? launch_k2_t<VWW, true>(p, stream) : launch_k2_t<VWW, false>(p, stream);
  switch (vsplit) {
    KDA_K2_CASE(1, 8)
    KDA_K2_CASE(2, 4)
    KDA_K2_CASE(4, 2)
    KDA_K2_CASE(8, 1)
    default:
      return cudaErrorInvalidValue;
  }
#undef KDA_K2_CASE
}

}  // namespace kda
