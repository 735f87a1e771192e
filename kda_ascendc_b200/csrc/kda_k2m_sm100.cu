// K2, "m16" organisation: the state rows on the MMA M dimension, 16 rows of h per warp.
//
// Same recurrence as kda_k2_sm100.cu (reference: src/kda_bt16/kernels.py:187-302,
// tests/test_torch_reference.py:175-194), evaluated in the transposed form
//   P1: [v_new^T | o^T] = h [w^T | qg^T]    (M = 16 rows v, N = 16+16 tokens, K = 128)  32 MMAs
//   P2: h += v_new^T kg                     (M = 16 rows v, N = 128 k, K = 16 tokens)  3 x 16 MMAs
//   P3: o^T += v_new^T Aqk^T                (M = 16 rows v, N = 16 tokens, K = 16)     6 MMAs
// The state tile h[16 v][128 k] lives in registers as fp32 accumulator fragments; the
// accumulator layout of two adjacent 8-column tiles IS the A-operand layout of a 16x16 tile,
// so bf16(h) and v_new feed the next product by a register pack alone.  The shared operands
// (w, qg, kg, Aqk) are the B side here: a B fragment is half the size of an A fragment, so this
// organisation reads half as many shared-memory bytes per MMA as the "n8" one, at the price of
// a chain twice as long per warp (86 MMAs per step).  Per state row it needs fewer instructions
// (no transposes, operand loads shared by 16 rows), which makes it the better choice once
// there are more 8-row tiles than SM sub-partitions (more than about 37 (batch, head) chains).
//
// Loads are interleaved with the MMA sequences so that their latency is covered (an m16n8k16
// holds the sub-partition's issue port for 8 cycles; the step time is 8 x MMAs + 2 x the other
// instructions): P1 carries its own rolling B-fragment loads,
// the decay row and the kg(hi) fragments; P2's first two passes carry kg(lo), its last pass the
// next step's first fragments; the output tile is transposed in-warp (movmatrix) and stored one
// step late.  Producer warp, stage ring, bounded waits: as in kda_k2_sm100.cu.
#include "kda_common.cuh"
#include "kda_kernels.h"

namespace kda {

constexpr int K2M_STAGES = 4;

template <int CW>
struct K2mSmem {
  static constexpr int STAGE = REC_SHARED_BYTES + CW * 2 * REC_U_TILE_BYTES;   // 16 rows = two 8-column u tiles
  static constexpr int BARS = K2M_STAGES * STAGE;
  static constexpr int FLAG = BARS + 2 * K2M_STAGES * 8;
  static constexpr int TOTAL = FLAG + 16;
};

// MINB = CTAs that must fit on one SM.  With 2 (register cap 168) eight consumer warps share an
// SM; that pays as soon as there are more CTAs than SMs (measured: B1 T8192 H96 765 -> 677 us),
// while a grid that fits in one wave is faster with the uncapped registers.
template <int CW, bool STATE_ONLY, int MINB>
__global__ void __launch_bounds__((CW + 1) * 32, MINB) kda_k2m_kernel(const K2Params p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  using SM = K2mSmem<CW>;
  constexpr int NV = 8 / CW;            // CTAs per (batch, head)
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int chain = blockIdx.x / NV + p.chain0;
  const bool pair = STATE_ONLY && p.pair_mode != 0;
  const int bh = pair ? (chain >> 1) : chain;      // the (batch, head) whose records are walked
  const int plane = pair ? (chain & 1) : 1;        // pair mode: 0 = transition matrix, 1 = offset
  const int vs = blockIdx.x % NV;
  int b = bh / p.H;
  const int h = bh % p.H;
  int NT = p.NT, Tlen = p.T, tok0 = 0;
  size_t rec_first = static_cast<size_t>(bh) * NT;
  if (p.seq_table != nullptr) {   // packed sequences: bh = sequence * H + head
    const int4 e = __ldg(p.seq_table + b);
    tok0 = e.x; NT = e.y; Tlen = e.w;
    rec_first = static_cast<size_t>(e.z) + static_cast<size_t>(h) * NT;
    b = 0;
  }

  const uint32_t sbase = smem_u32(smem);
  const uint32_t full0 = sbase + SM::BARS;
  const uint32_t empty0 = full0 + K2M_STAGES * 8;
  volatile int* sAbort = reinterpret_cast<volatile int*>(smem + SM::FLAG);
  volatile int* sIssued = sAbort + 1;

  if (tid == 0) {
    for (int s = 0; s < K2M_STAGES; ++s) {
      mbar_init(full0 + s * 8, 1);
      mbar_init(empty0 + s * 8, CW);
    }
    *sAbort = 0;
    *sIssued = 0;
    fence_mbar_init();
  }
  __syncthreads();

  const uint8_t* rec_bh = p.rec + rec_first * REC_BYTES;

  if (warp == CW) {
    // ------------------------------ producer -------------------------------
    if (lane == 0) {
      for (int n = 0; n < NT; ++n) {
        const int s = n % K2M_STAGES;
        if (n >= K2M_STAGES) {
          if (!mbar_wait_bounded(empty0 + s * 8, ((n / K2M_STAGES) - 1) & 1, sAbort)) {
            if (*sAbort == 0) { *sAbort = 1; atomicExch(p.status, ST_K2_EMPTY_TIMEOUT); }
            break;
          }
        }
        const uint8_t* rec = rec_bh + static_cast<size_t>(n) * REC_BYTES;
        const uint32_t dst = sbase + s * SM::STAGE;
        mbar_arrive_expect_tx(full0 + s * 8, SM::STAGE);
        bulk_g2s(dst, rec, REC_SHARED_BYTES, full0 + s * 8);
        bulk_g2s(dst + REC_SHARED_BYTES, rec + REC_U + vs * (CW * 2 * REC_U_TILE_BYTES), CW * 2 * REC_U_TILE_BYTES,
                 full0 + s * 8);
        *sIssued = n + 1;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ consumers ------------------------------
    const int gq = lane >> 2, tq = lane & 3;
    const int vrow0 = (vs * CW + warp) * 16;
    // hs[nt][e]: v = vrow0 + gq (+8 for e >= 2), k = 8nt + 2tq + (e & 1)
    float hs[16][4];
    bool h0_ok = true;
    if (pair) {
#pragma unroll
      for (int nt = 0; nt < 16; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e)
          hs[nt][e] = (plane == 0 && (vrow0 + gq + (e >> 1) * 8) == (nt * 8 + tq * 2 + (e & 1))) ? 1.f : 0.f;
    } else if (p.h0 != nullptr) {
      if (!STATE_ONLY && p.h0_n_flags > 0) {   // the entry state comes from other GPUs: wait for their flags (the producer warp is already loading records)
        int ok = 1;
        if (lane == 0)
          for (int i = 0; i < p.h0_n_flags; ++i) ok &= flag_wait_bounded(p.h0_flags + i, p.h0_epoch) ? 1 : 0;
        h0_ok = __shfl_sync(0xffffffffu, ok, 0) != 0;
      }
      const float* h0 = p.h0 + static_cast<size_t>(bh) * D * D;
#pragma unroll
      for (int nt = 0; nt < 16; ++nt) {
        if (p.k_first) {
          const float* c0 = h0 + (nt * 8 + tq * 2) * D + vrow0 + gq;
          hs[nt][0] = c0[0]; hs[nt][1] = c0[D]; hs[nt][2] = c0[8]; hs[nt][3] = c0[D + 8];
        } else {
          const float2 a = *reinterpret_cast<const float2*>(h0 + (vrow0 + gq) * D + nt * 8 + tq * 2);
          const float2 c = *reinterpret_cast<const float2*>(h0 + (vrow0 + gq + 8) * D + nt * 8 + tq * 2);
          hs[nt][0] = a.x; hs[nt][1] = a.y; hs[nt][2] = c.x; hs[nt][3] = c.y;
        }
      }
    } else {
#pragma unroll
      for (int nt = 0; nt < 16; ++nt) hs[nt][0] = hs[nt][1] = hs[nt][2] = hs[nt][3] = 0.f;
    }

    // per-lane ldmatrix address components (constant across steps)
    const int b1_row = (lane & 7) + (lane >> 4) * 8, b1_col = ((lane >> 3) & 1) * 8;   // w, qg: [N=tok][K=k]
    const int b2_row = (lane & 7) + ((lane >> 3) & 1) * 8, b2_col = (lane >> 4) * 8;   // kg: [K=tok][N=k], .trans
    // swizzled address of k-step ks = (256-byte aligned tile base + lane part) ^ (ks << 5)
    const uint32_t b1_lane = swz_off(b1_row, b1_col), b2_lane = swz_off(b2_row, b2_col);
    const uint32_t b3_off = REC_AQK + (((lane & 7) + (lane >> 4) * 8) * 16 + ((lane >> 3) & 1) * 8) * 2;
    // u^T fragment of this warp out of the record's [8-column tile][lane][4] blocks (see kda_common.cuh):
    // element (v = vrow0 + gq + 8a, tok = 2tq + j + 8c)  ->  tile 2*warp + a, lane (2tq+j)*4 + gq/2, slot 2c + gq%2
    const uint32_t u_off = REC_SHARED_BYTES + (warp * 2) * REC_U_TILE_BYTES + ((tq * 2) * 4 + (gq >> 1)) * 16 + (gq & 1) * 4;
    __nv_bfloat16* const ob = STATE_ONLY ? nullptr : p.o + b * p.o_s[0] + tok0 * p.o_s[1] + h * p.o_s[2] + vrow0 + tq * 2;
    const bool use_u = pair ? (plane == 1) : !(STATE_ONLY && p.zero_u);

    // rolling B fragments of P1: two k-steps ahead
    uint32_t bw[2][4], bq[2][4];
    float ut[2][4];             // u^T fragment: [token tile c][e]: e = 2a + j
    uint32_t o_st[2][2];        // previous step's output tile, already transposed and packed
    float2 dec[16];             // decay of the columns k = 8nt + 2tq, +1 (loaded one step ahead)

    auto load_u = [&](const uint8_t* spg) {
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
          for (int j = 0; j < 2; ++j)
            ut[c][a * 2 + j] = use_u ? *reinterpret_cast<const float*>(spg + u_off + a * REC_U_TILE_BYTES + j * 64 + c * 8)
                                     : 0.f;
    };
    auto load_dec = [&](const uint8_t* spg, int nt0, int nt1) {
#pragma unroll
      for (int nt = nt0; nt < nt1; ++nt) dec[nt] = *reinterpret_cast<const float2*>(spg + REC_DEC + (nt * 8 + tq * 2) * 4);
    };
    auto load_b1 = [&](uint32_t sp, int ks, int slot) {
      ldsm_x4(((sp + b1_lane) ^ (ks << 5)) + REC_W, bw[slot][0], bw[slot][1], bw[slot][2], bw[slot][3]);
      if (!STATE_ONLY)
        ldsm_x4(((sp + b1_lane) ^ (ks << 5)) + REC_QG, bq[slot][0], bq[slot][1], bq[slot][2], bq[slot][3]);
    };

    bool failed = false;
    if (!h0_ok) {
      if (*sAbort == 0) { *sAbort = 1; atomicExch(p.status, ST_PEER_TIMEOUT); }
      failed = true;
    } else if (!__all_sync(0xffffffffu, mbar_wait_bounded(full0, 0, sAbort))) {
      if (*sAbort == 0) { *sAbort = 1; atomicExch(p.status, ST_K2_FULL_TIMEOUT); }
      failed = true;
    } else {
      load_b1(sbase, 0, 0);
      load_b1(sbase, 1, 1);
      load_u(smem);
      load_dec(smem, 0, 16);
    }

    for (int n = 0; n < NT && !failed; ++n) {
      const int s = n % K2M_STAGES;
      const uint32_t sp = sbase + s * SM::STAGE;
      const uint8_t* spg = smem + s * SM::STAGE;

      // the previous step's output tile (always a full chunk): rows tok gq / gq+8, 2 value columns
      if (!STATE_ONLY && n > 0) {
        __nv_bfloat16* op = ob + static_cast<int64_t>((n - 1) * BT + gq) * p.o_s[1];
        *reinterpret_cast<uint32_t*>(op) = o_st[0][0];
        *reinterpret_cast<uint32_t*>(op + 8) = o_st[0][1];
        *reinterpret_cast<uint32_t*>(op + 8 * p.o_s[1]) = o_st[1][0];
        *reinterpret_cast<uint32_t*>(op + 8 * p.o_s[1] + 8) = o_st[1][1];
      }

      // P1 with the A fragments of bf16(h) packed on the fly; carries the decay of the fp32 state,
      // its own rolling B loads and the kg(hi) fragments of this step
      float pw[2][4] = {}, pq[2][4] = {};
      uint32_t kgh[8][4], kgl[8][4];
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        uint32_t ah[4];
        ah[0] = pack_bf16(hs[2 * ks][0], hs[2 * ks][1]);
        ah[1] = pack_bf16(hs[2 * ks][2], hs[2 * ks][3]);
        ah[2] = pack_bf16(hs[2 * ks + 1][0], hs[2 * ks + 1][1]);
        ah[3] = pack_bf16(hs[2 * ks + 1][2], hs[2 * ks + 1][3]);
        const int sl = ks & 1;
        mma_bf16_v(pw[0], ah, bw[sl][0], bw[sl][1]);
        mma_bf16_v(pw[1], ah, bw[sl][2], bw[sl][3]);
        if (!STATE_ONLY) {
          mma_bf16_v(pq[0], ah, bq[sl][0], bq[sl][1]);
          mma_bf16_v(pq[1], ah, bq[sl][2], bq[sl][3]);
        }
        if (ks + 2 < 8) load_b1(sp, ks + 2, sl);
        ldsm_x4_t(((sp + b2_lane) ^ (ks << 5)) + REC_KGH, kgh[ks][0], kgh[ks][1], kgh[ks][2], kgh[ks][3]);
        {
          const float2 d0 = dec[2 * ks], d1 = dec[2 * ks + 1];
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const float2 dd = half ? d1 : d0;
            float* t = hs[2 * ks + half];
            const float2 lo = __fmul2_rn(make_float2(t[0], t[1]), dd), hi = __fmul2_rn(make_float2(t[2], t[3]), dd);
            t[0] = lo.x; t[1] = lo.y; t[2] = hi.x; t[3] = hi.y;
          }
        }
      }

      // v_new^T (fp32, accumulator layout: rows v, cols tok) and its hi/lo A fragments
      uint32_t avh[4], avl[4];
      split_pack(ut[0][0] - pw[0][0], ut[0][1] - pw[0][1], avh[0], avl[0]);
      split_pack(ut[0][2] - pw[0][2], ut[0][3] - pw[0][3], avh[1], avl[1]);
      split_pack(ut[1][0] - pw[1][0], ut[1][1] - pw[1][1], avh[2], avl[2]);
      split_pack(ut[1][2] - pw[1][2], ut[1][3] - pw[1][3], avh[3], avl[3]);

      // P2 pass 1 (hi * hi), carrying the kg(lo) fragments
#pragma unroll
      for (int np = 0; np < 8; ++np) {
        mma_bf16_v(hs[2 * np], avh, kgh[np][0], kgh[np][1]);
        mma_bf16_v(hs[2 * np + 1], avh, kgh[np][2], kgh[np][3]);
        ldsm_x4_t(((sp + b2_lane) ^ (np << 5)) + REC_KGL, kgl[np][0], kgl[np][1], kgl[np][2], kgl[np][3]);
      }
      uint32_t ba[4], bl[4];
      if (!STATE_ONLY) {
        ldsm_x4(sp + b3_off, ba[0], ba[1], ba[2], ba[3]);
        ldsm_x4(sp + b3_off + (REC_AQL - REC_AQK), bl[0], bl[1], bl[2], bl[3]);
      }
      // P2 pass 2 (lo(v) * hi)
#pragma unroll
      for (int np = 0; np < 8; ++np) {
        mma_bf16_v(hs[2 * np], avl, kgh[np][0], kgh[np][1]);
        mma_bf16_v(hs[2 * np + 1], avl, kgh[np][2], kgh[np][3]);
      }

      // every shared-memory operand of this stage has been requested; once the loads have landed
      // (they are consumed below) the stage is released and the next one checked
      const bool more = n + 1 < NT;
      const int s1 = (n + 1) % K2M_STAGES;
      const uint32_t sp1 = sbase + s1 * SM::STAGE;
      const uint8_t* spg1 = smem + s1 * SM::STAGE;

      // P2 pass 3 (hi * lo(kg)), with P3 and the next step's first operands in its gaps
      float oa[2][4];
      if (!STATE_ONLY) {
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e) oa[j][e] = p.scale * pq[j][e];
      }
#pragma unroll
      for (int np = 0; np < 8; ++np) {
        mma_bf16_v(hs[2 * np], avh, kgl[np][0], kgl[np][1]);
        mma_bf16_v(hs[2 * np + 1], avh, kgl[np][2], kgl[np][3]);
        if (!STATE_ONLY) {
          if (np == 0) { mma_bf16_v(oa[0], avh, ba[0], ba[1]); mma_bf16_v(oa[1], avh, ba[2], ba[3]); }
          if (np == 2) { mma_bf16_v(oa[0], avl, ba[0], ba[1]); mma_bf16_v(oa[1], avl, ba[2], ba[3]); }
          if (np == 4) { mma_bf16_v(oa[0], avh, bl[0], bl[1]); mma_bf16_v(oa[1], avh, bl[2], bl[3]); }
        }
        if (np == 3) {
          // release the stage only when its fragment loads have landed: shared-memory loads of a
          // warp return in issue order, so reading a register of the last-issued ones makes the
          // warp wait for all of them
          uint32_t landed = kgl[7][0];
          if (!STATE_ONLY) landed ^= ba[0] ^ bl[0];
          asm volatile("" ::"r"(landed) : "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(empty0 + s * 8);
          if (more) {
            if (!__all_sync(0xffffffffu, mbar_wait_bounded(full0 + s1 * 8, ((n + 1) / K2M_STAGES) & 1, sAbort))) {
              if (*sAbort == 0) { *sAbort = 1; atomicExch(p.status, ST_K2_FULL_TIMEOUT); }
              failed = true;
            }
          }
        }
        if (more && !failed) {
          if (np == 4) { load_b1(sp1, 0, 0); load_dec(spg1, 0, 6); }
          if (np == 5) { load_b1(sp1, 1, 1); load_dec(spg1, 6, 12); }
          if (np == 6) { load_u(spg1); load_dec(spg1, 12, 16); }
        }
      }

      // output tile: o^T fragments (rows v, cols tok) -> in-warp transpose -> (rows tok, 2 value columns)
      if (!STATE_ONLY) {
        o_st[0][0] = movmatrix_t(pack_bf16(oa[0][0], oa[0][1]));   // tokens 0..7,  v = vrow0 + 2tq
        o_st[0][1] = movmatrix_t(pack_bf16(oa[0][2], oa[0][3]));   // tokens 0..7,  v = vrow0 + 8 + 2tq
        o_st[1][0] = movmatrix_t(pack_bf16(oa[1][0], oa[1][1]));   // tokens 8..15
        o_st[1][1] = movmatrix_t(pack_bf16(oa[1][2], oa[1][3]));
      }
    }

    // the last chunk's output tile (it may be a partial chunk)
    if (!STATE_ONLY && !failed) {
      const int tok = (NT - 1) * BT + gq;
      __nv_bfloat16* op = ob + static_cast<int64_t>(tok) * p.o_s[1];
      if (tok < Tlen) {
        *reinterpret_cast<uint32_t*>(op) = o_st[0][0];
        *reinterpret_cast<uint32_t*>(op + 8) = o_st[0][1];
      }
      if (tok + 8 < Tlen) {
        *reinterpret_cast<uint32_t*>(op + 8 * p.o_s[1]) = o_st[1][0];
        *reinterpret_cast<uint32_t*>(op + 8 * p.o_s[1] + 8) = o_st[1][1];
      }
    }

    if (!failed && p.ht != nullptr) {
      float* ht = p.ht + static_cast<size_t>(chain) * D * D;
#pragma unroll
      for (int nt = 0; nt < 16; ++nt) {
        if (p.k_first && !pair) {
          float* c0 = ht + (nt * 8 + tq * 2) * D + vrow0 + gq;
          c0[0] = hs[nt][0]; c0[D] = hs[nt][1]; c0[8] = hs[nt][2]; c0[D + 8] = hs[nt][3];
        } else {
          *reinterpret_cast<float2*>(ht + (vrow0 + gq) * D + nt * 8 + tq * 2) = make_float2(hs[nt][0], hs[nt][1]);
          *reinterpret_cast<float2*>(ht + (vrow0 + gq + 8) * D + nt * 8 + tq * 2) = make_float2(hs[nt][2], hs[nt][3]);
        }
      }
    }
  }

  __syncthreads();
  if (*sAbort != 0 && tid == 0) {
    const int issued = *sIssued;
    for (int n = max(0, issued - K2M_STAGES); n < issued; ++n)
      mbar_wait_bounded(full0 + (n % K2M_STAGES) * 8, (n / K2M_STAGES) & 1, nullptr);
  }
}

template <int CW, bool STATE_ONLY, int MINB>
static cudaError_t launch_k2m_t(const K2Params& p, int nblocks, cudaStream_t stream) {
  constexpr int smem_bytes = K2mSmem<CW>::TOTAL;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kda_k2m_kernel<CW, STATE_ONLY, MINB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         smem_bytes);
    if (e != cudaSuccess) return e;
    if (MINB > 1) {
      e = cudaFuncSetAttribute(kda_k2m_kernel<CW, STATE_ONLY, MINB>, cudaFuncAttributePreferredSharedMemoryCarveout,
                               cudaSharedmemCarveoutMaxShared);
      if (e != cudaSuccess) return e;
    }
    configured[dev] = true;
  }
  kda_k2m_kernel<CW, STATE_ONLY, MINB><<<nblocks, (CW + 1) * 32, smem_bytes, stream>>>(p);
  return cudaGetLastError();
}

template <int CW, bool STATE_ONLY>
static cudaError_t launch_k2m_c(const K2Params& p, cudaStream_t stream) {
  static int sms[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 64) return cudaErrorInvalidDevice;
  if (sms[dev] == 0) {
    cudaError_t e = cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
  }
  const int nblocks = (p.n_chains > 0 ? p.n_chains : (p.seq_table != nullptr ? p.n_seqs : p.B) * p.H) * (8 / CW);
  if (CW == 4 && nblocks > sms[dev]) return launch_k2m_t<CW, STATE_ONLY, 2>(p, nblocks, stream);
  return launch_k2m_t<CW, STATE_ONLY, 1>(p, nblocks, stream);
}

cudaError_t launch_k2m(const K2Params& p, int vsplit, bool state_only, cudaStream_t stream) {
  switch (vsplit) {
    case 2: return state_only ? launch_k2m_c<4, true>(p, stream) : launch_k2m_c<4, false>(p, stream);
    case 4: return state_only ? launch_k2m_c<2, true>(p, stream) : launch_k2m_c<2, false>(p, stream);
    case 8: return state_only ? launch_k2m_c<1, true>(p, stream) : launch_k2m_c<1, false>(p, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace kda
