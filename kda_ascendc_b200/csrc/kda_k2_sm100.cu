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
// A warp owns a 16-row x (128/KS)-column block of the state for the whole sequence and
// keeps it in registers (fp32) in the m16n8 accumulator layout.  That layout is also the
// A-operand layout of the next product, so the chain
//   bf16(h) -> P1 -> v_new -> P2 -> h
// never leaves the register file.  The kernel is bound by that serial chain (NT dependent
// steps per head) and by the legacy tensor pipe's issue rate per SM sub-partition, so the
// state of one head is spread over many warps: the 128 rows over 8 row tiles, and each
// row tile over KS warps that split the K dimension.  With KS > 1 the P1 partial sums of
// the KS warps are exchanged through shared memory once per step (fixed summation order,
// so every warp of a row tile derives bit-identical v_new), and the result does not
// depend on KS or on how many CTAs a head is split over beyond fp32 summation order of P1.
// P2 uses a hi/lo bf16 split of both v_new and kg (three MMAs) because the state must
// stay within 2e-3 of an fp32 implementation; P3 does the same with v_new and Aqk (the
// intra-chunk term dominates o); P1 uses plain bf16 operands.
//
// A CTA = VW row tiles x KS consumer warps (a slice of VW*16 state rows of one
// (batch, head)) plus one producer warp that streams the chunk records through a ring of
// shared-memory stages with bulk (TMA) copies: full/empty mbarriers, every wait bounded.
#include "kda_common.cuh"
#include "kda_kernels.h"

namespace kda {

#ifndef KDA_K2_STAGES
#define KDA_K2_STAGES 4
#endif
constexpr int K2_STAGES = KDA_K2_STAGES;

// Developer facility: with -DKDA_K2_PROFILE the first consumer warp of CTA 0 writes clock()
// stamps of every step's phases to K2Params::ht (which then is NOT a state) -- 8 stamps/step.
#ifdef KDA_K2_PROFILE
#define K2_STAMP(i)                                                                              \
  if (blockIdx.x == 0 && warp == 0 && lane == 0) reinterpret_cast<unsigned*>(p.ht)[n * 8 + (i)] = (unsigned)clock();
#else
#define K2_STAMP(i)
#endif

template <int VW, int KS>
struct K2Smem {
  static constexpr int STAGE = REC_SHARED_BYTES + VW * REC_U_TILE_BYTES;
  static constexpr int XCH = K2_STAGES * STAGE;                      // exchange: [2][VW][KS][4][32] float4
  static constexpr int XCH_BYTES = (KS > 1) ? 2 * VW * KS * 4 * 32 * 16 : 0;
  static constexpr int BARS = XCH + XCH_BYTES;                       // full[S], empty[S], xbar[2][VW]
  static constexpr int FLAG = BARS + (2 * K2_STAGES + 2 * VW) * 8;   // abort flag, issued count
  static constexpr int TOTAL = FLAG + 16;
};

template <int VW, int KS, bool STATE_ONLY>
__global__ void __launch_bounds__((VW * KS + 1) * 32, 1) kda_k2_kernel(const K2Params p) {
  extern __shared__ __align__(128) uint8_t smem[];
  using SM = K2Smem<VW, KS>;
  constexpr int NV = 8 / VW;          // CTAs per (batch, head)
  constexpr int NCW = VW * KS;        // consumer warps
  constexpr int NTL = 16 / KS;        // 8-column state tiles owned by a warp
  constexpr int KSL = 8 / KS;         // P1 k-steps (16 columns each) owned by a warp
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
  const uint32_t xbar0 = empty0 + K2_STAGES * 8;
  volatile int* sAbort = reinterpret_cast<volatile int*>(smem + SM::FLAG);
  volatile int* sIssued = sAbort + 1;

  if (tid == 0) {
    for (int s = 0; s < K2_STAGES; ++s) {
      mbar_init(full0 + s * 8, 1);
      mbar_init(empty0 + s * 8, NCW);
    }
    for (int i = 0; i < 2 * VW; ++i) mbar_init(xbar0 + i * 8, KS);
    *sAbort = 0;
    *sIssued = 0;
    fence_mbar_init();
  }
  __syncthreads();

  const uint8_t* rec_bh = p.rec + static_cast<size_t>(bh) * NT * REC_BYTES;

  if (warp == NCW) {
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
    const int vtl = warp / KS;                 // row tile inside the CTA
    const int kh = warp % KS;                  // which K block of the row tile
    const int vrow0 = (vs * VW + vtl) * 16;
    const int kbase = kh * (D / KS);
    float hs[NTL][4];
    if (p.h0 != nullptr) {
      const float* h0 = p.h0 + static_cast<size_t>(bh) * D * D;
#pragma unroll
      for (int nt = 0; nt < NTL; ++nt) {
        const float2 a = *reinterpret_cast<const float2*>(h0 + (vrow0 + gq) * D + kbase + nt * 8 + tq * 2);
        const float2 c = *reinterpret_cast<const float2*>(h0 + (vrow0 + gq + 8) * D + kbase + nt * 8 + tq * 2);
        hs[nt][0] = a.x; hs[nt][1] = a.y; hs[nt][2] = c.x; hs[nt][3] = c.y;
      }
    } else {
#pragma unroll
      for (int nt = 0; nt < NTL; ++nt) hs[nt][0] = hs[nt][1] = hs[nt][2] = hs[nt][3] = 0.f;
    }

    // per-lane ldmatrix address components (constant across steps)
    const int p1_row = (lane & 7) + (lane >> 4) * 8, p1_col = kbase + ((lane >> 3) & 1) * 8;   // [N=tok][K=k]
    const int p2_row = (lane & 7) + ((lane >> 3) & 1) * 8, p2_col = kbase + (lane >> 4) * 8;   // [K=tok][N=k], .trans
    const uint32_t p3_off = REC_AQK + (((lane & 7) + (lane >> 4) * 8) * 16 + ((lane >> 3) & 1) * 8) * 2;
    // output rows this warp finishes: all 16 tokens when the row tile has one warp, else 8
    constexpr int OJ = (KS == 1) ? 2 : 1;
    const bool o_owner = (KS == 1) || (kh < 2);
    const int oj0 = (KS == 1) ? 0 : kh;
    __nv_bfloat16* const ob = STATE_ONLY ? nullptr : p.o + b * p.o_s[0] + h * p.o_s[2] + vrow0 + gq;

    // One warp runs the whole chain in program order, so everything that is NOT on the chain
    // (operand loads, the previous step's output stores, barrier traffic) is placed in the
    // issue gaps of the two long MMA sequences: the tensor pipe accepts one m16n8k16 per
    // 8 cycles per sub-partition, which leaves ~6 issue slots between consecutive MMAs.
    //   P1 (h [w|qg]^T)  carries: this step's kg / Aqk fragment loads and the decay of h
    //   exchange wait    carries: the previous step's output stores
    //   P2 (h += vn kg)  carries: the next step's w / qg / dec / u loads
    uint32_t bw[KSL][4], bq[KSL][4];
    float2 dec[NTL];
    float4 u0 = make_float4(0, 0, 0, 0), u1 = u0;
    const bool use_u = !(STATE_ONLY && p.zero_u);

    bool failed = false;
    if (!__all_sync(0xffffffffu, mbar_wait_bounded(full0, 0, sAbort))) {
      if (*sAbort == 0) { *sAbort = 1; atomicExch(p.status, ST_K2_FULL_TIMEOUT); }
      failed = true;
    } else {
#pragma unroll
      for (int ks = 0; ks < KSL; ++ks) {
        ldsm_x4(sbase + REC_W + swz_off(p1_row, ks * 16 + p1_col), bw[ks][0], bw[ks][1], bw[ks][2], bw[ks][3]);
        if (!STATE_ONLY)
          ldsm_x4(sbase + REC_QG + swz_off(p1_row, ks * 16 + p1_col), bq[ks][0], bq[ks][1], bq[ks][2], bq[ks][3]);
      }
#pragma unroll
      for (int nt = 0; nt < NTL; ++nt)
        dec[nt] = *reinterpret_cast<const float2*>(smem + REC_DEC + (kbase + nt * 8 + tq * 2) * 4);
      if (use_u) {
        u0 = *reinterpret_cast<const float4*>(smem + REC_SHARED_BYTES + vtl * REC_U_TILE_BYTES + lane * 16);
        u1 = *reinterpret_cast<const float4*>(smem + REC_SHARED_BYTES + vtl * REC_U_TILE_BYTES + (32 + lane) * 16);
      }
    }
    float oa[OJ][4];          // output tile of the previous step, stored one step late
    for (int n = 0; n < NT && !failed; ++n) {
      const int s = n % K2_STAGES;
      const uint32_t sp = sbase + s * SM::STAGE;
      K2_STAMP(0)

      // A fragments of bf16(h) (pre-chunk state)
      uint32_t ah[KSL][4];
#pragma unroll
      for (int ks = 0; ks < KSL; ++ks) {
        ah[ks][0] = pack_bf16(hs[2 * ks][0], hs[2 * ks][1]);
        ah[ks][1] = pack_bf16(hs[2 * ks][2], hs[2 * ks][3]);
        ah[ks][2] = pack_bf16(hs[2 * ks + 1][0], hs[2 * ks + 1][1]);
        ah[ks][3] = pack_bf16(hs[2 * ks + 1][2], hs[2 * ks + 1][3]);
      }

      // P1 over this warp's K block (two accumulator sets: even / odd k-steps), interleaved with
      // the kg fragment loads of this step and the decay of the fp32 state
      float pw[2][2][4] = {}, pq[2][2][4] = {};
      uint32_t kgh[NTL / 2][4], kgl[NTL / 2][4], ba[4], bl[4];
#pragma unroll
      for (int ks = 0; ks < KSL; ++ks) {
        mma_bf16_v(pw[ks & 1][0], ah[ks], bw[ks][0], bw[ks][1]);
        mma_bf16_v(pw[ks & 1][1], ah[ks], bw[ks][2], bw[ks][3]);
        ldsm_x4_t(sp + REC_KGH + swz_off(p2_row, ks * 16 + p2_col), kgh[ks][0], kgh[ks][1], kgh[ks][2], kgh[ks][3]);
        if (!STATE_ONLY) {
          mma_bf16_v(pq[ks & 1][0], ah[ks], bq[ks][0], bq[ks][1]);
          mma_bf16_v(pq[ks & 1][1], ah[ks], bq[ks][2], bq[ks][3]);
        }
        ldsm_x4_t(sp + REC_KGL + swz_off(p2_row, ks * 16 + p2_col), kgl[ks][0], kgl[ks][1], kgl[ks][2], kgl[ks][3]);
#pragma unroll
        for (int nt = 2 * ks; nt < 2 * ks + 2; ++nt) {
          hs[nt][0] *= dec[nt].x; hs[nt][1] *= dec[nt].y; hs[nt][2] *= dec[nt].x; hs[nt][3] *= dec[nt].y;
        }
      }
      if (!STATE_ONLY && o_owner) {
        ldsm_x4(sp + p3_off, ba[0], ba[1], ba[2], ba[3]);
        ldsm_x4(sp + p3_off + (REC_AQL - REC_AQK), bl[0], bl[1], bl[2], bl[3]);
      }
      K2_STAMP(1)
      float sw[2][4], sq[2][4];   // full-K sums: [token tile][fragment element]
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          sw[j][e] = pw[0][j][e] + pw[1][j][e];
          sq[j][e] = pq[0][j][e] + pq[1][j][e];
        }

      float4* xb = reinterpret_cast<float4*>(smem + SM::XCH) + ((n & 1) * VW + vtl) * (KS * 4 * 32);
      const uint32_t xbar = xbar0 + ((n & 1) * VW + vtl) * 8;
      if (KS > 1) {
        // publish this warp's K-block partial sums to the other warps of the row tile
        float4* mine = xb + kh * (4 * 32) + lane;
        mine[0] = make_float4(sw[0][0], sw[0][1], sw[0][2], sw[0][3]);
        mine[32] = make_float4(sw[1][0], sw[1][1], sw[1][2], sw[1][3]);
        if (!STATE_ONLY) {
          mine[64] = make_float4(sq[0][0], sq[0][1], sq[0][2], sq[0][3]);
          mine[96] = make_float4(sq[1][0], sq[1][1], sq[1][2], sq[1][3]);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(xbar);
      }

      // the previous step's output tile goes out while the partner warps catch up
      if (!STATE_ONLY && o_owner && n > 0) {
#pragma unroll
        for (int jj = 0; jj < OJ; ++jj) {
          const int tok = (n - 1) * BT + (oj0 + jj) * 8 + tq * 2;   // always < T: not the last chunk
          __nv_bfloat16* op = ob + static_cast<int64_t>(tok) * p.o_s[1];
          op[0] = __float2bfloat16_rn(oa[jj][0]);
          op[8] = __float2bfloat16_rn(oa[jj][2]);
          op[p.o_s[1]] = __float2bfloat16_rn(oa[jj][1]);
          op[p.o_s[1] + 8] = __float2bfloat16_rn(oa[jj][3]);
        }
      }

      if (KS > 1) {
        if (!__all_sync(0xffffffffu, mbar_spin_bounded(xbar, (n >> 1) & 1, sAbort))) {
          if (*sAbort == 0) { *sAbort = 1; atomicExch(p.status, ST_K2_FULL_TIMEOUT); }
          failed = true;
          break;
        }
        // fixed order kh = 0..KS-1, identical in every warp of the row tile
#pragma unroll
        for (int k2 = 0; k2 < KS; ++k2) {
          const float4 a = xb[k2 * (4 * 32) + lane], c = xb[k2 * (4 * 32) + 32 + lane];
          if (k2 == 0) {
            sw[0][0] = a.x; sw[0][1] = a.y; sw[0][2] = a.z; sw[0][3] = a.w;
            sw[1][0] = c.x; sw[1][1] = c.y; sw[1][2] = c.z; sw[1][3] = c.w;
          } else {
            sw[0][0] += a.x; sw[0][1] += a.y; sw[0][2] += a.z; sw[0][3] += a.w;
            sw[1][0] += c.x; sw[1][1] += c.y; sw[1][2] += c.z; sw[1][3] += c.w;
          }
        }
        if (!STATE_ONLY && o_owner) {
#pragma unroll
          for (int k2 = 0; k2 < KS; ++k2) {
            const float4 a = xb[k2 * (4 * 32) + (2 + oj0) * 32 + lane];
            if (k2 == 0) { sq[0][0] = a.x; sq[0][1] = a.y; sq[0][2] = a.z; sq[0][3] = a.w; }
            else { sq[0][0] += a.x; sq[0][1] += a.y; sq[0][2] += a.z; sq[0][3] += a.w; }
          }
        }
      }

      K2_STAMP(2)
      // v_new^T (fp32, C layout: rows v, cols tok) and its hi/lo A fragments
      float vn[2][4];
      vn[0][0] = u0.x - sw[0][0]; vn[0][1] = u0.y - sw[0][1]; vn[0][2] = u0.z - sw[0][2]; vn[0][3] = u0.w - sw[0][3];
      vn[1][0] = u1.x - sw[1][0]; vn[1][1] = u1.y - sw[1][1]; vn[1][2] = u1.z - sw[1][2]; vn[1][3] = u1.w - sw[1][3];
      uint32_t avh[4], avl[4];
      split_pack(vn[0][0], vn[0][1], avh[0], avl[0]);
      split_pack(vn[0][2], vn[0][3], avh[1], avl[1]);
      split_pack(vn[1][0], vn[1][1], avh[2], avl[2]);
      split_pack(vn[1][2], vn[1][3], avh[3], avl[3]);

      // every shared-memory operand of this stage now sits in registers: release the stage and
      // make sure the next one has landed
      __syncwarp();
      if (lane == 0) mbar_arrive(empty0 + s * 8);
      const bool more = n + 1 < NT;
      const int s1 = (n + 1) % K2_STAGES;
      const uint32_t sp1 = sbase + s1 * SM::STAGE;
      const uint8_t* spg1 = smem + s1 * SM::STAGE;
      if (more) {
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(full0 + s1 * 8, ((n + 1) / K2_STAGES) & 1, sAbort))) {
          if (*sAbort == 0) { *sAbort = 1; atomicExch(p.status, ST_K2_FULL_TIMEOUT); }
          failed = true;
          break;
        }
      }
      K2_STAMP(3)

      // P2: h += v_new^T kg  (hi*hi, then lo*hi, then hi*lo: three passes over independent tiles),
      // interleaved with the next step's operand loads
#pragma unroll
      for (int np = 0; np < NTL / 2; ++np) {
        mma_bf16_v(hs[2 * np], avh, kgh[np][0], kgh[np][1]);
        mma_bf16_v(hs[2 * np + 1], avh, kgh[np][2], kgh[np][3]);
        if (more) ldsm_x4(sp1 + REC_W + swz_off(p1_row, np * 16 + p1_col), bw[np][0], bw[np][1], bw[np][2], bw[np][3]);
      }
#pragma unroll
      for (int np = 0; np < NTL / 2; ++np) {
        mma_bf16_v(hs[2 * np], avl, kgh[np][0], kgh[np][1]);
        mma_bf16_v(hs[2 * np + 1], avl, kgh[np][2], kgh[np][3]);
        if (!STATE_ONLY && more)
          ldsm_x4(sp1 + REC_QG + swz_off(p1_row, np * 16 + p1_col), bq[np][0], bq[np][1], bq[np][2], bq[np][3]);
      }
#pragma unroll
      for (int np = 0; np < NTL / 2; ++np) {
        mma_bf16_v(hs[2 * np], avh, kgl[np][0], kgl[np][1]);
        mma_bf16_v(hs[2 * np + 1], avh, kgl[np][2], kgl[np][3]);
        if (more) {
          dec[2 * np] = *reinterpret_cast<const float2*>(spg1 + REC_DEC + (kbase + (2 * np) * 8 + tq * 2) * 4);
          dec[2 * np + 1] = *reinterpret_cast<const float2*>(spg1 + REC_DEC + (kbase + (2 * np + 1) * 8 + tq * 2) * 4);
        }
      }
      if (more && use_u) {
        u0 = *reinterpret_cast<const float4*>(spg1 + REC_SHARED_BYTES + vtl * REC_U_TILE_BYTES + lane * 16);
        u1 = *reinterpret_cast<const float4*>(spg1 + REC_SHARED_BYTES + vtl * REC_U_TILE_BYTES + (32 + lane) * 16);
      }

      K2_STAMP(4)
      // P3: o^T = scale * (h qg^T) + v_new^T Aqk^T for this warp's token tile(s)
      if (!STATE_ONLY && o_owner) {
#pragma unroll
        for (int jj = 0; jj < OJ; ++jj) {
          const int j = oj0 + jj;                 // token tile: tokens 8j .. 8j+7
#pragma unroll
          for (int e = 0; e < 4; ++e) oa[jj][e] = p.scale * sq[jj][e];
          const uint32_t bh0 = (j == 0) ? ba[0] : ba[2], bh1 = (j == 0) ? ba[1] : ba[3];
          const uint32_t bl0 = (j == 0) ? bl[0] : bl[2], bl1 = (j == 0) ? bl[1] : bl[3];
          mma_bf16_v(oa[jj], avh, bh0, bh1);
          mma_bf16_v(oa[jj], avl, bh0, bh1);
          mma_bf16_v(oa[jj], avh, bl0, bl1);
        }
      }
      K2_STAMP(5)
      K2_STAMP(6)
      K2_STAMP(7)
    }
    // the last chunk's output tile (it may be a partial chunk)
    if (!STATE_ONLY && o_owner && !failed) {
#pragma unroll
      for (int jj = 0; jj < OJ; ++jj) {
        const int tok = (NT - 1) * BT + (oj0 + jj) * 8 + tq * 2;
        __nv_bfloat16* op = ob + static_cast<int64_t>(tok) * p.o_s[1];
        if (tok < p.T) {
          op[0] = __float2bfloat16_rn(oa[jj][0]);
          op[8] = __float2bfloat16_rn(oa[jj][2]);
        }
        if (tok + 1 < p.T) {
          op[p.o_s[1]] = __float2bfloat16_rn(oa[jj][1]);
          op[p.o_s[1] + 8] = __float2bfloat16_rn(oa[jj][3]);
        }
      }
    }

#ifdef KDA_K2_PROFILE
    failed = true;   // ht holds clock stamps
#endif
    if (!failed && p.ht != nullptr) {
      float* ht = p.ht + static_cast<size_t>(bh) * D * D;
#pragma unroll
      for (int nt = 0; nt < NTL; ++nt) {
        *reinterpret_cast<float2*>(ht + (vrow0 + gq) * D + kbase + nt * 8 + tq * 2) = make_float2(hs[nt][0], hs[nt][1]);
        *reinterpret_cast<float2*>(ht + (vrow0 + gq + 8) * D + kbase + nt * 8 + tq * 2) = make_float2(hs[nt][2], hs[nt][3]);
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

template <int VW, int KS, bool STATE_ONLY>
static cudaError_t launch_k2_t(const K2Params& p, cudaStream_t stream) {
  constexpr int smem_bytes = K2Smem<VW, KS>::TOTAL;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kda_k2_kernel<VW, KS, STATE_ONLY>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const int nblocks = p.B * p.H * (8 / VW);
  kda_k2_kernel<VW, KS, STATE_ONLY><<<nblocks, (VW * KS + 1) * 32, smem_bytes, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_k2(const K2Params& p, int vsplit, int ksplit, bool state_only, cudaStream_t stream) {
#define KDA_K2_CASE(NVV, KSS)                                                                   \
  if (vsplit == NVV && ksplit == KSS)                                                           \
    return state_only ? launch_k2_t<8 / NVV, KSS, true>(p, stream) : launch_k2_t<8 / NVV, KSS, false>(p, stream);
  KDA_K2_CASE(1, 1)
  KDA_K2_CASE(2, 1)
  KDA_K2_CASE(4, 1)
  KDA_K2_CASE(8, 1)
  KDA_K2_CASE(2, 2)
  KDA_K2_CASE(4, 2)
  KDA_K2_CASE(8, 2)
  KDA_K2_CASE(4, 4)
  KDA_K2_CASE(8, 4)
#undef KDA_K2_CASE
  return cudaErrorInvalidValue;
}

}  // namespace kda
