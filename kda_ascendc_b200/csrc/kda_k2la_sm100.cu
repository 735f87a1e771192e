// K2, look-ahead form: delta-rule state recurrence and output of the KDA forward.  sm_100a.
//
// Replaces kda_bt16_kernel_k2 of the reference (src/kda_bt16/kernels.py:187-302); the arithmetic
// is the recurrence of the reference's torch chunk implementation
// (tests/test_torch_reference.py:175-194), V-first state S[V][K]:
//   V_n = u_n - w_n S_n^T ;  o_n = scale (qg_n S_n^T) + Aqk_n V_n ;  S_{n+1} = S_n diag(dec_n) + V_n^T kg_n
//
// Written that way every chunk is one link of a serial chain S_n -> V_n -> S_{n+1}: the products with
// the state cannot start before the previous update has finished, and a warp that is alone on its SM
// sub-partition spends two thirds of a step waiting for its own results.  This kernel breaks the link
// with the identity (exact in real arithmetic)
//   x S_{n+1}^T = x (S_n diag(dec_n))^T + (x kg_n^T) V_n            for x = w_{n+1}, qg_{n+1}
// The first term needs only the decayed OLD state X_n = S_n diag(dec_n); the second is a 16x16
// state-independent "cross Gram" (C_{n+1} = w_{n+1} kg_n^T, A'_{n+1} = qg_{n+1} kg_n^T) times the V_n the
// step has anyway.  So in step n the products of chunk n+1 with X_n, the state update with V_n, the
// cross Gram of chunk n+2 and the output of chunk n are all independent of one another: the step is
// one stream of 53 tensor-core instructions without a dependent hand-over inside, and the chain
// S_n -> X_n -> V_{n+1} -> S_{n+2} spans two steps.
//
// Mapping (as in the plain 8-row form): the recurrence is independent per state row v, a warp owns
// 8 rows and keeps them transposed, hT[k][v], in m16n8 accumulator fragments for the whole sequence;
// V is the MMA N dimension.  Per chunk and warp:
//   P1  [pw | pq] = [w ; qg]_{n+1} X_n          M = 16+16 tokens, N = 8 v, K = 128      16 MMAs
//   X   pw += C_{n+1} V_n ; pq += A'_{n+1} V_n  M = 16, N = 8, K = 16                   2 MMAs
//   P2  hT = hT dec_n + kg_n^T V_n              M = 128 k, N = 8 v, K = 16, hi/lo split 24 MMAs
//   P3  o_n = scale pq_n + Aqk_n V_n            hi/lo split                             3 MMAs
//   G   one 16x8 tile of [C ; A']_{n+2} = [w ; qg]_{n+2} kg_{n+1}^T, K = 128            8 MMAs
// The four G tiles of a chunk are shared by the consumer warps of the CTA through shared memory (one
// tile each with four warps), a step ahead of their use, so the exchange never stalls.  Rounding: the
// cross Grams are kept in bf16 and multiply the bf16 high part of V_n -- the same class of error as
// the bf16 state snapshot they replace; P2 and P3 keep their hi/lo splits (the state must stay within
// 2e-3 of an fp32 implementation).  The result does not depend on how the rows are spread over warps
// and CTAs.
//
// Measured on B200 (B1 T8192 H32, K2 alone): 418 us against 282 us for the plain 8-row form, and 294 us
// even with the cross Grams left out: with the dependent chain gone the step is still bound by the
// shared-memory traffic of the operand fragments (every warp reads all four tiles of the chunk) and
// by the warp's serial issue of about 8 cycles per mma.sync.  This form is therefore never chosen
// automatically; it stays selectable (k2_variant 5) as the measured answer to "would cutting the
// dependent steps help", with its own parity tests.
//
// A CTA = CW consumer warps (CW*8 state rows of one (batch, head)) plus one producer warp that streams
// the chunk records through a ring of shared-memory stages with bulk (TMA) copies: full/empty
// mbarriers, every wait bounded.  Step n reads records n (kg, Aqk, dec), n+1 (w, qg, u, kg) and n+2
// (w, qg).
#include <type_traits>

#include "kda_common.cuh"
#include "kda_kernels.h"

namespace kda {

constexpr int K2L_STAGES = 8;
constexpr int ST_K2_XCHG_TIMEOUT = 4;

template <int CW>
struct K2LSmem {
  static constexpr int STAGE = REC_SHARED_BYTES + CW * REC_U_TILE_BYTES;
  static constexpr int XG = K2L_STAGES * STAGE;                 // 2 x {C tile, A' tile}, 512 B each
  static constexpr int BARS = XG + 2 * 1024;                    // full[S], empty[S], xbar[2]
  static constexpr int FLAG = BARS + (2 * K2L_STAGES + 2) * 8;  // abort flag, issued count
  static constexpr int TOTAL = FLAG + 16;
};

template <int CW, bool STATE_ONLY>
__global__ void __launch_bounds__((CW + 1) * 32, 1) kda_k2la_kernel(const K2Params p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  using SM = K2LSmem<CW>;
  constexpr int S = K2L_STAGES;
  constexpr int VCOLS = CW * 8;   // state rows (v) per CTA
  constexpr int NV = D / VCOLS;   // CTAs per (batch, head)
  // cross-Gram tiles per chunk: (w | qg) x (first | second half of the previous chunk's tokens)
  constexpr int NTILES = STATE_ONLY ? 2 : 4;
  constexpr int TPW = (NTILES + CW - 1) / CW;   // tiles per consumer warp
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int bh = blockIdx.x / NV + p.chain0;
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
  const uint32_t empty0 = full0 + S * 8;
  const uint32_t xbar0 = empty0 + S * 8;
  volatile int* sAbort = reinterpret_cast<volatile int*>(smem + SM::FLAG);
  volatile int* sIssued = sAbort + 1;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full0 + s * 8, 1);
      mbar_init(empty0 + s * 8, CW);
    }
    mbar_init(xbar0, CW);
    mbar_init(xbar0 + 8, CW);
    *sAbort = 0;
    *sIssued = 0;
    fence_mbar_init();
  }
  __syncthreads();

  const uint8_t* rec_bh = p.rec + rec_first * REC_BYTES;

  if (warp == CW) {
    // ------------------------------ producer -------------------------------
    if (lane == 0) {
      int s = 0, round = 0;   // record n sits in slot n % S, round n / S
      for (int n = 0; n < NT; ++n) {
        if (round > 0) {
          if (!mbar_wait_bounded(empty0 + s * 8, (round - 1) & 1, sAbort)) {
            if (*sAbort == 0) { *sAbort = 1; atomicExch(p.status, ST_K2_EMPTY_TIMEOUT); }
            break;
          }
        }
        const uint8_t* rec = rec_bh + static_cast<size_t>(n) * REC_BYTES;
        const uint32_t dst = sbase + s * SM::STAGE;
        mbar_arrive_expect_tx(full0 + s * 8, SM::STAGE);
        bulk_g2s(dst, rec, REC_SHARED_BYTES, full0 + s * 8);
        bulk_g2s(dst + REC_SHARED_BYTES, rec + REC_U + vs * (CW * REC_U_TILE_BYTES), CW * REC_U_TILE_BYTES,
                 full0 + s * 8);
        *sIssued = n + 1;
        if (++s == S) { s = 0; ++round; }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ consumers ------------------------------
    const int gq = lane >> 2, tq = lane & 3;
    const int v0 = vs * VCOLS + warp * 8;   // first state row of this warp
    // hT[m][e]: k = 16m + gq (+8 for e >= 2), v = v0 + 2tq + (e & 1)
    float hT[8][4];
    if (p.h0 != nullptr) {
      const float* h0 = p.h0 + static_cast<size_t>(bh) * D * D;
#pragma unroll
      for (int m = 0; m < 8; ++m)
#pragma unroll
        for (int e = 0; e < 4; ++e)
          hT[m][e] = p.k_first ? h0[(m * 16 + gq + (e >> 1) * 8) * D + v0 + tq * 2 + (e & 1)]
                               : h0[(v0 + tq * 2 + (e & 1)) * D + m * 16 + gq + (e >> 1) * 8];
    } else {
#pragma unroll
      for (int m = 0; m < 8; ++m) hT[m][0] = hT[m][1] = hT[m][2] = hT[m][3] = 0.f;
    }

    // per-lane ldmatrix address components (constant across steps).  A swizzled tile address of
    // k-step ks is (256-byte aligned tile base + lane part) ^ (ks << 5): the k-step only moves bits
    // 5..7, which the tile bases leave clear.
    static_assert(SM::STAGE % 256 == 0 && REC_W % 256 == 0 && REC_QG % 256 == 0 && REC_KGH % 256 == 0 && REC_KGL % 256 == 0,
                  "tile bases must keep address bits 5..7 clear");
    const int a1_row = (lane & 7) + ((lane >> 3) & 1) * 8, a1_col = (lane >> 4) * 8;   // [w;qg]: rows tok, cols k
    const int a2_row = (lane & 7) + (lane >> 4) * 8, a2_col = ((lane >> 3) & 1) * 8;   // kg^T via .trans
    const uint32_t a1_lane = swz_off(a1_row, a1_col), a2_lane = swz_off(a2_row, a2_col);
    const uint32_t a3_off = (a1_row * 16 + a1_col) * 2;                                // 16x16 tiles: rows i, cols j
    const uint32_t u_off = REC_SHARED_BYTES + warp * REC_U_TILE_BYTES + lane * 16;
    // this warp's cross-Gram tiles: tile t -> part (0 = w -> C, 1 = qg -> A'), half of the 16 kg rows
    const int tile0 = warp * TPW;
    const bool has_tile = tile0 < NTILES;
    uint32_t g_aoff[TPW], g_blane[TPW], g_xoff[TPW];
#pragma unroll
    for (int t = 0; t < TPW; ++t) {
      const int tile = (tile0 + t) % NTILES, part = tile >> 1, half = tile & 1;
      g_aoff[t] = part ? REC_QG : REC_W;
      g_blane[t] = swz_off(8 * half + (lane & 7), ((lane >> 3) & 1) * 8) + REC_KGH;
      g_xoff[t] = SM::XG + part * 512 + (gq * 16 + 8 * half + 2 * tq) * 2;
    }
    __nv_bfloat16* const ob = STATE_ONLY ? nullptr : p.o + b * p.o_s[0] + tok0 * p.o_s[1] + h * p.o_s[2] + v0 + tq * 2;
    const bool use_u = !(STATE_ONLY && p.zero_u);

    bool failed = false;
    auto give_up = [&](int code) {
      if (*sAbort == 0) { *sAbort = 1; atomicExch(p.status, code); }
      failed = true;
    };
    auto wait_full = [&](int s, int ph) {
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(full0 + s * 8, ph, sAbort))) give_up(ST_K2_FULL_TIMEOUT);
    };

    // One 16x8 cross-Gram tile per t: rows = tokens of the chunk in stage sa, columns = 8 kg rows of
    // the chunk in stage sb; rounded to bf16 into the exchange buffer xb.
    auto cross_gram_now = [&](uint32_t spa, uint32_t spb, int xb) {
#pragma unroll
      for (int t = 0; t < TPW; ++t) {
        float acc[2][4];
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          uint32_t a[4], b0, b1;
          ldsm_x4(((spa + a1_lane) ^ (ks << 5)) + g_aoff[t], a[0], a[1], a[2], a[3]);
          ldsm_x2(((spb + g_blane[t]) ^ (ks << 5)), b0, b1);
          if (ks < 2) mma_bf16_z(acc[ks & 1], a, b0, b1);
          else mma_bf16_v(acc[ks & 1], a, b0, b1);
        }
        *reinterpret_cast<uint32_t*>(smem + g_xoff[t] + xb * 1024) = pack_bf16(acc[0][0] + acc[1][0], acc[0][1] + acc[1][1]);
        *reinterpret_cast<uint32_t*>(smem + g_xoff[t] + xb * 1024 + 8 * 32) = pack_bf16(acc[0][2] + acc[1][2], acc[0][3] + acc[1][3]);
      }
    };

    // ---- prologue: records 0..2, products of chunk 0 with the initial state, V_0, C_1 ----
    wait_full(0, 0);
    if (!failed && NT > 1) wait_full(1, 0);
    if (!failed && NT > 2) wait_full(2, 0);

    float pq[4] = {0.f, 0.f, 0.f, 0.f};      // qg_n X_{n-1}^T + A'_n V_{n-1} of the current chunk
    float oa[4] = {0.f, 0.f, 0.f, 0.f};      // output tile of the previous step, stored one step late
    uint32_t bvh[2] = {0u, 0u}, bvl[2] = {0u, 0u};   // B fragments of V_n, hi / lo
    if (!failed) {
      float pw[2][4] = {}, pq2[2][4] = {};
      if (p.h0 != nullptr) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          uint32_t a[4];
          const uint32_t b0 = movmatrix_t(pack_bf16(hT[ks][0], hT[ks][1])), b1 = movmatrix_t(pack_bf16(hT[ks][2], hT[ks][3]));
          ldsm_x4(((sbase + a1_lane) ^ (ks << 5)) + REC_W, a[0], a[1], a[2], a[3]);
          mma_bf16_v(pw[ks & 1], a, b0, b1);
          if (!STATE_ONLY) {
            ldsm_x4(((sbase + a1_lane) ^ (ks << 5)) + REC_QG, a[0], a[1], a[2], a[3]);
            mma_bf16_v(pq2[ks & 1], a, b0, b1);
          }
        }
      }
      const float4 u0 = use_u ? *reinterpret_cast<const float4*>(smem + u_off) : make_float4(0, 0, 0, 0);
      uint32_t h01, l01, h23, l23;
      split_pack(u0.x - (pw[0][0] + pw[1][0]), u0.y - (pw[0][1] + pw[1][1]), h01, l01);
      split_pack(u0.z - (pw[0][2] + pw[1][2]), u0.w - (pw[0][3] + pw[1][3]), h23, l23);
      bvh[0] = movmatrix_t(h01); bvh[1] = movmatrix_t(h23);
      bvl[0] = movmatrix_t(l01); bvl[1] = movmatrix_t(l23);
#pragma unroll
      for (int e = 0; e < 4; ++e) pq[e] = pq2[0][e] + pq2[1][e];
      if (NT > 1) {
        if (has_tile) cross_gram_now(sbase + SM::STAGE, sbase, 1);   // [C ; A']_1 -> buffer 1
        __syncwarp();
        if (lane == 0) mbar_arrive(xbar0 + 8);
      }
    }

    // stage indices of records n, n+1, n+2, and of the record to wait for at the end of a step (n+3)
    int s0 = 0, s1 = 1 % S, s2 = 2 % S, sw = 3 % S, phw = (3 / S) & 1;
    // phase parity of the two exchange barriers: xph[b] = parity to wait for at the next use of buffer b
    int xph0 = 0, xph1 = 0;

    auto step = [&](auto more_c, auto more2_c, int n) {
      constexpr bool MORE = decltype(more_c)::value;     // chunk n+1 exists
      constexpr bool MORE2 = decltype(more2_c)::value;   // chunk n+2 exists
      const uint32_t sp0 = sbase + s0 * SM::STAGE, sp1 = sbase + s1 * SM::STAGE, sp2 = sbase + s2 * SM::STAGE;
      const uint8_t* spg0 = smem + s0 * SM::STAGE;
      const uint8_t* spg1 = smem + s1 * SM::STAGE;
      const uint32_t t0k = sp0 + a2_lane, t1a = sp1 + a1_lane, t2a = sp2 + a1_lane;
      const int xb = (n + 1) & 1;   // exchange buffer of [C ; A']_{n+1}; that of chunk n+2 is xb ^ 1

      // the previous step's output tile (always a full chunk)
      if (!STATE_ONLY && n > 0) {
        __nv_bfloat16* op = ob + static_cast<int64_t>((n - 1) * BT + gq) * p.o_s[1];
        *reinterpret_cast<uint32_t*>(op) = pack_bf16(oa[0], oa[1]);
        *reinterpret_cast<uint32_t*>(op + 8 * p.o_s[1]) = pack_bf16(oa[2], oa[3]);
      }

      uint32_t kgh[8][4], kgl[8][4], aw[8][4], aq[8][4], ga[TPW][8][4], gb[TPW][8][2];
      float dk[8][2];
      // the record the NEXT step needs first: probe its barrier now, look at the answer at the end
      const bool next_ready = (n + 3 < NT) ? mbar_test_wait(full0 + sw * 8, phw) : true;
#pragma unroll
      for (int m = 0; m < 8; ++m) {
        dk[m][0] = *reinterpret_cast<const float*>(spg0 + REC_DEC + (m * 16 + gq) * 4);
        dk[m][1] = *reinterpret_cast<const float*>(spg0 + REC_DEC + (m * 16 + gq + 8) * 4);
      }
      auto load_pair = [&](int m0) {
#pragma unroll
        for (int m = m0; m < m0 + 2; ++m) {
          if (MORE) {
            ldsm_x4((t1a ^ (m << 5)) + REC_W, aw[m][0], aw[m][1], aw[m][2], aw[m][3]);
            if (!STATE_ONLY) ldsm_x4((t1a ^ (m << 5)) + REC_QG, aq[m][0], aq[m][1], aq[m][2], aq[m][3]);
          }
          ldsm_x4_t((t0k ^ (m << 5)) + REC_KGH, kgh[m][0], kgh[m][1], kgh[m][2], kgh[m][3]);
          ldsm_x4_t((t0k ^ (m << 5)) + REC_KGL, kgl[m][0], kgl[m][1], kgl[m][2], kgl[m][3]);
          if (MORE2 && has_tile) {
#pragma unroll
            for (int t = 0; t < TPW; ++t) {
              ldsm_x4((t2a ^ (m << 5)) + g_aoff[t], ga[t][m][0], ga[t][m][1], ga[t][m][2], ga[t][m][3]);
              ldsm_x2(((sp1 + g_blane[t]) ^ (m << 5)), gb[t][m][0], gb[t][m][1]);
            }
          }
        }
      };
      load_pair(0);

      // cross terms of chunk n+1 with V_n, from the exchange buffer written one step ago
      float pwn[2][4], pqn[2][4], gacc[TPW][2][4];
      float4 un = make_float4(0, 0, 0, 0);
      uint32_t ah3[4], al3[4], cfw[4], cfq[4];
      if (!STATE_ONLY) {
        ldsm_x4(sp0 + REC_AQK + a3_off, ah3[0], ah3[1], ah3[2], ah3[3]);
        ldsm_x4(sp0 + REC_AQL + a3_off, al3[0], al3[1], al3[2], al3[3]);
#pragma unroll
        for (int e = 0; e < 4; ++e) oa[e] = p.scale * pq[e];
      }
      if (MORE) {
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(xbar0 + xb * 8, xb ? xph1 : xph0, sAbort))) {
          give_up(ST_K2_XCHG_TIMEOUT);
          return;
        }
        if (xb) xph1 ^= 1; else xph0 ^= 1;
        ldsm_x4(sbase + SM::XG + xb * 1024 + a3_off, cfw[0], cfw[1], cfw[2], cfw[3]);
        if (!STATE_ONLY) ldsm_x4(sbase + SM::XG + xb * 1024 + 512 + a3_off, cfq[0], cfq[1], cfq[2], cfq[3]);
        if (use_u) un = *reinterpret_cast<const float4*>(spg1 + u_off);
      }

      // decay of the fp32 state, and B fragments of its bf16 snapshot X_n (accumulator fragment ->
      // pack -> 8x8 transpose); done one pair ahead of the MMAs that read them
      uint32_t bx[8][2];
      auto snap_pair = [&](int m0) {
#pragma unroll
        for (int m = m0; m < m0 + 2; ++m) {
          const float2 lo = __fmul2_rn(make_float2(hT[m][0], hT[m][1]), make_float2(dk[m][0], dk[m][0]));
          const float2 hi = __fmul2_rn(make_float2(hT[m][2], hT[m][3]), make_float2(dk[m][1], dk[m][1]));
          hT[m][0] = lo.x; hT[m][1] = lo.y; hT[m][2] = hi.x; hT[m][3] = hi.y;
          if (MORE) {
            bx[m][0] = movmatrix_t(pack_bf16(lo.x, lo.y));
            bx[m][1] = movmatrix_t(pack_bf16(hi.x, hi.y));
          }
        }
      };
      snap_pair(0);

#pragma unroll
      for (int m = 0; m < 8; m += 2) {
        if (m + 2 < 8) {
          load_pair(m + 2);
          snap_pair(m + 2);
        }
        // dependent MMAs (same accumulator) are kept at least four instructions apart; the products
        // that do not need V_n go first
        if (MORE) {
          if (m == 0) {
            mma_bf16_z(pwn[0], aw[m], bx[m][0], bx[m][1]);
            mma_bf16_z(pwn[1], aw[m + 1], bx[m + 1][0], bx[m + 1][1]);
          } else {
            mma_bf16_v(pwn[0], aw[m], bx[m][0], bx[m][1]);
            mma_bf16_v(pwn[1], aw[m + 1], bx[m + 1][0], bx[m + 1][1]);
          }
        }
        mma_bf16_v(hT[m], kgh[m], bvh[0], bvh[1]);
        mma_bf16_v(hT[m + 1], kgh[m + 1], bvh[0], bvh[1]);
        if (MORE && !STATE_ONLY) {
          if (m == 0) {
            mma_bf16_z(pqn[0], aq[m], bx[m][0], bx[m][1]);
            mma_bf16_z(pqn[1], aq[m + 1], bx[m + 1][0], bx[m + 1][1]);
          } else {
            mma_bf16_v(pqn[0], aq[m], bx[m][0], bx[m][1]);
            mma_bf16_v(pqn[1], aq[m + 1], bx[m + 1][0], bx[m + 1][1]);
          }
        }
        mma_bf16_v(hT[m], kgh[m], bvl[0], bvl[1]);
        mma_bf16_v(hT[m + 1], kgh[m + 1], bvl[0], bvl[1]);
        if (MORE2 && has_tile) {
#pragma unroll
          for (int t = 0; t < TPW; ++t) {
            if (m == 0) {
              mma_bf16_z(gacc[t][0], ga[t][m], gb[t][m][0], gb[t][m][1]);
              mma_bf16_z(gacc[t][1], ga[t][m + 1], gb[t][m + 1][0], gb[t][m + 1][1]);
            } else {
              mma_bf16_v(gacc[t][0], ga[t][m], gb[t][m][0], gb[t][m][1]);
              mma_bf16_v(gacc[t][1], ga[t][m + 1], gb[t][m + 1][0], gb[t][m + 1][1]);
            }
          }
        }
        // P3 (o_n = scale pq_n + Aqk_n V_n) and the cross terms of chunk n+1, spread over the pairs
        if (!STATE_ONLY) {
          if (m == 0) mma_bf16_v(oa, ah3, bvh[0], bvh[1]);
          if (m == 2) mma_bf16_v(oa, ah3, bvl[0], bvl[1]);
          if (m == 4) mma_bf16_v(oa, al3, bvh[0], bvh[1]);
        }
        if (MORE) {
          if (m == 2) mma_bf16_v(pwn[0], cfw, bvh[0], bvh[1]);
          if (m == 4 && !STATE_ONLY) mma_bf16_v(pqn[0], cfq, bvh[0], bvh[1]);
        }
        mma_bf16_v(hT[m], kgl[m], bvh[0], bvh[1]);
        mma_bf16_v(hT[m + 1], kgl[m + 1], bvh[0], bvh[1]);
      }

      // every load from stage s0 has been consumed by an issued MMA: hand the stage back
      __syncwarp();
      if (lane == 0) mbar_arrive(empty0 + s0 * 8);

      // publish this warp's tiles of [C ; A']_{n+2}
      if (MORE2) {
        if (has_tile) {
#pragma unroll
          for (int t = 0; t < TPW; ++t) {
            uint8_t* x = smem + g_xoff[t] + (xb ^ 1) * 1024;
            *reinterpret_cast<uint32_t*>(x) = pack_bf16(gacc[t][0][0] + gacc[t][1][0], gacc[t][0][1] + gacc[t][1][1]);
            *reinterpret_cast<uint32_t*>(x + 8 * 32) = pack_bf16(gacc[t][0][2] + gacc[t][1][2], gacc[t][0][3] + gacc[t][1][3]);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(xbar0 + (xb ^ 1) * 8);
      }

      // V_{n+1} and the products of chunk n+1 for the next step
      if (MORE) {
        uint32_t h01, l01, h23, l23;
        split_pack((un.x - pwn[1][0]) - pwn[0][0], (un.y - pwn[1][1]) - pwn[0][1], h01, l01);
        split_pack((un.z - pwn[1][2]) - pwn[0][2], (un.w - pwn[1][3]) - pwn[0][3], h23, l23);
        bvh[0] = movmatrix_t(h01); bvh[1] = movmatrix_t(h23);
        bvl[0] = movmatrix_t(l01); bvl[1] = movmatrix_t(l23);
        if (!STATE_ONLY) {
#pragma unroll
          for (int e = 0; e < 4; ++e) pq[e] = pqn[0][e] + pqn[1][e];
        }
      }

      // the next step also reads record n+3
      if (!__all_sync(0xffffffffu, next_ready)) wait_full(sw, phw);
      s0 = s1; s1 = s2; s2 = sw;
      if (++sw == S) { sw = 0; phw ^= 1; }
    };

    if (!failed) {
      int n = 0;
      for (; n + 2 < NT && !failed; ++n) step(std::true_type{}, std::true_type{}, n);
      if (n + 1 < NT && !failed) { step(std::true_type{}, std::false_type{}, n); ++n; }
      if (n < NT && !failed) step(std::false_type{}, std::false_type{}, n);
    }

    // the last chunk's output tile (it may be a partial chunk)
    if (!STATE_ONLY && !failed) {
      const int tok = (NT - 1) * BT + gq;
      __nv_bfloat16* op = ob + static_cast<int64_t>(tok) * p.o_s[1];
      if (tok < Tlen) *reinterpret_cast<uint32_t*>(op) = pack_bf16(oa[0], oa[1]);
      if (tok + 8 < Tlen) *reinterpret_cast<uint32_t*>(op + 8 * p.o_s[1]) = pack_bf16(oa[2], oa[3]);
    }

    if (!failed && p.ht != nullptr) {
      float* ht = p.ht + static_cast<size_t>(bh) * D * D;
#pragma unroll
      for (int m = 0; m < 8; ++m)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if (p.k_first) ht[(m * 16 + gq + (e >> 1) * 8) * D + v0 + tq * 2 + (e & 1)] = hT[m][e];
          else ht[(v0 + tq * 2 + (e & 1)) * D + m * 16 + gq + (e >> 1) * 8] = hT[m][e];
        }
    }
  }

  __syncthreads();
  if (*sAbort != 0 && tid == 0) {
    // give copies that are still in flight a bounded chance to land before the CTA's shared memory
    // is released
    const int issued = *sIssued;
    for (int n = max(0, issued - S); n < issued; ++n)
      mbar_wait_bounded(full0 + (n % S) * 8, (n / S) & 1, nullptr);
  }
}

template <int CW, bool STATE_ONLY>
static cudaError_t launch_k2la_t(const K2Params& p, cudaStream_t stream) {
  constexpr int smem_bytes = K2LSmem<CW>::TOTAL;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kda_k2la_kernel<CW, STATE_ONLY>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         smem_bytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const int nblocks = (p.n_chains > 0 ? p.n_chains : (p.seq_table != nullptr ? p.n_seqs : p.B) * p.H) * (D / (CW * 8));
  kda_k2la_kernel<CW, STATE_ONLY><<<nblocks, (CW + 1) * 32, smem_bytes, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_k2la(const K2Params& p, int vsplit, bool state_only, cudaStream_t stream) {
  // vsplit CTAs per head, 8 state rows per warp  =>  16 / vsplit consumer warps per CTA
#define KDA_K2LA_CASE(VS, CW_) \
  if (vsplit == VS) return state_only ? launch_k2la_t<CW_, true>(p, stream) : launch_k2la_t<CW_, false>(p, stream);
  KDA_K2LA_CASE(4, 4)
  KDA_K2LA_CASE(8, 2)
  KDA_K2LA_CASE(16, 1)
#undef KDA_K2LA_CASE
  return cudaErrorInvalidValue;
}

}  // namespace kda
