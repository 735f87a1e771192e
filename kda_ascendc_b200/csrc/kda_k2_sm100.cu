// K2: delta-rule state recurrence and output of the KDA forward.  sm_100a.
//
// Replaces kda_bt16_kernel_k2 of the reference (src/kda_bt16/kernels.py:187-302); the
// arithmetic is the recurrence of the reference's torch chunk implementation
// (tests/test_torch_reference.py:175-194), V-first state h[V][K]:
//   v_new = u - w h^T ;  o = scale (qg h^T) + Aqk v_new ;  h = h diag(dec) + v_new^T kg
//
// The recurrence is independent per state row v (v_new[:, v], o[:, v] and h[v, :] only use
// row v), so V is the dimension that is spread over warps.  It is mapped to the MMA *N*
// dimension, whose granularity is 8: a warp owns NVT tiles of 8 rows of h and keeps them,
// transposed, in registers for the whole sequence:  hT[k][v], fp32, m16n8 accumulator
// fragments (8 k-tiles of 16).  Per chunk, per warp:
//   P1: [v_new | o] = [w ; qg] hT       M = 16+16 tokens, N = 8 v, K = 128   (16 MMAs / tile)
//   P2: hT += kg^T v_new                M = 128 k,        N = 8 v, K = 16    (3 x 8 MMAs)
//   P3: o += Aqk v_new                  M = 16 tokens,    N = 8 v, K = 16    (3 MMAs)
// A operands ([w;qg], kg^T, Aqk) are state independent and come from the chunk record in
// shared memory by ldmatrix; B operands are the warp's own data (bf16(hT), v_new): an
// accumulator fragment becomes a B fragment by an in-warp 8x8 transpose (movmatrix), so the
// serial chain  hT -> P1 -> v_new -> P2 -> hT  never leaves the warp: no shared-memory round
// trip and no inter-warp synchronisation sits on it.  That chain, NT dependent steps per
// head, is what bounds this kernel, together with the legacy tensor pipe (one m16n8k16 per
// 8 cycles per SM sub-partition).  P2 uses a hi/lo bf16 split of both v_new and kg (three
// MMAs) because the state must stay within 2e-3 of an fp32 implementation; P3 does the same
// with v_new and Aqk (the intra-chunk term dominates o); P1 uses plain bf16 operands.
// The result does not depend on how the rows are distributed over warps and CTAs.
//
// One warp executes its chain in program order.  Measured on B200: an mma.sync holds the
// sub-partition's issue port for its 8 cycles (neither this warp nor another one on the same
// sub-partition issues meanwhile), so a step costs about 8 cycles per MMA plus 2 per other
// instruction and what matters is the instruction count.  Loads are still interleaved with the
// MMA sequences so that their latency is covered: P1 carries this step's kg fragment loads and
// the decay of hT; P2 carries the next step's [w;qg] / decay / u loads; the previous step's output
// tile is stored at the start of the next step.
//
// A CTA = CW consumer warps (CW*NVT*8 state rows of one (batch, head)) plus one producer warp
// that streams the chunk records through a ring of shared-memory stages with bulk (TMA)
// copies: full/empty mbarriers, every wait bounded.
#include "kda_common.cuh"
#include "kda_kernels.h"

namespace kda {

constexpr int K2_STAGES = 4;

// UT = 8-column u tiles a warp reads per step (its NVT row tiles; one in the transform-pair mode)
template <int CW, int UT>
struct K2Smem {
  static constexpr int STAGE = REC_SHARED_BYTES + CW * UT * REC_U_TILE_BYTES;
  static constexpr int BARS = K2_STAGES * STAGE;               // full[S], empty[S]
  static constexpr int FLAG = BARS + 2 * K2_STAGES * 8;        // abort flag, issued count
  static constexpr int TOTAL = FLAG + 16;
};

// PAIR (state-only, NVT = 2): the transform-pair pass of the sequence split.  The two 8-row tiles
// of a warp are the SAME eight state rows of two recurrences over the same records -- tile 0 starts
// from the identity with the u term dropped (the segment's transition matrix M), tile 1 from zero
// with u (its offset Q) -- so every operand fragment fetched from shared memory feeds two MMAs.
// The states leave as [chains][2][128][128].
template <int CW, int NVT, bool STATE_ONLY, bool PAIR = false>
__global__ void __launch_bounds__((CW + 1) * 32, 1) kda_k2_kernel(const K2Params p) {
  static_assert(!PAIR || (STATE_ONLY && NVT == 2), "the pair mode is a state-only pass over two tiles");
  extern __shared__ __align__(1024) uint8_t smem[];
  constexpr int RT = PAIR ? 1 : NVT;    // distinct 8-row tiles per warp
  using SM = K2Smem<CW, RT>;
  constexpr int VCOLS = CW * RT * 8;    // state rows (v) per CTA
  constexpr int NV = D / VCOLS;         // CTAs per (batch, head)
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  // chain: index of the recurrence this CTA works on.  With K2Params::pair_mode (state-only, one
  // tile per warp) the launch runs two chains per (batch, head): 2c from the identity without u,
  // 2c + 1 from zero with u, and writes them as [chains][2][128][128].
  const int chain = blockIdx.x / NV + p.chain0;
  const bool pair_rt = !PAIR && STATE_ONLY && p.pair_mode != 0;
  const int bh = pair_rt ? (chain >> 1) : chain;   // the (batch, head) whose records are walked
  const int plane = pair_rt ? (chain & 1) : 1;
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
  const uint32_t empty0 = full0 + K2_STAGES * 8;
  volatile int* sAbort = reinterpret_cast<volatile int*>(smem + SM::FLAG);
  volatile int* sIssued = sAbort + 1;

  if (tid == 0) {
    for (int s = 0; s < K2_STAGES; ++s) {
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
        bulk_g2s(dst + REC_SHARED_BYTES, rec + REC_U + vs * (CW * RT * REC_U_TILE_BYTES),
                 CW * RT * REC_U_TILE_BYTES, full0 + s * 8);
        *sIssued = n + 1;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ consumers ------------------------------
    const int gq = lane >> 2, tq = lane & 3;
    const int v0 = vs * VCOLS + warp * (RT * 8);   // first state row of this warp
    // hT[m][nv][e]: k = 16m + gq (+8 for e >= 2), v = v0 + 8nv + 2tq + (e & 1)   (PAIR: v = v0 + 2tq + (e & 1))
    float hT[8][NVT][4];
    bool h0_ok = true;
    if (PAIR) {
#pragma unroll
      for (int m = 0; m < 8; ++m)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          hT[m][0][e] = ((v0 + tq * 2 + (e & 1)) == (m * 16 + gq + (e >> 1) * 8)) ? 1.f : 0.f;
          hT[m][NVT - 1][e] = (NVT > 1) ? 0.f : hT[m][0][e];
        }
    } else if (pair_rt) {
#pragma unroll
      for (int m = 0; m < 8; ++m)
#pragma unroll
        for (int nv = 0; nv < NVT; ++nv)
#pragma unroll
          for (int e = 0; e < 4; ++e)
            hT[m][nv][e] = (plane == 0 && (v0 + nv * 8 + tq * 2 + (e & 1)) == (m * 16 + gq + (e >> 1) * 8)) ? 1.f : 0.f;
    } else if (p.h0 != nullptr) {
      if (p.h0_n_flags > 0) {   // the entry state comes from other GPUs: wait for their flags (the producer warp is already loading records)
        int ok = 1;
        if (lane == 0)
          for (int i = 0; i < p.h0_n_flags; ++i) ok &= flag_wait_bounded(p.h0_flags + i, p.h0_epoch) ? 1 : 0;
        h0_ok = __shfl_sync(0xffffffffu, ok, 0) != 0;
      }
      const float* h0 = p.h0 + static_cast<size_t>(bh) * D * D;
#pragma unroll
      for (int m = 0; m < 8; ++m)
#pragma unroll
        for (int nv = 0; nv < NVT; ++nv)
#pragma unroll
          for (int e = 0; e < 4; ++e)
            hT[m][nv][e] = p.k_first ? h0[(m * 16 + gq + (e >> 1) * 8) * D + v0 + nv * 8 + tq * 2 + (e & 1)]
                                     : h0[(v0 + nv * 8 + tq * 2 + (e & 1)) * D + m * 16 + gq + (e >> 1) * 8];
    } else {
#pragma unroll
      for (int m = 0; m < 8; ++m)
#pragma unroll
        for (int nv = 0; nv < NVT; ++nv) hT[m][nv][0] = hT[m][nv][1] = hT[m][nv][2] = hT[m][nv][3] = 0.f;
    }

    // per-lane ldmatrix address components (constant across steps)
    const int a1_row = (lane & 7) + ((lane >> 3) & 1) * 8, a1_col = (lane >> 4) * 8;   // [w;qg]: rows tok, cols k
    const int a2_row = (lane & 7) + (lane >> 4) * 8, a2_col = ((lane >> 3) & 1) * 8;   // kg^T via .trans
    const uint32_t a3_off = REC_AQK + (a1_row * 16 + a1_col) * 2;                      // Aqk: rows i, cols j
    // Swizzled tile address of k-step ks = (256-byte aligned tile base + lane part) ^ (ks << 5): the
    // k-step only moves bits 5..7 of the address, which the tile base leaves clear (stages and tile
    // offsets are multiples of 256 bytes), so one XOR with an immediate replaces the index arithmetic.
    static_assert(SM::STAGE % 256 == 0 && REC_W % 256 == 0 && REC_QG % 256 == 0 && REC_KGH % 256 == 0 && REC_KGL % 256 == 0,
                  "tile bases must keep address bits 5..7 clear");
    const uint32_t a1_lane = swz_off(a1_row, a1_col), a2_lane = swz_off(a2_row, a2_col);
    const uint32_t u_off = REC_SHARED_BYTES + warp * (RT * REC_U_TILE_BYTES) + lane * 16;
    __nv_bfloat16* const ob = STATE_ONLY ? nullptr : p.o + b * p.o_s[0] + tok0 * p.o_s[1] + h * p.o_s[2] + v0 + tq * 2;
    const bool use_u = PAIR || (pair_rt ? plane == 1 : !(STATE_ONLY && p.zero_u));

    uint32_t aw[8][4], aq[8][4];     // A fragments of w and qg (one per 16-wide k-step)
    float dk[8][2];                  // decay of the rows k = 16m+gq and 16m+gq+8
    float4 u[NVT];
    float oa[NVT][4];                // output tile of the previous step, stored one step late

    bool failed = false;
    if (!h0_ok) {
      if (*sAbort == 0) { *sAbort = 1; atomicExch(p.status, ST_PEER_TIMEOUT); }
      failed = true;
    } else if (!__all_sync(0xffffffffu, mbar_wait_bounded(full0, 0, sAbort))) {
      if (*sAbort == 0) { *sAbort = 1; atomicExch(p.status, ST_K2_FULL_TIMEOUT); }
      failed = true;
    } else {
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        ldsm_x4(((sbase + a1_lane) ^ (ks << 5)) + REC_W, aw[ks][0], aw[ks][1], aw[ks][2], aw[ks][3]);
        if (!STATE_ONLY)
          ldsm_x4(((sbase + a1_lane) ^ (ks << 5)) + REC_QG, aq[ks][0], aq[ks][1], aq[ks][2], aq[ks][3]);
        dk[ks][0] = *reinterpret_cast<const float*>(smem + REC_DEC + (ks * 16 + gq) * 4);
        dk[ks][1] = *reinterpret_cast<const float*>(smem + REC_DEC + (ks * 16 + gq + 8) * 4);
      }
#pragma unroll
      for (int nv = 0; nv < NVT; ++nv)
        u[nv] = (use_u && !(PAIR && nv == 0)) ? *reinterpret_cast<const float4*>(smem + u_off + (PAIR ? 0 : nv) * REC_U_TILE_BYTES)
                                              : make_float4(0, 0, 0, 0);
    }

    for (int n = 0; n < NT && !failed; ++n) {
      const int s = n % K2_STAGES;
      const uint32_t sp = sbase + s * SM::STAGE;
      const uint32_t t2 = sp + a2_lane;

      // the previous step's output tile (always a full chunk)
      if (!STATE_ONLY && n > 0) {
        __nv_bfloat16* op = ob + static_cast<int64_t>((n - 1) * BT + gq) * p.o_s[1];
#pragma unroll
        for (int nv = 0; nv < NVT; ++nv) {
          *reinterpret_cast<uint32_t*>(op + nv * 8) = pack_bf16(oa[nv][0], oa[nv][1]);
          *reinterpret_cast<uint32_t*>(op + 8 * p.o_s[1] + nv * 8) = pack_bf16(oa[nv][2], oa[nv][3]);
        }
      }

      // B fragments of bf16(hT) (pre-chunk state): accumulator fragment -> pack -> 8x8 transpose
      uint32_t bh[8][NVT][2];
#pragma unroll
      for (int m = 0; m < 8; ++m)
#pragma unroll
        for (int nv = 0; nv < NVT; ++nv) {
          bh[m][nv][0] = movmatrix_t(pack_bf16(hT[m][nv][0], hT[m][nv][1]));
          bh[m][nv][1] = movmatrix_t(pack_bf16(hT[m][nv][2], hT[m][nv][3]));
        }

      // P1 (two accumulator sets: even / odd k-steps), carrying the kg fragment loads of this
      // step and the decay of the fp32 state
      float pw[2][NVT][4], pq[2][NVT][4];
      uint32_t kgh[8][4], kgl[8][4];
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
#pragma unroll
        for (int nv = 0; nv < NVT; ++nv) {
          if (ks < 2) mma_bf16_z(pw[ks & 1][nv], aw[ks], bh[ks][nv][0], bh[ks][nv][1]);
          else mma_bf16_v(pw[ks & 1][nv], aw[ks], bh[ks][nv][0], bh[ks][nv][1]);
        }
        ldsm_x4_t((t2 ^ (ks << 5)) + REC_KGH, kgh[ks][0], kgh[ks][1], kgh[ks][2], kgh[ks][3]);
        if (!STATE_ONLY) {
#pragma unroll
          for (int nv = 0; nv < NVT; ++nv) {
            if (ks < 2) mma_bf16_z(pq[ks & 1][nv], aq[ks], bh[ks][nv][0], bh[ks][nv][1]);
            else mma_bf16_v(pq[ks & 1][nv], aq[ks], bh[ks][nv][0], bh[ks][nv][1]);
          }
        }
        ldsm_x4_t((t2 ^ (ks << 5)) + REC_KGL, kgl[ks][0], kgl[ks][1], kgl[ks][2], kgl[ks][3]);
#pragma unroll
        for (int nv = 0; nv < NVT; ++nv) {
          const float2 lo = __fmul2_rn(make_float2(hT[ks][nv][0], hT[ks][nv][1]), make_float2(dk[ks][0], dk[ks][0]));
          const float2 hi = __fmul2_rn(make_float2(hT[ks][nv][2], hT[ks][nv][3]), make_float2(dk[ks][1], dk[ks][1]));
          hT[ks][nv][0] = lo.x; hT[ks][nv][1] = lo.y; hT[ks][nv][2] = hi.x; hT[ks][nv][3] = hi.y;
        }
      }
      uint32_t ah3[4], al3[4];
      if (!STATE_ONLY) {
        ldsm_x4(sp + a3_off, ah3[0], ah3[1], ah3[2], ah3[3]);
        ldsm_x4(sp + a3_off + (REC_AQL - REC_AQK), al3[0], al3[1], al3[2], al3[3]);
      }

      // v_new (fp32, accumulator layout: rows tok, cols v) and its hi/lo B fragments
      uint32_t bvh[NVT][2], bvl[NVT][2];
#pragma unroll
      for (int nv = 0; nv < NVT; ++nv) {
        const float x0 = u[nv].x - (pw[0][nv][0] + pw[1][nv][0]), x1 = u[nv].y - (pw[0][nv][1] + pw[1][nv][1]);
        const float x2 = u[nv].z - (pw[0][nv][2] + pw[1][nv][2]), x3 = u[nv].w - (pw[0][nv][3] + pw[1][nv][3]);
        uint32_t h01, l01, h23, l23;
        split_pack(x0, x1, h01, l01);
        split_pack(x2, x3, h23, l23);
        bvh[nv][0] = movmatrix_t(h01); bvh[nv][1] = movmatrix_t(h23);
        bvl[nv][0] = movmatrix_t(l01); bvl[nv][1] = movmatrix_t(l23);
      }

      // release the stage only when its fragment loads have landed: shared-memory loads of a warp
      // return in issue order, so reading a register of the last-issued ones makes the warp wait
      // for all of them
      {
        uint32_t landed = kgh[7][0] ^ kgl[7][0];
        if (!STATE_ONLY) landed ^= ah3[0] ^ al3[0];
        asm volatile("" ::"r"(landed) : "memory");
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty0 + s * 8);
      const bool more = n + 1 < NT;
      const int s1 = (n + 1) % K2_STAGES;
      const uint32_t sp1 = sbase + s1 * SM::STAGE;
      const uint8_t* spg1 = smem + s1 * SM::STAGE;
      const uint32_t t1n = sp1 + a1_lane;
      if (more) {
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(full0 + s1 * 8, ((n + 1) / K2_STAGES) & 1, sAbort))) {
          if (*sAbort == 0) { *sAbort = 1; atomicExch(p.status, ST_K2_FULL_TIMEOUT); }
          failed = true;
          break;
        }
      }

      // P2: hT += kg^T v_new  (hi*hi, then hi*lo(v), then lo(kg)*hi: three passes over independent
      // tiles), carrying the next step's operand loads
#pragma unroll
      for (int m = 0; m < 8; ++m) {
#pragma unroll
        for (int nv = 0; nv < NVT; ++nv) mma_bf16_v(hT[m][nv], kgh[m], bvh[nv][0], bvh[nv][1]);
        if (more) ldsm_x4((t1n ^ (m << 5)) + REC_W, aw[m][0], aw[m][1], aw[m][2], aw[m][3]);
      }
#pragma unroll
      for (int m = 0; m < 8; ++m) {
#pragma unroll
        for (int nv = 0; nv < NVT; ++nv) mma_bf16_v(hT[m][nv], kgh[m], bvl[nv][0], bvl[nv][1]);
        if (more) {
          dk[m][0] = *reinterpret_cast<const float*>(spg1 + REC_DEC + (m * 16 + gq) * 4);
          dk[m][1] = *reinterpret_cast<const float*>(spg1 + REC_DEC + (m * 16 + gq + 8) * 4);
        }
      }
#pragma unroll
      for (int m = 0; m < 8; ++m) {
#pragma unroll
        for (int nv = 0; nv < NVT; ++nv) mma_bf16_v(hT[m][nv], kgl[m], bvh[nv][0], bvh[nv][1]);
        if (!STATE_ONLY && more)
          ldsm_x4((t1n ^ (m << 5)) + REC_QG, aq[m][0], aq[m][1], aq[m][2], aq[m][3]);
      }

      // P3: o = scale * (qg hT) + Aqk v_new
      if (!STATE_ONLY) {
#pragma unroll
        for (int nv = 0; nv < NVT; ++nv) {
#pragma unroll
          for (int e = 0; e < 4; ++e) oa[nv][e] = p.scale * (pq[0][nv][e] + pq[1][nv][e]);
          mma_bf16_v(oa[nv], ah3, bvh[nv][0], bvh[nv][1]);
          mma_bf16_v(oa[nv], ah3, bvl[nv][0], bvl[nv][1]);
          mma_bf16_v(oa[nv], al3, bvh[nv][0], bvh[nv][1]);
        }
      }
      if (more) {
#pragma unroll
        for (int nv = 0; nv < NVT; ++nv)
          u[nv] = (use_u && !(PAIR && nv == 0)) ? *reinterpret_cast<const float4*>(spg1 + u_off + (PAIR ? 0 : nv) * REC_U_TILE_BYTES)
                                                : make_float4(0, 0, 0, 0);
      }
    }

    // the last chunk's output tile (it may be a partial chunk)
    if (!STATE_ONLY && !failed) {
      const int tok = (NT - 1) * BT + gq;
      __nv_bfloat16* op = ob + static_cast<int64_t>(tok) * p.o_s[1];
#pragma unroll
      for (int nv = 0; nv < NVT; ++nv) {
        if (tok < Tlen) *reinterpret_cast<uint32_t*>(op + nv * 8) = pack_bf16(oa[nv][0], oa[nv][1]);
        if (tok + 8 < Tlen) *reinterpret_cast<uint32_t*>(op + 8 * p.o_s[1] + nv * 8) = pack_bf16(oa[nv][2], oa[nv][3]);
      }
    }

    if (!failed && (p.ht != nullptr || (PAIR && p.push_on))) {
      float* ht = (PAIR && p.push_on)
                      ? p.push_dst[bh / p.push_hp] + p.push_dst_offset + static_cast<size_t>(2 * (bh % p.push_hp)) * D * D
                      : p.ht + static_cast<size_t>(PAIR ? 2 * bh : chain) * D * D;
#pragma unroll
      for (int m = 0; m < 8; ++m)
#pragma unroll
        for (int nv = 0; nv < NVT; ++nv)
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (PAIR) ht[(static_cast<size_t>(nv) * D + v0 + tq * 2 + (e & 1)) * D + m * 16 + gq + (e >> 1) * 8] = hT[m][nv][e];
            else if (p.k_first) ht[(m * 16 + gq + (e >> 1) * 8) * D + v0 + nv * 8 + tq * 2 + (e & 1)] = hT[m][nv][e];
            else ht[(v0 + nv * 8 + tq * 2 + (e & 1)) * D + m * 16 + gq + (e >> 1) * 8] = hT[m][nv][e];
    }
  }

  __syncthreads();
  if (PAIR && p.push_on && tid == 0 && *sAbort == 0) {
    // the tiles went into another rank's receive buffer: the CTA barrier has put every warp's stores before
    // this count; the CTA that counts last for a destination raises its flag behind one system-scope fence
    const int owner = bh / p.push_hp;
    __threadfence();
    const int done = atomicAdd(p.push_counter + owner, 1);
    __threadfence();
    if (done == p.push_ctas_per_dst - 1) {
      p.push_counter[owner] = 0;
      __threadfence_system();
      st_release_sys(p.push_flag[owner], p.push_epoch);
    }
  }
  if (*sAbort != 0 && tid == 0) {
    // give copies that are still in flight a bounded chance to land before the CTA's
    // shared memory is released
    const int issued = *sIssued;
    for (int n = max(0, issued - K2_STAGES); n < issued; ++n)
      mbar_wait_bounded(full0 + (n % K2_STAGES) * 8, (n / K2_STAGES) & 1, nullptr);
  }
}

template <int CW, int NVT, bool STATE_ONLY, bool PAIR = false>
static cudaError_t launch_k2_t(const K2Params& p, cudaStream_t stream) {
  constexpr int RT = PAIR ? 1 : NVT;
  constexpr int smem_bytes = K2Smem<CW, RT>::TOTAL;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kda_k2_kernel<CW, NVT, STATE_ONLY, PAIR>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const int nblocks = (p.n_chains > 0 ? p.n_chains : (p.seq_table != nullptr ? p.n_seqs : p.B) * p.H) * (D / (CW * RT * 8));
  kda_k2_kernel<CW, NVT, STATE_ONLY, PAIR><<<nblocks, (CW + 1) * 32, smem_bytes, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_k2n(const K2Params& p, int vsplit, int ntile, bool state_only, cudaStream_t stream) {
  // vsplit CTAs per head, ntile 8-row tiles per warp  =>  16 / (vsplit * ntile) consumer warps per CTA
  // (at most 4: a fifth warp is the producer, and CTAs of more than 8 warps lose registers per thread)
#define KDA_K2_CASE(VS, NT_, CW_)                                                                  \
  if (vsplit == VS && ntile == NT_)                                                                \
    return state_only ? launch_k2_t<CW_, NT_, true>(p, stream) : launch_k2_t<CW_, NT_, false>(p, stream);
  KDA_K2_CASE(4, 1, 4)
  KDA_K2_CASE(8, 1, 2)
  KDA_K2_CASE(16, 1, 1)
#undef KDA_K2_CASE
  return cudaErrorInvalidValue;
}

cudaError_t launch_k2n_pair(const K2Params& p0, int vsplit, cudaStream_t stream) {
  // the transform-pair pass: two recurrences over the same eight rows per warp, 16 / vsplit consumer warps per CTA
  K2Params p = p0;
  p.push_ctas_per_dst = p.push_hp * vsplit;   // vsplit CTAs share a chain
  switch (vsplit) {
    case 4: return launch_k2_t<4, 2, true, true>(p, stream);
    case 8: return launch_k2_t<2, 2, true, true>(p, stream);
    case 16: return launch_k2_t<1, 2, true, true>(p, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace kda
