// K2 on the 5th-generation tensor cores (tcgen05 + TMEM): the throughput form of the state
// recurrence for problems with many (batch, head) chains.  sm_100a.
//
// Same arithmetic and record contract as kda_k2_sm100.cu (which replaces kda_bt16_kernel_k2 of the
// reference, src/kda_bt16/kernels.py:187-302):
//   v_new = u - w h^T ;  o = scale (qg h^T) + Aqk v_new ;  h = h diag(dec) + v_new^T kg
// One CTA owns ALL 128 state rows of one (batch, head): the fp32 state lives in tensor memory
// (128 lanes = rows v, 128 columns = k) for the whole sequence.  Per chunk:
//   P1  D1[v][32]  = bf16(h)[v][:] . [w ; qg]^T          8 x tcgen05.mma M128 N32 K16   (A from TMEM)
//   E1  v_new = u - D1[:, 0:16]  ->  hi/lo bf16 pair back into TMEM          (256 threads)
//   P2  h[v][:]   += v_new^T[v][:] . kg                   3 x M128 N128 K16 (hi.hi, lo.hi, hi.lo)
//   P3  D3[v][16]  = v_new^T[v][:] . Aqk^T                3 x M128 N16 K16
//   E2  read h, write bf16(h) (next P1's A operand) and h * dec(next chunk); o = scale D1[:, 16:32] + D3
// The record tiles become tensor-core operands without a second pass over them: a 5-D tiled TMA
// map over the record array lands every [16 tok][128 k] tile as two 64-column atoms in the
// canonical 128-byte-swizzled layout (the records are already XOR-swizzled per 128-byte half row).
//
// A commit -> mbarrier -> waiting-thread round trip costs ~430 cycles on this part and a step needs
// two of them, so ONE chain per SM is slower than the mma.sync kernels (~2,200 against ~1,100
// cycles per step); two CTAs are resident per SM (256 of the 512 TMEM columns, 81 KB of shared
// memory each) and the form pays once there are enough chains to fill both slots of every SM.
//
// Warp roles: 0-7 element-wise work (warp w: TMEM lanes 32 (w%4).., column / token half w/4),
// 8 = producer (TMA), 9 = MMA issuer and TMEM owner.  Every wait is bounded.
#include <cuda.h>

#include "kda_common.cuh"
#include "kda_kernels.h"

namespace kda {

namespace {

constexpr int KT_STAGES = 3;
constexpr int KT_EPI_WARPS = 8;
constexpr int KT_THREADS = (KT_EPI_WARPS + 2) * 32;
// stage layout (1024-byte aligned base: the swizzled atoms need it)
constexpr int T_WQ = 0;        // [2 atoms][32 rows: w 0..15, qg 16..31][128 B]
constexpr int T_KGH = 8192;    // [2 atoms][16 tok][128 B]
constexpr int T_KGL = 12288;
constexpr int T_U = 16384;     // fp32 u, fragment order (8192 B)
constexpr int T_AQ = 24576;    // Aqk hi, Aqk lo, dec as in the record (1536 B)
constexpr int T_AQF = 26112;   // Aqk hi / lo re-laid as 8x8 core matrices (2 x 512 B)
constexpr int T_STAGE = 27648;
constexpr int T_BARS = KT_STAGES * T_STAGE;
// The state snapshot reaches the MMA thread in KT_PG column groups, so that the first k-steps of the
// next P1 are issued while the element-wise warps still convert the rest of the state.
constexpr int KT_PG = 2;
static_assert(KT_PG == 1 || KT_PG == 2 || KT_PG == 4, "column groups of the snapshot");
// barriers: full[S], empty[S], p1, v, p2, o, p3, s[KT_PG]
constexpr int T_NBARS = 2 * KT_STAGES + 5 + KT_PG;
constexpr int T_SLOT = T_BARS + T_NBARS * 8;      // TMEM base address, abort flag, issued count
constexpr int T_OST = (T_SLOT + 32 + 15) / 16 * 16;                // two [16 tok][128 v] bf16 output staging tiles
constexpr int T_TOTAL = T_OST + 2 * TILE_BYTES;
static_assert(T_OST % 16 == 0, "staging tiles are read 16 bytes at a time");
// TMEM columns
constexpr uint32_t C_S = 0, C_D1 = 128, C_D3 = 160, C_AS = 176, C_VH = 240, C_VL = 248, C_TOTAL = 256;

constexpr int ST_K2T_TIMEOUT = 4;

// ---- tcgen05 wrappers ------------------------------------------------------------------------
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem descriptor]
__device__ __forceinline__ void umma_ts(uint32_t d, uint32_t a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}" ::"r"(d),
      "r"(a), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t a, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(a));
}
__device__ __forceinline__ void tmem_ld16(uint32_t a, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(a));
}
// The registers of a tcgen05.ld are valid only after tcgen05.wait::ld; the compiler sees the wait
// as an unrelated statement, so after it the registers are passed through an empty asm that pins
// every later use behind the wait.
__device__ __forceinline__ void pin8(uint32_t (&r)[8]) {
  asm volatile("" : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7])::"memory");
}
__device__ __forceinline__ void pin16(uint32_t (&r)[16]) {
  asm volatile(""
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]),
                 "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])::"memory");
}
__device__ __forceinline__ void tmem_st4(uint32_t a, const uint32_t (&r)[4]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(r[0]), "r"(r[1]), "r"(r[2]),
               "r"(r[3])
               : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t a, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(a), "r"(r[0]), "r"(r[1]),
               "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t a, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(a),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
// 16-lane shapes: thread (g = lane / 4, t = lane % 4) of the warp holds, per repeat n, the fp32 pairs
// (row g, columns 8n + 2t, 8n + 2t + 1) and (row g + 8, same columns) -- the mma.sync accumulator layout,
// whose rows are 32-byte pieces of memory rows: the state moves between global memory and TMEM with
// fully used sectors.  The 128-bit shape is the same with one 32-bit column per thread and repeat.
__device__ __forceinline__ void tmem_st_16x256b_x8(uint32_t a, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.16x256b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(a),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_ld_16x256b_x8(uint32_t a, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(a));
}
__device__ __forceinline__ void tmem_st_16x128b_x8(uint32_t a, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.16x128b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(a),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst_smem, const void* tmap, int c0, int c1, int c2, int c3, int c4,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];" ::
          "r"(dst_smem), "l"(tmap), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(bar)
      : "memory");
}

// shared-memory matrix descriptor (sm_100 format): start address, leading / stride byte offsets in
// 16-byte units, descriptor version 1, layout type (0 = no swizzle, 2 = 128-byte swizzle)
__host__ __device__ constexpr uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
  return static_cast<uint64_t>((saddr >> 4) & 0x3FFF) | (static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16) |
         (static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32) | (static_cast<uint64_t>(1) << 46) |
         (static_cast<uint64_t>(layout) << 61);
}
// instruction descriptor: fp32 accumulate, bf16 x bf16, A K-major, B K-major (0) or MN-major (1)
__host__ __device__ constexpr uint32_t instr_desc(int M, int N, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(b_mn_major) << 16) |
         (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}

struct K2tParams {
  K2Params k;
  CUtensorMap tm_rec;   // 5-D view of the record array: (64 bf16, 2 halves, 16 rows, 4 tiles, records)
};

__global__ void __launch_bounds__(KT_THREADS, 2) kda_k2t_kernel(const __grid_constant__ K2tParams pp) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const K2Params& p = pp.k;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int bh = blockIdx.x + p.chain0;
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
  const uint32_t bar0 = sbase + T_BARS;
  auto full = [&](int s) { return bar0 + s * 8; };
  auto empty = [&](int s) { return bar0 + (KT_STAGES + s) * 8; };
  const uint32_t bar_p1 = bar0 + (2 * KT_STAGES + 0) * 8, bar_v = bar0 + (2 * KT_STAGES + 1) * 8;
  const uint32_t bar_p2 = bar0 + (2 * KT_STAGES + 2) * 8, bar_o = bar0 + (2 * KT_STAGES + 3) * 8;
  const uint32_t bar_p3 = bar0 + (2 * KT_STAGES + 4) * 8;
  auto bar_s = [&](int q) { return bar0 + (2 * KT_STAGES + 5 + q) * 8; };
  uint32_t* slot = reinterpret_cast<uint32_t*>(smem + T_SLOT);
  volatile int* sAbort = reinterpret_cast<volatile int*>(smem + T_SLOT + 4);
  volatile int* sIssued = sAbort + 1;

  if (tid == 0) {
    for (int s = 0; s < KT_STAGES; ++s) { mbar_init(full(s), 1); mbar_init(empty(s), 1); }
    mbar_init(bar_p1, 1);
    mbar_init(bar_v, KT_EPI_WARPS);    // one arrival per element-wise warp (lane 0, after __syncwarp)
    mbar_init(bar_p2, 1);
    mbar_init(bar_p3, 1);
    for (int q = 0; q < KT_PG; ++q) mbar_init(bar_s(q), KT_EPI_WARPS);
    mbar_init(bar_o, KT_EPI_WARPS);
    *sAbort = 0;
    *sIssued = 0;
    fence_mbar_init();
  }
  if (warp == KT_EPI_WARPS + 1) {   // the MMA warp owns the tensor memory of the CTA
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(C_TOTAL)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = *slot;

  auto give_up = [&]() {
    if (*sAbort == 0) { *sAbort = 1; atomicExch(p.status, ST_K2T_TIMEOUT); }
  };

  if (warp == KT_EPI_WARPS) {
    // ------------------------------ producer -------------------------------
    if (lane == 0) {
      for (int n = 0; n < NT; ++n) {
        const int s = n % KT_STAGES;
        if (n >= KT_STAGES && !mbar_wait_bounded(empty(s), ((n / KT_STAGES) - 1) & 1, sAbort)) { give_up(); break; }
        const int rec_i = static_cast<int>(rec_first) + n;
        const uint8_t* rec = p.rec + (rec_first + n) * REC_BYTES;
        const uint32_t dst = sbase + s * T_STAGE;
        mbar_arrive_expect_tx(full(s), 4 * TILE_BYTES + (REC_U - REC_AQK) + (REC_BYTES - REC_U));
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          tma_load_5d(dst + T_WQ + half * 4096, &pp.tm_rec, 0, half, 0, 0, rec_i, full(s));          // w
          tma_load_5d(dst + T_WQ + half * 4096 + 2048, &pp.tm_rec, 0, half, 0, 1, rec_i, full(s));   // qg
          tma_load_5d(dst + T_KGH + half * 2048, &pp.tm_rec, 0, half, 0, 2, rec_i, full(s));         // kg hi
          tma_load_5d(dst + T_KGL + half * 2048, &pp.tm_rec, 0, half, 0, 3, rec_i, full(s));         // kg lo
        }
        bulk_g2s(dst + T_AQ, rec + REC_AQK, REC_U - REC_AQK, full(s));
        bulk_g2s(dst + T_U, rec + REC_U, REC_BYTES - REC_U, full(s));
        *sIssued = n + 1;
      }
    }
    __syncwarp();
  } else if (warp == KT_EPI_WARPS + 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      constexpr uint32_t ID_P1 = instr_desc(128, 32, 0), ID_P2 = instr_desc(128, 128, 1), ID_P3 = instr_desc(128, 16, 0);
      int s = 0;
      for (int n = 0; n < NT; ++n, s = (s + 1 == KT_STAGES) ? 0 : s + 1) {
        const uint32_t st = sbase + s * T_STAGE;
        if (!mbar_wait_bounded(full(s), (n / KT_STAGES) & 1, sAbort)) { give_up(); break; }
        const uint64_t dwq = smem_desc(st + T_WQ, 16, 1024, 2);   // k-step ks: start address + atom * 4096 + (ks % 4) * 32 bytes
        bool ready = true;
#pragma unroll
        for (int q = 0; q < KT_PG; ++q) {
          // column group q of both halves of bf16(h) is in TMEM (with the last group: the decayed h too)
          if (!mbar_wait_bounded(bar_s(q), n & 1, sAbort)) { ready = false; break; }
          tc_fence_after();
#pragma unroll
          for (int cc = q * (4 / KT_PG); cc < (q + 1) * (4 / KT_PG); ++cc)
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
              const int ks = hf * 4 + cc;
              umma_ts(tbase + C_D1, tbase + C_AS + ks * 8, dwq + static_cast<uint64_t>((hf * 4096 + cc * 32) >> 4), ID_P1,
                      !(cc == 0 && hf == 0));
            }
        }
        if (!ready) { give_up(); break; }
        umma_commit(bar_p1);
        if (!mbar_wait_bounded(bar_v, n & 1, sAbort)) { give_up(); break; }     // v_new hi/lo are in TMEM
        tc_fence_after();
        const uint64_t dkh = smem_desc(st + T_KGH, 2048, 1024, 2), dkl = smem_desc(st + T_KGL, 2048, 1024, 2);
        umma_ts(tbase + C_S, tbase + C_VH, dkh, ID_P2, 1);
        umma_ts(tbase + C_S, tbase + C_VL, dkh, ID_P2, 1);
        umma_ts(tbase + C_S, tbase + C_VH, dkl, ID_P2, 1);
        umma_commit(bar_p2);   // the state pass of the element-wise warps starts while P3 runs
        const uint64_t dah = smem_desc(st + T_AQF, 128, 256, 0), dal = smem_desc(st + T_AQF + 512, 128, 256, 0);
        umma_ts(tbase + C_D3, tbase + C_VH, dah, ID_P3, 0);
        umma_ts(tbase + C_D3, tbase + C_VL, dah, ID_P3, 1);
        umma_ts(tbase + C_D3, tbase + C_VH, dal, ID_P3, 1);
        umma_commit(bar_p3);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ element-wise warps ----------------------
    const int quad = warp & 3, half = warp >> 2;
    const int v = quad * 32 + lane;                       // state row = TMEM lane
    const uint32_t tl = tbase + (static_cast<uint32_t>(quad * 32) << 16);
    // u[tok = 8 half + j][v] in the record's fragment order
    const uint32_t u_off = T_U + (v >> 3) * 512 + ((v & 7) >> 1) * 16 + (half * 2 + (v & 1)) * 4;
    bool ok = true;

    // initial state: TMEM <- h0 * dec(chunk 0); bf16(h0) as the first A operand
    ok = mbar_wait_bounded(full(0), 0, sAbort);
    if (ok) {
      // this warp's 32 rows x 64 columns in two 16-row halves, through the 16-lane access shapes
      const float* dec0 = reinterpret_cast<const float*>(smem + T_AQ + (REC_DEC - REC_AQK)) + half * 64;
      const int g4 = lane >> 2, t4 = lane & 3;
#pragma unroll 1
      for (int hh = 0; hh < 2; ++hh) {
        const int r0 = quad * 32 + hh * 16 + g4;
        // element (v, k) sits at v*128 + k (V-first) or k*128 + v (K-first); this thread holds rows
        // v = r0, r0 + 8 and columns k = 64 half + 8 n8 + 2 t4, +1
        const float* src = p.h0 == nullptr ? nullptr
                           : p.k_first ? p.h0 + (static_cast<size_t>(bh) * D + half * 64 + t4 * 2) * D + r0
                                       : p.h0 + (static_cast<size_t>(bh) * D + r0) * D + half * 64 + t4 * 2;
        uint32_t sr[32], ar[16];
#pragma unroll
        for (int n8 = 0; n8 < 8; ++n8) {
          float2 x = make_float2(0.f, 0.f), y = x;
          if (src != nullptr) {
            if (p.k_first) {
              const float* c0 = src + n8 * 8 * D;
              x = make_float2(c0[0], c0[D]);
              y = make_float2(c0[8], c0[D + 8]);
            } else {
              x = *reinterpret_cast<const float2*>(src + n8 * 8);
              y = *reinterpret_cast<const float2*>(src + 8 * D + n8 * 8);
            }
          }
          const float2 dd = *reinterpret_cast<const float2*>(dec0 + n8 * 8 + t4 * 2);
          ar[n8 * 2] = pack_bf16(x.x, x.y);
          ar[n8 * 2 + 1] = pack_bf16(y.x, y.y);
          sr[n8 * 4 + 0] = __float_as_uint(x.x * dd.x); sr[n8 * 4 + 1] = __float_as_uint(x.y * dd.y);
          sr[n8 * 4 + 2] = __float_as_uint(y.x * dd.x); sr[n8 * 4 + 3] = __float_as_uint(y.y * dd.y);
        }
        const uint32_t th = tbase + (static_cast<uint32_t>(quad * 32 + hh * 16) << 16);
        tmem_st_16x256b_x8(th + C_S + half * 64, sr);
        tmem_st_16x128b_x8(th + C_AS + half * 32, ar);
      }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0)
        for (int q = 0; q < KT_PG; ++q) mbar_arrive(bar_s(q));
    } else {
      give_up();
    }

    float oq[8], o3[8], uv[8];
    uint32_t aq[8];
    __nv_bfloat16* const orow = p.o + b * p.o_s[0] + tok0 * p.o_s[1] + h * p.o_s[2];

    // State-independent operands of chunk n1: this thread's eight u values and, by warp 0, Aqk hi / lo
    // re-laid as 8x8 core matrices (the B operand of P3).  Runs while the tensor core works.
    auto prepare = [&](int n1) -> bool {
      const int s1 = n1 % KT_STAGES;
      if (!mbar_wait_bounded(full(s1), (n1 / KT_STAGES) & 1, sAbort)) return false;
      const uint8_t* stg = smem + s1 * T_STAGE;
      if (warp == 0) {
        const int mat = lane >> 4, i = lane & 15;
#pragma unroll
        for (int c = 0; c < 2; ++c)
          *reinterpret_cast<uint4*>(smem + s1 * T_STAGE + T_AQF + mat * 512 + (i >> 3) * 256 + c * 128 + (i & 7) * 16) =
              *reinterpret_cast<const uint4*>(stg + T_AQ + mat * 512 + i * 32 + c * 16);
        fence_proxy_async();
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) uv[j] = *reinterpret_cast<const float*>(stg + u_off + j * 64);
      return true;
    };
    // o[tok][v] = scale * (qg h^T) + Aqk v_new of chunk nd, from the registers filled by its E2:
    // transposed through a staging tile so that every thread stores 16 contiguous bytes of a token row
    auto store_o = [&](int nd) -> bool {
      uint8_t* buf = smem + T_OST + (nd & 1) * TILE_BYTES;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        *reinterpret_cast<__nv_bfloat16*>(buf + (half * 8 + j) * 256 + v * 2) = __float2bfloat16(fmaf(p.scale, oq[j], o3[j]));
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_o);
      if (!mbar_wait_bounded(bar_o, nd & 1, sAbort)) return false;
      const int row = tid >> 4, seg = tid & 15;
      const int tok = nd * BT + row;
      if (tok < Tlen)
        *reinterpret_cast<uint4*>(orow + static_cast<int64_t>(tok) * p.o_s[1] + seg * 8) =
            *reinterpret_cast<const uint4*>(buf + row * 256 + seg * 16);
      return true;
    };

    if (ok) ok = prepare(0);
    for (int n = 0; n < NT && ok; ++n) {
      const int s = n % KT_STAGES;
      const bool more = n + 1 < NT;

      // ---- E1: v_new = u - w h^T for this thread's row and eight tokens ----
      if (!mbar_wait_bounded(bar_p1, n & 1, sAbort)) { ok = false; break; }
      tc_fence_after();
      {
        uint32_t d1[8];
        tmem_ld8(tl + C_D1 + half * 8, d1);
        tmem_ld8(tl + C_D1 + 16 + half * 8, aq);   // qg h^T of this chunk: it must leave TMEM before the next P1
        tc_wait_ld();
        pin8(d1);
        pin8(aq);
        uint32_t vh[4], vl[4];
#pragma unroll
        for (int c = 0; c < 4; ++c)
          split_pack(uv[2 * c] - __uint_as_float(d1[2 * c]), uv[2 * c + 1] - __uint_as_float(d1[2 * c + 1]), vh[c], vl[c]);
        tmem_st4(tl + C_VH + half * 4, vh);
        tmem_st4(tl + C_VL + half * 4, vl);
        tc_wait_st();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_v);

      // while P2 runs: the next chunk's operands
#pragma unroll
      for (int j = 0; j < 8; ++j) oq[j] = __uint_as_float(aq[j]);
      if (more && !prepare(n + 1)) { ok = false; break; }

      // ---- E2: after P2 / P3 ----
      if (!mbar_wait_bounded(bar_p2, n & 1, sAbort)) { ok = false; break; }
      tc_fence_after();
      // dec of the next chunk (its stage was waited for in prepare)
      const float* decn = reinterpret_cast<const float*>(smem + ((n + 1) % KT_STAGES) * T_STAGE + T_AQ + (REC_DEC - REC_AQK)) + half * 64;
      // the TMEM loads of the state are issued one 16-column step ahead of their use
      uint32_t sr[2][16];
      tmem_ld16(tl + C_S + half * 64, sr[0]);
      tc_wait_ld();
      pin16(sr[0]);
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        uint32_t (&cur)[16] = sr[cc & 1];
        if (cc < 3) tmem_ld16(tl + C_S + half * 64 + (cc + 1) * 16, sr[(cc + 1) & 1]);
        if (more) {
          uint32_t ar[8];
#pragma unroll
          for (int j4 = 0; j4 < 4; ++j4) {
            const float4 dd = *reinterpret_cast<const float4*>(decn + cc * 16 + j4 * 4);
            const float x0 = __uint_as_float(cur[j4 * 4]), x1 = __uint_as_float(cur[j4 * 4 + 1]);
            const float x2 = __uint_as_float(cur[j4 * 4 + 2]), x3 = __uint_as_float(cur[j4 * 4 + 3]);
            ar[j4 * 2] = pack_bf16(x0, x1);
            ar[j4 * 2 + 1] = pack_bf16(x2, x3);
            const float2 lo = __fmul2_rn(make_float2(x0, x1), make_float2(dd.x, dd.y));
            const float2 hi = __fmul2_rn(make_float2(x2, x3), make_float2(dd.z, dd.w));
            cur[j4 * 4 + 0] = __float_as_uint(lo.x); cur[j4 * 4 + 1] = __float_as_uint(lo.y);
            cur[j4 * 4 + 2] = __float_as_uint(hi.x); cur[j4 * 4 + 3] = __float_as_uint(hi.y);
          }
          tmem_st16(tl + C_S + half * 64 + cc * 16, cur);
          tmem_st8(tl + C_AS + half * 32 + cc * 8, ar);
        }
        if (more && (cc + 1) % (4 / KT_PG) == 0) {   // a column group of the snapshot is complete
          tc_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_s((cc + 1) / (4 / KT_PG) - 1));
        }
        if (cc < 3) {
          tc_wait_ld();
          pin16(sr[(cc + 1) & 1]);
        }
      }
      // Aqk v_new of this chunk (P3 was committed after P2; it must leave TMEM before the next P3)
      if (!mbar_wait_bounded(bar_p3, n & 1, sAbort)) { ok = false; break; }
      tc_fence_after();
      if (tid == 0) mbar_arrive(empty(s));   // every operand of this stage has been consumed
      {
        uint32_t c3[8];
        tmem_ld8(tl + C_D3 + half * 8, c3);
        tc_wait_ld();
        pin8(c3);
#pragma unroll
        for (int j = 0; j < 8; ++j) o3[j] = __uint_as_float(c3[j]);
      }
      if (!store_o(n)) { ok = false; break; }   // while the next P1 runs
    }
    if (ok && p.ht != nullptr) {
      // final state: TMEM -> global through the 16-lane shape (32-byte pieces of the state's rows);
      // every element-wise thread has seen the last P2 complete
      const int g4 = lane >> 2, t4 = lane & 3;
#pragma unroll 1
      for (int hh = 0; hh < 2; ++hh) {
        uint32_t fr[32];
        tmem_ld_16x256b_x8(tbase + (static_cast<uint32_t>(quad * 32 + hh * 16) << 16) + C_S + half * 64, fr);
        tc_wait_ld();
        pin16(reinterpret_cast<uint32_t (&)[16]>(fr[0]));
        pin16(reinterpret_cast<uint32_t (&)[16]>(fr[16]));
        const int vr = quad * 32 + hh * 16 + g4;
        float* dst = p.k_first ? p.ht + (static_cast<size_t>(bh) * D + half * 64 + t4 * 2) * D + vr
                               : p.ht + (static_cast<size_t>(bh) * D + vr) * D + half * 64 + t4 * 2;
#pragma unroll
        for (int n8 = 0; n8 < 8; ++n8) {
          if (p.k_first) {
            float* c0 = dst + n8 * 8 * D;
            c0[0] = __uint_as_float(fr[n8 * 4]); c0[D] = __uint_as_float(fr[n8 * 4 + 1]);
            c0[8] = __uint_as_float(fr[n8 * 4 + 2]); c0[D + 8] = __uint_as_float(fr[n8 * 4 + 3]);
          } else {
            *reinterpret_cast<float2*>(dst + n8 * 8) = make_float2(__uint_as_float(fr[n8 * 4]), __uint_as_float(fr[n8 * 4 + 1]));
            *reinterpret_cast<float2*>(dst + 8 * D + n8 * 8) =
                make_float2(__uint_as_float(fr[n8 * 4 + 2]), __uint_as_float(fr[n8 * 4 + 3]));
          }
        }
      }
    }
    if (!ok) give_up();
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (*sAbort != 0 && tid == 0) {
    // give copies that are still in flight a bounded chance to land before the shared memory goes
    const int issued = *sIssued;
    for (int n = max(0, issued - KT_STAGES); n < issued; ++n)
      mbar_wait_bounded(full(n % KT_STAGES), (n / KT_STAGES) & 1, nullptr);
  }
  __syncthreads();
  if (warp == KT_EPI_WARPS + 1)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tbase), "r"(C_TOTAL) : "memory");
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

}  // namespace

// n_records: chunk records in the workspace (the tensor map must cover every record the grid reads)
cudaError_t launch_k2t(const K2Params& p, long long n_records, cudaStream_t stream) {
  EncodeTiledFn enc = encode_fn();
  if (enc == nullptr) return cudaErrorNotSupported;
  K2tParams pp;
  pp.k = p;
  // (64 bf16 = one 128-byte half row, 2 halves, 16 rows, 4 tiles, records); strides in bytes for dims 1..4
  const cuuint64_t dims[5] = {64, 2, 16, 4, static_cast<cuuint64_t>(n_records)};
  const cuuint64_t strides[4] = {128, 256, 4096, static_cast<cuuint64_t>(REC_BYTES)};
  const cuuint32_t box[5] = {64, 1, 16, 1, 1};
  const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = enc(&pp.tm_rec, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<uint8_t*>(p.rec), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kda_k2t_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T_TOTAL);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(kda_k2t_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const int nblocks = p.n_chains > 0 ? p.n_chains : (p.seq_table != nullptr ? p.n_seqs : p.B) * p.H;
  kda_k2t_kernel<<<nblocks, KT_THREADS, T_TOTAL, stream>>>(pp);
  return cudaGetLastError();
}

}  // namespace kda
