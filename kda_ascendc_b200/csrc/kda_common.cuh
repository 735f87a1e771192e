// Shared device helpers and the K1 -> K2 chunk-record contract (sm_100a only).
//
// A "chunk record" is the 26,112-byte block K1 writes and K2 reads for one
// (batch, head, chunk-of-16-tokens).  Records are chunk-major:
//   record index c = (b * H + h) * NT + n        (same order as the reference's
//   chunk-major packing, python/kda_ascendc_v1/layout.py:17-25)
// so the stream one (b, h) recurrence walks is contiguous in HBM and every
// stage is one bulk (TMA) copy.
//
//   offset  bytes  contents
//   0       4096   w    bf16 [16 tok][128 k]   swizzled tile (see swz_off)
//   4096    4096   qg   bf16 [16][128]  = bf16(qhat * 2^g)
//   8192    4096   kg_h bf16 [16][128]  \ hi/lo split of khat * 2^(g_last - g)
//   12288   4096   kg_l bf16 [16][128]  /
//   16384   512    Aqk_h bf16 [16 i][16 j] row-major \ hi/lo split of the scaled lower
//   16896   512    Aqk_l bf16 [16][16]               / triangle (incl. diagonal)
//   17408   512    dec  fp32 [128]      = 2^(g_last)
//   17920   8192   u    fp32, accumulator-fragment order [16 column tile][32 lane][4]:
//                       lane (g = lane/4, t = lane%4) holds u[tok g][v], u[tok g][v+1],
//                       u[tok g+8][v], u[tok g+8][v+1] with v = 8*tile + 2t
//
// Swizzled bf16 tile: element (r, c) of a [16][128] tile lives at byte
//   r*256 + ((((c>>3) ^ (r&7)) << 4) | ((c&7) << 1))
// i.e. the eight 16-byte units of each 128-byte half-row are XOR-permuted by the
// row index, which makes every ldmatrix (8 rows, same column unit) bank-conflict
// free after a straight, unpadded bulk copy.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace kda {

constexpr int BT = 16;
constexpr int D = 128;
constexpr int TILE_BYTES = BT * D * 2;  // 4096
constexpr int REC_W = 0;
constexpr int REC_QG = 4096;
constexpr int REC_KGH = 8192;
constexpr int REC_KGL = 12288;
constexpr int REC_AQK = 16384;
constexpr int REC_AQL = 16896;
constexpr int REC_DEC = 17408;
constexpr int REC_U = 17920;
constexpr int REC_SHARED_BYTES = 17920;  // everything every V-slice needs
constexpr int REC_U_TILE_BYTES = 512;    // one 8-column tile of u
constexpr int REC_BYTES = 26112;
constexpr int WS_HEADER_BYTES = 256;     // status block at the start of the workspace

// status codes written to workspace[0] by a kernel that gave up on a wait
constexpr int ST_OK = 0;
constexpr int ST_K1_LOAD_TIMEOUT = 1;
constexpr int ST_K2_FULL_TIMEOUT = 2;
constexpr int ST_K2_EMPTY_TIMEOUT = 3;
constexpr int ST_PEER_TIMEOUT = 7;   // a flag from another GPU did not arrive in time (sequence-split exchange)

constexpr float RCP_LN2 = 1.44269504089f;  // literal of tests/test_torch_reference.py:87
constexpr float L2NORM_EPS = 1e-6f;

// one second is plenty for a copy that normally takes a microsecond
constexpr unsigned long long WAIT_LIMIT_NS = 1000000000ull;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t swz_off(int r, int c) {
  return static_cast<uint32_t>(r * 256 + ((((c >> 3) ^ (r & 7)) << 4) | ((c & 7) << 1)));
}

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ---- mbarrier ---------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after WAIT_LIMIT_NS (or as soon as *abort_flag is set by
// another warp of the CTA) and returns false; the caller records a status code and
// unwinds.  Never spins forever.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity,
                                                  volatile int* abort_flag) {
  if (mbar_test_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (abort_flag != nullptr && *abort_flag != 0) return false;
    if (globaltimer_ns() - t0 > WAIT_LIMIT_NS) return false;
  }
}

// Bounded busy-poll for waits that are expected to last a few dozen cycles (a partner warp
// on another SM sub-partition): polls with the non-blocking test_wait, same limits.
__device__ __forceinline__ bool mbar_spin_bounded(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
#pragma unroll 1
  for (int i = 0; i < 4096; ++i)
    if (mbar_test_wait(bar, parity)) return true;
  return mbar_wait_bounded(bar, parity, abort_flag);
}

// ---- flags between GPUs (peer memory) ------------------------------------------
// A flag is an int32 epoch counter in the waiting GPU's own memory; a peer raises it with a
// system-scope release store after its data stores, the owner polls it with system-scope acquire
// loads.  Bounded like every other wait: false after WAIT_LIMIT_NS.
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ bool flag_wait_bounded(const int* flag, int epoch) {
  if (ld_acquire_sys(flag) - epoch >= 0) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (ld_acquire_sys(flag) - epoch >= 0) return true;
    if (globaltimer_ns() - t0 > WAIT_LIMIT_NS) return false;
  }
}

// ---- bulk (TMA, untiled) copies ---------------------------------------------
// global -> shared, completion counted in bytes on an mbarrier.  Both addresses
// 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
// tiled TMA load of one box of a 4-D tensor map (coordinates innermost first)
__device__ __forceinline__ void tma_load_4d(uint32_t dst_smem, const void* tmap, int c0, int c1, int c2, int c3,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::
          "r"(dst_smem), "l"(tmap), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}
// the same box, only pulled into L2 (no shared-memory destination, nothing to wait for)
__device__ __forceinline__ void tma_prefetch_l2_4d(const void* tmap, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];" ::"l"(tmap), "r"(c0), "r"(c1),
               "r"(c2), "r"(c3)
               : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

// ---- ldmatrix / mma ---------------------------------------------------------
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
// transpose an 8x8 b16 matrix held as one register per lane (fragment layout) inside the warp
__device__ __forceinline__ uint32_t movmatrix_t(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}
__device__ __forceinline__ void ldsm_x2(uint32_t addr, uint32_t& r0, uint32_t& r1) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
// D(16x8,f32) += A(16x16,bf16,row) * B(16x8,bf16,col)
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// same instruction, but pinned in program order (used where independent loads and stores are
// deliberately interleaved with a long MMA sequence so that their latency is covered)
__device__ __forceinline__ void mma_bf16_v(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// D = A * B with a zero accumulator: the first MMA of a chain needs no register initialisation
__device__ __forceinline__ void mma_bf16_z(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
}

// Read-only global loads pinned where they are written: used to fetch per-item parameters a whole
// iteration before their use, which the compiler would otherwise sink next to the use.
__device__ __forceinline__ float ldg_pinned(const float* p) {
  float v;
  asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ float2 ldg_pinned2(const float* p) {
  float2 v;
  asm volatile("ld.global.nc.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "l"(p));
  return v;
}

// ---- bf16 helpers -----------------------------------------------------------
// pack two floats (round to nearest even) into one register: lo -> bits 0..15
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float bf16_lo_to_f32(uint32_t p) { return __uint_as_float(p << 16); }
__device__ __forceinline__ float bf16_hi_to_f32(uint32_t p) { return __uint_as_float(p & 0xffff0000u); }
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ unsigned short bf16_bits(float x) { return __bfloat16_as_ushort(__float2bfloat16_rn(x)); }
// hi/lo split of two floats: hi = bf16(x), lo = bf16(x - hi)
__device__ __forceinline__ void split_pack(float x0, float x1, uint32_t& hi, uint32_t& lo) {
  hi = pack_bf16(x0, x1);
  lo = pack_bf16(x0 - bf16_lo_to_f32(hi), x1 - bf16_hi_to_f32(hi));
}
// packed variant on a float2 (one f32x2 FMA for the residual)
__device__ __forceinline__ void split_pack2(float2 x, uint32_t& hi, uint32_t& lo) {
  hi = pack_bf16(x.x, x.y);
  const float2 r = __ffma2_rn(make_float2(bf16_lo_to_f32(hi), bf16_hi_to_f32(hi)), make_float2(-1.f, -1.f), x);
  lo = pack_bf16(r.x, r.y);
}
__device__ __forceinline__ float rcpf(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

}  // namespace kda
