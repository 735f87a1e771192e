// K1: intra-chunk stage of the KDA forward.  Persistent CTAs of 128 threads, each walking
// (batch, head, chunk-of-16-tokens) work items with the next chunk's inputs in flight while
// the current one computes.  sm_100a.
//
// Replaces kda_bt16_kernel_k1 of the reference (src/kda_bt16/kernels.py:53-184) and
// follows the arithmetic and rounding points of the reference's torch chunk
// implementation (tests/test_torch_reference.py:77-173):
//   1. gate pre-pass: beta sigmoid, q/k l2-norm (eps 1e-6, result rounded to bf16),
//      gate = lower_bound*sigmoid(exp(A_log)*(g+dt_bias))*RCP_LN2, chunk-local cumsum
//   2. Aqk = scale*tril((qhat 2^gm)(khat 2^-gm)^T), Akk = tril_-1((khat 2^gm)(khat 2^-gm)^T)*beta_i
//      with gm = g - g[centre]; tensor-core MMAs on hi/lo bf16 splits of the fp32 operands
//      (three partial products, fp32 accumulate => ~2^-16 relative, "fp32-like")
//   3. X = (I + Akk)^-1 by forward substitution, fp32, one lane per column of X
//   4. w = X (khat beta 2^g)   (bf16 out),   u = X (v beta)   (fp32 out, split-bf16 MMAs)
// and additionally pre-computes what the reference's Triton K2 re-derives every step
// (src/kda_bt16/kernels.py:255-259,271,286-287): qg = bf16(qhat 2^g),
// kg = khat 2^(g_last-g) as a hi/lo bf16 pair, dec = 2^g_last -- the arrangement of
// the reference's Ascend pipeline (python/kda_ascendc_v1/api.py:890-897).
//
// Data movement: the four 16x128 input tiles arrive by tiled TMA copies (4-D tensor maps over
// (d, head, token, batch) built from the caller's strides, so head-shard and segment views
// need no copy; rows past T are zero-filled by the copy) that complete on one mbarrier; as soon as
// a chunk's inputs have been consumed the copies of the CTA's next chunk are issued into the
// same tiles, so the ~2.5 us load latency hides behind the rest of the chunk.  Of the
// 26,112-byte chunk record (kda_common.cuh) the qg / kg / Aqk / dec part and w leave by three
// bulk stores; u is stored straight from the accumulator fragments (512 contiguous bytes per warp).
#include "kda_common.cuh"
#include "kda_kernels.h"

namespace kda {

// shared-memory map (bytes): four CTAs of the production variant (bf16 gate, FAST_EXP) per SM
constexpr int S_QG = 0, S_KGH = 4096, S_KGL = 8192;   // -> record[4096, 16384)
constexpr int S_AQK = 12288, S_AQL = 12800, S_DEC = 13312;   // -> record[16384, 17920)
constexpr int S_L = 13824;                            // fp32 [16][16], -Akk
constexpr int S_XH = 14848, S_XL = 15360;             // bf16 [16][16] hi / lo of (I+Akk)^-1
constexpr int S_GRAM = 15872;
constexpr int S_QGH = S_GRAM, S_QGL = S_GRAM + 4096, S_KQH = S_GRAM + 8192, S_KQL = S_GRAM + 12288,
              S_KNH = S_GRAM + 16384, S_KNL = S_GRAM + 20480;   // KN tiles only without FAST_EXP
// once the Grams are done their A tiles hold the B operands of w and u
constexpr int S_KBH = S_GRAM, S_VBH = S_GRAM + 4096, S_VBL = S_GRAM + 8192;
constexpr int S_WST = S_GRAM + 12288;   // staging tile of w (the fourth Gram tile slot), -> record[0, 4096)

template <bool G_BF16, bool FAST_EXP>
struct K1Smem {
  static constexpr int IN = S_GRAM + (FAST_EXP ? 16384 : 24576);
  static constexpr int Q = IN, K = IN + 4096, V = IN + 8192, G = IN + 12288;
  static constexpr int G_BYTES = G_BF16 ? 4096 : 8192;
  static constexpr int SMALL = G + G_BYTES;
  static constexpr int BETA = SMALL;          // fp32 [2][16] activated beta + [2] exp(A_log): this item / next item
  static constexpr int TOT = BETA + 144;      // fp32 [2][128]: column sums of the gate over rows 0..7 and rows 8..15
  static constexpr int GMID = TOT + 1024;     // fp32 [128] g[mid] (not needed with FAST_EXP)
  static constexpr int MBAR = GMID + (FAST_EXP ? 0 : 512);
  static constexpr int FLAG = MBAR + 8;
  static constexpr int TOTAL = FLAG + 8;
};

struct K1Item {   // one (batch, head, chunk) work item
  int b, h, hq, t0, nvalid;   // hq: the q/k head this (value) head reads
  size_t rec_idx;
};

__device__ __forceinline__ K1Item k1_item(const K1Params& p, int id) {
  // id -> (b, n, h) with h fastest: CTAs that run together read one contiguous span of tokens
  K1Item w;
  const int bn = static_cast<int>(p.div_h.div(id));
  w.h = id - bn * p.H;
  w.hq = static_cast<int>(p.div_g.div(w.h));
  if (p.chunk_table != nullptr) {   // packed sequences: the chunk's place comes from the table
    const int4 e = __ldg(p.chunk_table + bn);
    w.b = 0;
    w.t0 = e.x;
    w.nvalid = e.y;
    w.rec_idx = static_cast<size_t>(e.z) + static_cast<size_t>(w.h) * e.w;
    return w;
  }
  w.b = static_cast<int>(p.div_nt.div(bn));
  const int n = bn - w.b * p.NT;
  w.t0 = n * BT;
  w.nvalid = min(BT, p.T - w.t0);
  w.rec_idx = (static_cast<size_t>(w.b) * p.H + w.h) * p.NT + n;
  return w;
}

template <bool G_BF16, bool FAST_EXP>
__global__ void __launch_bounds__(128, 4) kda_k1_kernel(const __grid_constant__ K1Params p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  using SM = K1Smem<G_BF16, FAST_EXP>;
  constexpr int S_Q = SM::Q, S_K = SM::K, S_V = SM::V, S_G = SM::G;
  constexpr uint32_t ROW_BYTES = D * 2;
  constexpr uint32_t G_ROW_BYTES = G_BF16 ? D * 2 : D * 4;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int gq = lane >> 2, tq = lane & 3;
  const int n_items = (p.chunk_table != nullptr ? p.n_chunks : p.B * p.NT) * p.H;

  const uint32_t sbase = smem_u32(smem);
  const uint32_t mbar = sbase + SM::MBAR;
  float* sL = reinterpret_cast<float*>(smem + S_L);
  float* sBetaAll = reinterpret_cast<float*>(smem + SM::BETA);   // [2][16], then expA[2] at +32
  float* sTot = reinterpret_cast<float*>(smem + SM::TOT);
  float* sGmid = reinterpret_cast<float*>(smem + SM::GMID);
  float* sTot1 = sTot + D;
  volatile int* sFlag = reinterpret_cast<volatile int*>(smem + SM::FLAG);

  const bool use_gate = (p.flags & 1u) != 0;
  const bool use_l2 = (p.flags & 2u) != 0;
  const int cp = tid & 63, rh = tid >> 6;   // phase-B mapping: column pair, row half
  const int c0 = cp * 2, r0 = rh * 8;

  if (tid == 0) {
    mbar_init(mbar, 1);
    sFlag[0] = 0;   // a wait gave up
    sFlag[1] = 0;   // the next item's q and k are already normalised
    fence_mbar_init();
  }
  __syncthreads();

  // issue the input copies of one work item: one tiled TMA box (16 tokens x 128) per tensor.
  // The box may reach past T in the last chunk; those rows arrive as zeros and still count
  // towards the transaction bytes.
  auto issue_loads = [&](const K1Item& w) {
    if (tid == 0) {
      mbar_arrive_expect_tx(mbar, BT * (3 * ROW_BYTES + G_ROW_BYTES));
      tma_load_4d(sbase + S_Q, &p.tm_q, 0, w.hq, w.t0, w.b, mbar);
      tma_load_4d(sbase + S_K, &p.tm_k, 0, w.hq, w.t0, w.b, mbar);
      tma_load_4d(sbase + S_V, &p.tm_v, 0, w.h, w.t0, w.b, mbar);
      tma_load_4d(sbase + S_G, &p.tm_g, 0, w.h, w.t0, w.b, mbar);
    }
  };
  // per-item parameters, fetched one item ahead so that their global-load latency is hidden
  struct Par { float a_log, bias0, bias1, beta; };
  auto load_params = [&](const K1Item& w) {
    Par q;
    q.a_log = use_gate ? ldg_pinned(p.A_log + w.h) : 0.f;
    q.bias0 = q.bias1 = 0.f;
    if (use_gate && p.dt_bias != nullptr) {
      const float2 bb = ldg_pinned2(p.dt_bias + w.h * D + c0);
      q.bias0 = bb.x; q.bias1 = bb.y;
    }
    q.beta = 0.f;   // held by threads 32..47 (warp 1), one token each
    if (tid >= 32 && tid < 48 && tid - 32 < w.nvalid)
      q.beta = ldg_pinned(p.beta + w.b * p.beta_s[0] + static_cast<int64_t>(w.t0 + tid - 32) * p.beta_s[1] + w.h * p.beta_s[2]);
    return q;
  };

  // Scalar per-item work -- exp(A_log) and the beta activation -- is done by warp 1 while warp 0
  // runs the triangular solve of the previous item, and handed over through shared memory.
  auto publish_params = [&](const Par& q, int nvalid_, int slot) {
    if (tid >= 32 && tid < 48) {
      float bv = q.beta;
      if (tid - 32 < nvalid_) { if (p.flags & 4u) bv = 1.0f / (1.0f + __expf(-bv)); } else bv = 0.f;
      sBetaAll[slot * 16 + tid - 32] = bv;
    }
    if (tid == 48) sBetaAll[32 + slot] = use_gate ? expf(q.a_log) : 1.f;
  };

  // l2-normalisation of the q and k tiles in place: 8 threads per row, two 16-byte units each (units seg
  // and seg + 8, so that a quarter-warp's 16-byte accesses cover 128 contiguous bytes).  `gid` numbers
  // the participating threads 0 .. nthr-1 (whole warps, nthr a multiple of 32).
  auto l2_normalise = [&](int gid, int nthr) {
    for (int task = gid; task < 128; task += nthr) {
      const int r = task >> 3, seg = task & 7;
      uint4 qa[2], ka[2];
      float sq = 0.f, sk = 0.f;
#pragma unroll
      for (int hseg = 0; hseg < 2; ++hseg) {
        qa[hseg] = *reinterpret_cast<const uint4*>(smem + S_Q + r * 256 + (seg + hseg * 8) * 16);
        ka[hseg] = *reinterpret_cast<const uint4*>(smem + S_K + r * 256 + (seg + hseg * 8) * 16);
        const uint32_t aw[4] = {qa[hseg].x, qa[hseg].y, qa[hseg].z, qa[hseg].w};
        const uint32_t cw[4] = {ka[hseg].x, ka[hseg].y, ka[hseg].z, ka[hseg].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float x0 = bf16_lo_to_f32(aw[i]), x1 = bf16_hi_to_f32(aw[i]);
          const float y0 = bf16_lo_to_f32(cw[i]), y1 = bf16_hi_to_f32(cw[i]);
          sq = fmaf(x0, x0, sq); sq = fmaf(x1, x1, sq);
          sk = fmaf(y0, y0, sk); sk = fmaf(y1, y1, sk);
        }
      }
#pragma unroll
      for (int m = 1; m < 8; m <<= 1) {
        sq += __shfl_xor_sync(0xffffffffu, sq, m);
        sk += __shfl_xor_sync(0xffffffffu, sk, m);
      }
      const float rq = rsqrtf(sq + L2NORM_EPS), rk = rsqrtf(sk + L2NORM_EPS);
      auto scale4 = [](uint4 v, float f) {
        uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) w[i] = pack_bf16(bf16_lo_to_f32(w[i]) * f, bf16_hi_to_f32(w[i]) * f);
        return make_uint4(w[0], w[1], w[2], w[3]);
      };
#pragma unroll
      for (int hseg = 0; hseg < 2; ++hseg) {
        *reinterpret_cast<uint4*>(smem + S_Q + r * 256 + (seg + hseg * 8) * 16) = scale4(qa[hseg], rq);
        *reinterpret_cast<uint4*>(smem + S_K + r * 256 + (seg + hseg * 8) * 16) = scale4(ka[hseg], rk);
      }
    }
  };

  int id = blockIdx.x;
  bool pre_normalised = false;   // the current item's q and k were normalised one iteration early
  K1Item cur{}, nxt{};
  Par par{}, par_next{};
  if (id < n_items) {
    cur = k1_item(p, id);
    issue_loads(cur);
    par = load_params(cur);
    publish_params(par, cur.nvalid, 0);
  }

  for (int it = 0; id < n_items; ++it, id += gridDim.x) {
    const int b = cur.b, h = cur.h, t0 = cur.t0, nvalid = cur.nvalid;
    uint8_t* rec = p.rec + cur.rec_idx * REC_BYTES;
    const bool has_next = id + static_cast<int>(gridDim.x) < n_items;
    if (has_next) {
      nxt = k1_item(p, id + gridDim.x);
      par_next = load_params(nxt);
    }
    const float bias0 = par.bias0, bias1 = par.bias1;
    const float* sBeta = sBetaAll + (it & 1) * 16;

    // every thread waits for the input copies itself (no CTA barrier here); a thread whose wait runs
    // out raises the flag, and the whole CTA leaves together behind the barrier that ends phase A
    const bool ok = mbar_wait_bounded(mbar, it & 1, sFlag);
    if (!ok) *sFlag = 1;

    // ---- phase A: l2-normalise q and k in place, unless warps 1..3 already did it under the previous
    //      item's solve ----
    if (use_l2 && ok && !pre_normalised) l2_normalise(tid, 128);
    __syncthreads();
    if (*sFlag != 0) {
      // a copy never completed: report, give in-flight copies one more bounded wait, leave
      if (tid == 0) {
        atomicExch(p.status, ST_K1_LOAD_TIMEOUT);
        mbar_wait_bounded(mbar, it & 1, nullptr);
      }
      __syncthreads();
      return;
    }

    // ---- phase B: thread = (column pair, row half): gate, cumsum, gated operands ----
    // Two adjacent columns per thread: every bf16 conversion is the packed cvt.rn.bf16x2
    // (full-rate pipe), every tile store is 32 bits wide and the fp32 arithmetic runs as
    // packed f32x2 instructions.
    // Centring of the Gram exponents.  General path: the chunk's middle row, as in the reference
    // (src/kda_bt16/kernels.py:129-139), which keeps every factor finite for any lower_bound
    // in (-11, 0).  FAST_EXP (16*|lower_bound|*RCP_LN2 <= 120, e.g. the production -5): the
    // LAST row, where 2^(g_last-g) <= 1 is exactly K2's kg operand, so the Grams reuse the kg
    // tiles as their B operand and 2^g = 2^(g-g_last) * 2^g_last costs no third exponential.
    uint32_t kbh[8], vbh[8], vbl[8];
    float2 dec2;
    {
      float2 gv[8];
      float2 gmid, glast;
      auto ld_g = [&](int r) -> float2 {
        if (G_BF16) {
          const uint32_t gp = *reinterpret_cast<const uint32_t*>(smem + S_G + (r * D + c0) * 2);
          return make_float2(bf16_lo_to_f32(gp), bf16_hi_to_f32(gp));
        }
        return *reinterpret_cast<const float2*>(smem + S_G + (r * D + c0) * 4);
      };
      if (use_gate) {
        // exp(-z) = 2^(nA * x + nb) with nA = -exp(A_log) log2(e), nb = nA * bias
        const float nA = -sBetaAll[32 + (it & 1)] * 1.4426950408889634f;
        const float2 nA2 = make_float2(nA, nA), nb2 = make_float2(nA * bias0, nA * bias1);
        const float2 one2 = make_float2(1.f, 1.f);
        const float lbr = p.lower_bound * RCP_LN2;
        const int mid = min(BT / 2, nvalid - 1);
        float2 run = make_float2(0.f, 0.f), gm = run;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = r0 + i;
          const float2 z = __ffma2_rn(ld_g(r), nA2, nb2);
          const float2 den = __fadd2_rn(make_float2(ex2f(z.x), ex2f(z.y)), one2);
          const float lb_r = (r < nvalid) ? lbr : 0.f;           // rows past the end add nothing
          const float2 gate = __fmul2_rn(make_float2(rcpf(den.x), rcpf(den.y)), make_float2(lb_r, lb_r));
          run = __fadd2_rn(run, gate);
          gv[i] = run;
          if (r == mid) gm = run;
        }
        // rows 8..15 need the sum over rows 0..7, all rows need g[last] and g[centre]: both halves
        // publish their column sums (and the half that owns the centre row its running sum there),
        // one barrier, and every thread completes its own values
        *reinterpret_cast<float2*>((rh == 0 ? sTot : sTot1) + c0) = run;
        if (!FAST_EXP && rh == (mid >> 3)) *reinterpret_cast<float2*>(sGmid + c0) = gm;
        // the previous item's bulk stores must have read the qg / kg / Aqk / dec tiles before the
        // operand loop below rewrites them; by now they have had two phases to do so
        if (tid == 0) bulk_wait_read_all();
        __syncthreads();
        const float2 t0 = *reinterpret_cast<const float2*>(sTot + c0);
        const float2 t1 = *reinterpret_cast<const float2*>(sTot1 + c0);
        if (rh == 1) {
#pragma unroll
          for (int i = 0; i < 8; ++i) gv[i] = __fadd2_rn(gv[i], t0);
        }
        glast = __fadd2_rn(t1, t0);
        gmid = make_float2(0.f, 0.f);
        if (!FAST_EXP) {
          gmid = *reinterpret_cast<const float2*>(sGmid + c0);
          if ((mid >> 3) == 1) gmid = __fadd2_rn(gmid, t0);
        }
      } else {
        // g already holds the chunk-local log2 cumsum; rows past the end repeat the last valid row
#pragma unroll
        for (int i = 0; i < 8; ++i) gv[i] = ld_g(min(r0 + i, nvalid - 1));
        gmid = ld_g(min(BT / 2, nvalid - 1));
        glast = ld_g(nvalid - 1);
        if (tid == 0) bulk_wait_read_all();   // as above
        __syncthreads();
      }
      dec2 = make_float2(ex2f(glast.x), ex2f(glast.y));
      if (rh == 1) *reinterpret_cast<float2*>(smem + S_DEC + c0 * 4) = dec2;

      if (p.g_out != nullptr) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (r0 + i < nvalid)
            *reinterpret_cast<float2*>(p.g_out + ((static_cast<size_t>(b) * p.T + t0 + r0 + i) * p.H + h) * D + c0) = gv[i];
      }

      const float2 centre = FAST_EXP ? glast : gmid;
      const float2 ncentre = make_float2(-centre.x, -centre.y);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int r = r0 + i;
        const uint32_t off = swz_off(r, c0);
        const uint32_t qp = *reinterpret_cast<const uint32_t*>(smem + S_Q + (r * D + c0) * 2);
        const uint32_t kp = *reinterpret_cast<const uint32_t*>(smem + S_K + (r * D + c0) * 2);
        const uint32_t vp = *reinterpret_cast<const uint32_t*>(smem + S_V + (r * D + c0) * 2);
        const float2 qn = make_float2(bf16_lo_to_f32(qp), bf16_hi_to_f32(qp));   // already normalised
        const float2 kn = make_float2(bf16_lo_to_f32(kp), bf16_hi_to_f32(kp));
        const float br = sBeta[r];
        const float2 d = __fadd2_rn(gv[i], ncentre);                  // g - centre
        const float2 e = make_float2(ex2f(d.x), ex2f(d.y));           // 2^(g - centre)
        const float2 en = make_float2(ex2f(-d.x), ex2f(-d.y));        // 2^(centre - g)
        float2 eg, ekg;                                               // 2^g, 2^(g_last - g)
        if (FAST_EXP) { eg = __fmul2_rn(e, dec2); ekg = en; }
        else {
          eg = make_float2(ex2f(gv[i].x), ex2f(gv[i].y));
          ekg = make_float2(ex2f(glast.x - gv[i].x), ex2f(glast.y - gv[i].y));
        }
        uint32_t hi, lo;
        split_pack2(__fmul2_rn(qn, e), hi, lo);
        *reinterpret_cast<uint32_t*>(smem + S_QGH + off) = hi;
        *reinterpret_cast<uint32_t*>(smem + S_QGL + off) = lo;
        split_pack2(__fmul2_rn(kn, e), hi, lo);
        *reinterpret_cast<uint32_t*>(smem + S_KQH + off) = hi;
        *reinterpret_cast<uint32_t*>(smem + S_KQL + off) = lo;
        if (!FAST_EXP) {
          split_pack2(__fmul2_rn(kn, en), hi, lo);
          *reinterpret_cast<uint32_t*>(smem + S_KNH + off) = hi;
          *reinterpret_cast<uint32_t*>(smem + S_KNL + off) = lo;
        }
        split_pack2(__fmul2_rn(kn, ekg), hi, lo);
        *reinterpret_cast<uint32_t*>(smem + S_KGH + off) = hi;
        *reinterpret_cast<uint32_t*>(smem + S_KGL + off) = lo;
        const float2 qgo = __fmul2_rn(qn, eg);
        *reinterpret_cast<uint32_t*>(smem + S_QG + off) = pack_bf16(qgo.x, qgo.y);
        const float2 kbv = __fmul2_rn(__fmul2_rn(kn, make_float2(br, br)), eg);
        kbh[i] = pack_bf16(kbv.x, kbv.y);
        split_pack2(__fmul2_rn(make_float2(bf16_lo_to_f32(vp), bf16_hi_to_f32(vp)), make_float2(br, br)), vbh[i], vbl[i]);
      }
    }
    __syncthreads();  // every thread has read its q/k/v/g elements: the input tiles are free

    // ---- prefetch: the next item's inputs go into the same tiles while this one finishes ----
    if (has_next) {
      if (tid == 0) fence_proxy_async();   // order the earlier generic accesses (made visible by the barrier) before the async writes
      issue_loads(nxt);
    }

    // ---- phase C: Grams on the tensor cores (one 16x8 output tile per warp) ----
    {
      const int mt = warp >> 1;  // 0: Aqk, 1: Akk
      const int nt = warp & 1;   // column block j in [8nt, 8nt+8)
      const int arow = (lane & 7) + ((lane >> 3) & 1) * 8, acol = (lane >> 4) * 8;
      const int brow = nt * 8 + (lane & 7), bcol = ((lane >> 3) & 1) * 8;
      // swizzled address of k-step ks = (256-byte aligned tile base + lane part) ^ (ks << 5)
      const uint32_t a_hi = sbase + (mt == 0 ? S_QGH : S_KQH) + swz_off(arow, acol);
      const uint32_t b_hi = sbase + (FAST_EXP ? S_KGH : S_KNH) + swz_off(brow, bcol);
      constexpr uint32_t A_LO = S_QGL - S_QGH, B_LO = FAST_EXP ? S_KGL - S_KGH : S_KNL - S_KNH;
      static_assert(S_KQL - S_KQH == S_QGL - S_QGH && S_GRAM % 256 == 0, "tile layout");
      float acc0[4] = {0, 0, 0, 0}, acc1[4] = {0, 0, 0, 0}, acc2[4] = {0, 0, 0, 0};
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        uint32_t ah[4], al[4], bh0, bh1, bl0, bl1;
        ldsm_x4(a_hi ^ (ks << 5), ah[0], ah[1], ah[2], ah[3]);
        ldsm_x4((a_hi ^ (ks << 5)) + A_LO, al[0], al[1], al[2], al[3]);
        ldsm_x2(b_hi ^ (ks << 5), bh0, bh1);
        ldsm_x2((b_hi ^ (ks << 5)) + B_LO, bl0, bl1);
        mma_bf16(acc0, ah, bh0, bh1);
        mma_bf16(acc1, ah, bl0, bl1);
        mma_bf16(acc2, al, bh0, bh1);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) acc0[e] += acc1[e] + acc2[e];
      const int j0 = nt * 8 + tq * 2;
      if (mt == 0) {
#pragma unroll
        for (int hrow = 0; hrow < 2; ++hrow) {
          const int i = gq + hrow * 8;
          const float v0 = (i >= j0) ? acc0[hrow * 2] * p.scale : 0.f;
          const float v1 = (i >= j0 + 1) ? acc0[hrow * 2 + 1] * p.scale : 0.f;
          uint32_t hi2, lo2;
          split_pack(v0, v1, hi2, lo2);
          *reinterpret_cast<uint32_t*>(smem + S_AQK + (i * 16 + j0) * 2) = hi2;
          *reinterpret_cast<uint32_t*>(smem + S_AQL + (i * 16 + j0) * 2) = lo2;
        }
      } else {
#pragma unroll
        for (int hrow = 0; hrow < 2; ++hrow) {
          const int i = gq + hrow * 8;
          const float bi = sBeta[i];
          // the solve consumes -Akk
          *reinterpret_cast<float2*>(sL + i * 16 + j0) =
              make_float2((i > j0) ? -acc0[hrow * 2] * bi : 0.f, (i > j0 + 1) ? -acc0[hrow * 2 + 1] * bi : 0.f);
        }
      }
    }
    __syncthreads();   // Grams done: their A tiles are free, -Akk is visible

    // B operands of w and u take the place of the Gram A tiles
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t off = swz_off(r0 + i, c0);
      *reinterpret_cast<uint32_t*>(smem + S_KBH + off) = kbh[i];
      *reinterpret_cast<uint32_t*>(smem + S_VBH + off) = vbh[i];
      *reinterpret_cast<uint32_t*>(smem + S_VBL + off) = vbl[i];
    }

    // next item's scalar parameters (warp 1, while warp 0 solves)
    if (has_next) publish_params(par_next, nxt.nvalid, (it + 1) & 1);

    // Warps 1..3 have nothing to do during the solve.  The next item's inputs were requested two
    // phases ago: if they have landed already (one probe, no waiting), those warps normalise its q
    // and k now, and the next iteration starts at the gate phase.
    if (warp != 0 && use_l2) {
      if (tid == 32) sFlag[1] = (has_next && mbar_test_wait(mbar, (it + 1) & 1)) ? 1 : 0;
      asm volatile("bar.sync 1, 96;" ::: "memory");   // warps 1..3 only
      if (sFlag[1] != 0) l2_normalise(tid - 32, 96);
    }

    // ---- phase D: X = (I + L)^-1, lane j of warp 0 owns column j ---------------
    // Column sweep (right-looking): once x[m] is final, every later row takes its update, so the
    // dependent chain is 16 FMAs long; -L is read four columns at a time.
    if (warp == 0 && lane < 16) {
      float x[BT];
#pragma unroll
      for (int i = 0; i < BT; ++i) x[i] = (i == lane) ? 1.f : 0.f;
#pragma unroll
      for (int mb = 0; mb < 4; ++mb) {
#pragma unroll
        for (int i = mb * 4 + 1; i < BT; ++i) {
          const float4 l4 = *reinterpret_cast<const float4*>(sL + i * 16 + mb * 4);
          const float lv[4] = {l4.x, l4.y, l4.z, l4.w};
#pragma unroll
          for (int mm = 0; mm < 4; ++mm)
            if (mb * 4 + mm < i) x[i] = fmaf(lv[mm], x[mb * 4 + mm], x[i]);
        }
      }
#pragma unroll
      for (int i = 0; i < BT; ++i) {
        const float hi = bf16_round(x[i]);
        *reinterpret_cast<unsigned short*>(smem + S_XH + (i * 16 + lane) * 2) = bf16_bits(hi);
        *reinterpret_cast<unsigned short*>(smem + S_XL + (i * 16 + lane) * 2) = bf16_bits(x[i] - hi);
      }
      if (p.ainv_out != nullptr) {
#pragma unroll
        for (int i = 0; i < BT; ++i)
          if (i < nvalid) p.ainv_out[((static_cast<size_t>(b) * p.T + t0 + i) * p.H + h) * BT + lane] = x[i];
      }
    }
    fence_proxy_async();   // qg / kg / Aqk / dec tiles were written with plain stores
    __syncthreads();
    const bool pre_next = use_l2 && sFlag[1] != 0;

    // the finished tiles leave while phase E runs
    if (tid == 0) {
      bulk_s2g(rec + REC_QG, sbase + S_QG, REC_AQK - REC_QG);
      bulk_s2g(rec + REC_AQK, sbase + S_AQK, REC_U - REC_AQK);
      bulk_commit();
    }

    // ---- phase E: u = X (v beta) (fp32-like, three split MMAs), w = X (khat beta 2^g) (bf16),
    //      u stored to the record straight from the accumulator fragments, w staged for a bulk store ----
    {
      // X as A operand (row-major [M=i][K=m]), hi and lo parts
      uint32_t xah[4], xal[4];
      {
        const int row2 = (lane & 7) + ((lane >> 3) & 1) * 8, col2 = (lane >> 4) * 8;
        ldsm_x4(sbase + S_XH + (row2 * 16 + col2) * 2, xah[0], xah[1], xah[2], xah[3]);
        ldsm_x4(sbase + S_XL + (row2 * 16 + col2) * 2, xal[0], xal[1], xal[2], xal[3]);
      }
      // B operands come from [tok][col] tiles through transposing ldmatrix; one x4 covers 16 columns
      const int btok = (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
      for (int ni = 0; ni < 2; ++ni) {
        const int n0 = warp * 32 + ni * 16;
        const int ccol = n0 + (lane >> 4) * 8;
        uint32_t bvh[4], bvl[4], bk[4];
        ldsm_x4_t(sbase + S_VBH + swz_off(btok, ccol), bvh[0], bvh[1], bvh[2], bvh[3]);
        ldsm_x4_t(sbase + S_VBL + swz_off(btok, ccol), bvl[0], bvl[1], bvl[2], bvl[3]);
        ldsm_x4_t(sbase + S_KBH + swz_off(btok, ccol), bk[0], bk[1], bk[2], bk[3]);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          // u tile: tokens x 8 value columns, stored as the raw accumulator fragment (K2 reads it back
          // into the same fragment): [column tile][lane][4]
          float acc[4] = {0, 0, 0, 0}, accl[4] = {0, 0, 0, 0};
          mma_bf16(acc, xah, bvh[2 * j], bvh[2 * j + 1]);
          mma_bf16(accl, xal, bvh[2 * j], bvh[2 * j + 1]);
          mma_bf16(accl, xah, bvl[2 * j], bvl[2 * j + 1]);
          const int vtile = (n0 >> 3) + j;
          *reinterpret_cast<float4*>(rec + REC_U + (vtile * 32 + lane) * 16) =
              make_float4(acc[0] + accl[0], acc[1] + accl[1], acc[2] + accl[2], acc[3] + accl[3]);
          float accw[4] = {0, 0, 0, 0};
          mma_bf16(accw, xah, bk[2 * j], bk[2 * j + 1]);
          mma_bf16(accw, xal, bk[2 * j], bk[2 * j + 1]);
          const int kc = n0 + j * 8 + tq * 2;
          *reinterpret_cast<uint32_t*>(smem + S_WST + swz_off(gq, kc)) = pack_bf16(accw[0], accw[1]);
          *reinterpret_cast<uint32_t*>(smem + S_WST + swz_off(gq + 8, kc)) = pack_bf16(accw[2], accw[3]);
        }
      }
    }
    // w leaves as one more bulk store (4-byte stores of a swizzled tile straight to global memory
    // would cost eight sectors per instruction)
    fence_proxy_async();
    __syncthreads();   // also orders phase E's reads of X / KB / VB before the next item rewrites them
    if (tid == 0) {
      bulk_s2g(rec + REC_W, sbase + S_WST, TILE_BYTES);
      bulk_commit();
    }
    cur = nxt;
    par = par_next;
    pre_normalised = pre_next;
  }
  if (tid == 0) bulk_wait_read_all();
}

template <bool G_BF16, bool FAST_EXP>
static cudaError_t launch_k1_t(const K1Params& p, cudaStream_t stream) {
  constexpr int smem_bytes = K1Smem<G_BF16, FAST_EXP>::TOTAL;
  static int grid_cap[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 64) return cudaErrorInvalidDevice;
  if (grid_cap[dev] == 0) {
    auto kern = kda_k1_kernel<G_BF16, FAST_EXP>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) return e;
    // ask for the full shared-memory carve-out so that four CTAs are resident per SM
    e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return e;
    int sms = 0, per_sm = 0;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, 128, smem_bytes);
    if (e != cudaSuccess) return e;
    grid_cap[dev] = sms * (per_sm > 0 ? per_sm : 1);   // persistent: one CTA per resident slot
  }
  const long long n_items = (p.chunk_table != nullptr ? static_cast<long long>(p.n_chunks) : static_cast<long long>(p.B) * p.NT) * p.H;
  const int grid = static_cast<int>(n_items < grid_cap[dev] ? n_items : grid_cap[dev]);
  kda_k1_kernel<G_BF16, FAST_EXP><<<grid, 128, smem_bytes, stream>>>(p);
  return cudaGetLastError();
}

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode_fn() {
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

cudaError_t k1_encode_tensor_maps(K1Params& p, bool g_bf16, const char** what) {
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) { *what = "cuTensorMapEncodeTiled is not available from this driver"; return cudaErrorNotSupported; }
  struct T { CUtensorMap* m; const void* ptr; const int64_t* s; CUtensorMapDataType dt; int es; const char* name; };
  const T ts[4] = {
      {&p.tm_q, p.q, p.q_s, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, "q"},
      {&p.tm_k, p.k, p.k_s, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, "k"},
      {&p.tm_v, p.v, p.v_s, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, "v"},
      {&p.tm_g, p.g, p.g_s, g_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, g_bf16 ? 2 : 4, "g"}};
  for (const T& t : ts) {
    // dims innermost first: (d, head, token, batch); strides in bytes for dims 1..3.  A size-1
    // dimension may come with any stride: give it a legal one (it is never stepped).  A zero
    // stride on a larger dimension (an expanded view) is refused by the argument check.
    const bool qk = (t.m == &p.tm_q || t.m == &p.tm_k);
    const cuuint64_t dims[4] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(qk ? p.Hq : p.H),
                                static_cast<cuuint64_t>(p.T), static_cast<cuuint64_t>(p.B)};
    cuuint64_t strides[3] = {static_cast<cuuint64_t>(t.s[2]) * t.es, static_cast<cuuint64_t>(t.s[1]) * t.es,
                             static_cast<cuuint64_t>(t.s[0]) * t.es};
    for (int i = 0; i < 3; ++i)
      if (dims[i + 1] == 1) strides[i] = static_cast<cuuint64_t>(D) * t.es;
    const cuuint32_t box[4] = {static_cast<cuuint32_t>(D), 1, static_cast<cuuint32_t>(BT), 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(t.m, t.dt, 4, const_cast<void*>(t.ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { *what = t.name; return cudaErrorInvalidValue; }
  }
  return cudaSuccess;
}

cudaError_t launch_k1(const K1Params& p, bool g_bf16, bool fast_exp, cudaStream_t stream) {
  if (g_bf16) return fast_exp ? launch_k1_t<true, true>(p, stream) : launch_k1_t<true, false>(p, stream);
  return fast_exp ? launch_k1_t<false, true>(p, stream) : launch_k1_t<false, false>(p, stream);
}

}  // namespace kda
