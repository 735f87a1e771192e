// Token-by-token KDA recurrence for decode and short sequences.  sm_100a.
//
// The reference has no decode kernel (its README lists prefill/decode separation as future work,
// README.md:503-505); the arithmetic is the token recurrence its tests use as the gold
// (fused_recurrent_kda at tests/test_kda_bt16.py:26-39), with the rounding points of the chunk
// path (normalised q, k rounded to bf16, everything else fp32), V-first state h[V][K]:
//   h   <- h * 2^gate[k]                       gate = lower_bound * sigmoid(e^A_log (g + bias)) / ln 2
//   v'  =  beta * (v - h khat)
//   h   <- h + v' (x) khat
//   o   =  scale * h qhat
// Every state row v is independent, so a warp owns ROWS rows of one (batch, head) state and keeps
// them in registers over all T tokens: lane l holds columns 4l..4l+3 of each row (one 16-byte
// load per row), the two dot products per row and token are warp reductions.  The kernel moves
// 64 KiB of state in and out per (batch, head) and a few hundred bytes per token: HBM bound; the
// grid is (batch x head) x (128 / rows per CTA) CTAs.  A K-first state h[K][V] (the layout
// flash-linear-attention keeps) is read and written in place: for one column k the warp's ROWS
// rows are ROWS consecutive floats, so the lane moves them as 16- or 8-byte pieces (full 32-byte
// sectors at 8 rows per warp) into the same registers.
#include "kda_common.cuh"
#include "kda_kernels.h"

namespace kda {

namespace {
constexpr int REC_WARPS = 4;   // warps per CTA

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) x += __shfl_xor_sync(0xffffffffu, x, m);
  return x;
}

// Sums N per-lane values over the warp at once: each exchange halves the number of values a lane
// still carries (the upper half of the lanes keeps the upper half of the rows), so N values cost
// N - 1 + (5 - log2 N) shuffles instead of 5 N.  Afterwards the lanes l with l >> (5 - log2 N) == r
// hold the total of value r.
template <int N> struct Log2 { static constexpr int v = 1 + Log2<N / 2>::v; };
template <> struct Log2<1> { static constexpr int v = 0; };
template <int N>
__device__ __forceinline__ float warp_sum_rows(float (&p)[N], int lane) {
  constexpr int LG = Log2<N>::v;
#pragma unroll
  for (int lv = 0; lv < LG; ++lv) {
    const int half = N >> (lv + 1), mask = 16 >> lv;
    const bool up = (lane & mask) != 0;
#pragma unroll
    for (int i = 0; i < half; ++i) {
      const float send = up ? p[i] : p[i + half];
      const float keep = up ? p[i + half] : p[i];
      p[i] = keep + __shfl_xor_sync(0xffffffffu, send, mask);
    }
  }
  float x = p[0];
#pragma unroll
  for (int lv = LG; lv < 5; ++lv) x += __shfl_xor_sync(0xffffffffu, x, 16 >> lv);
  return x;
}

template <int ROWS, bool G_BF16>
__global__ void __launch_bounds__(REC_WARPS * 32) kda_recurrent_kernel(const RecurrentParams p) {
  constexpr int ROWS_PER_CTA = ROWS * REC_WARPS;
  constexpr int SLICES = D / ROWS_PER_CTA;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int bh = blockIdx.x / SLICES, slice = blockIdx.x % SLICES;
  const int b = bh / p.H, h = bh % p.H;
  const int v0 = slice * ROWS_PER_CTA + warp * ROWS;   // first state row of this warp
  const int k0 = lane * 4;                             // first state column of this lane

  float4 s[ROWS];
  constexpr int PIECE = (ROWS % 4 == 0) ? 4 : 2;   // floats per access along v in the K-first layout
  if (p.h0 != nullptr && p.k_first) {
    const float* h0 = p.h0 + (static_cast<size_t>(bh) * D + k0) * D + v0;   // element (k0 + c, v0 + r) at c * D + r
    float t[4][ROWS];
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
      for (int r = 0; r < ROWS; r += PIECE) {
        if (PIECE == 4) {
          const float4 x = *reinterpret_cast<const float4*>(h0 + c * D + r);
          t[c][r] = x.x; t[c][r + 1] = x.y; t[c][r + 2] = x.z; t[c][r + 3] = x.w;
        } else {
          const float2 x = *reinterpret_cast<const float2*>(h0 + c * D + r);
          t[c][r] = x.x; t[c][r + 1] = x.y;
        }
      }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) s[r] = make_float4(t[0][r], t[1][r], t[2][r], t[3][r]);
  } else if (p.h0 != nullptr) {
    const float* h0 = p.h0 + (static_cast<size_t>(bh) * D + v0) * D + k0;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) s[r] = *reinterpret_cast<const float4*>(h0 + r * D);
  } else {
#pragma unroll
    for (int r = 0; r < ROWS; ++r) s[r] = make_float4(0.f, 0.f, 0.f, 0.f);
  }

  const float expA = expf(p.A_log[h]);
  float4 bias = make_float4(0.f, 0.f, 0.f, 0.f);
  if (p.dt_bias != nullptr) bias = *reinterpret_cast<const float4*>(p.dt_bias + h * D + k0);
  const float lbr = p.lower_bound * RCP_LN2;

  const int hq = h / p.group;   // grouped value heads share a q/k head
  const __nv_bfloat16* qp = p.q + b * p.q_s[0] + hq * p.q_s[2] + k0;
  const __nv_bfloat16* kp = p.k + b * p.k_s[0] + hq * p.k_s[2] + k0;
  const __nv_bfloat16* vp = p.v + b * p.v_s[0] + h * p.v_s[2] + v0 + (lane >> (5 - Log2<ROWS>::v));   // v of the row this lane reduces
  const uint8_t* gp = static_cast<const uint8_t*>(p.g) + (b * p.g_s[0] + h * p.g_s[2] + k0) * (G_BF16 ? 2 : 4);
  const float* bp = p.beta + b * p.beta_s[0] + h * p.beta_s[2];
  __nv_bfloat16* op = p.o + b * p.o_s[0] + h * p.o_s[2] + v0;

  auto load4 = [](const __nv_bfloat16* src) {
    const uint2 raw = *reinterpret_cast<const uint2*>(src);
    return make_float4(bf16_lo_to_f32(raw.x), bf16_hi_to_f32(raw.x), bf16_lo_to_f32(raw.y), bf16_hi_to_f32(raw.y));
  };

  for (int t = 0; t < p.T; ++t) {
    const float4 qr = load4(qp + t * p.q_s[1]);
    const float4 kr = load4(kp + t * p.k_s[1]);
    float4 gr;
    if (G_BF16) gr = load4(reinterpret_cast<const __nv_bfloat16*>(gp + t * p.g_s[1] * 2));
    else gr = *reinterpret_cast<const float4*>(gp + t * p.g_s[1] * 4);
    const float vmine = __bfloat162float(vp[t * p.v_s[1]]);
    float beta = bp[t * p.beta_s[1]];
    beta = 1.0f / (1.0f + __expf(-beta));

    // l2 normalisation, rounded to bf16 like the chunk path
    const float rq = rsqrtf(warp_sum(qr.x * qr.x + qr.y * qr.y + qr.z * qr.z + qr.w * qr.w) + L2NORM_EPS);
    const float rk = rsqrtf(warp_sum(kr.x * kr.x + kr.y * kr.y + kr.z * kr.z + kr.w * kr.w) + L2NORM_EPS);
    const float4 qn = make_float4(bf16_round(qr.x * rq), bf16_round(qr.y * rq), bf16_round(qr.z * rq), bf16_round(qr.w * rq));
    const float4 kn = make_float4(bf16_round(kr.x * rk), bf16_round(kr.y * rk), bf16_round(kr.z * rk), bf16_round(kr.w * rk));

    // decay 2^(lb * sigmoid(e^A (g + bias)) / ln 2) of this lane's four columns
    auto dec1 = [&](float g, float bi) {
      const float z = expA * (g + bi);
      return ex2f(lbr / (1.0f + __expf(-z)));
    };
    const float4 dc = make_float4(dec1(gr.x, bias.x), dec1(gr.y, bias.y), dec1(gr.z, bias.z), dec1(gr.w, bias.w));

    // the ROWS predictions h khat are reduced together; the lanes that end up with row r's total are
    // the ones that loaded v of row r (lane >> SH == r)
    constexpr int SH = 5 - Log2<ROWS>::v;
    float part[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      s[r].x *= dc.x; s[r].y *= dc.y; s[r].z *= dc.z; s[r].w *= dc.w;
      part[r] = s[r].x * kn.x + s[r].y * kn.y + s[r].z * kn.z + s[r].w * kn.w;
    }
    const float pred = warp_sum_rows<ROWS>(part, lane);
    const float vn_mine = beta * (vmine - pred);          // v' of row lane >> SH
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const float vn = __shfl_sync(0xffffffffu, vn_mine, r << SH);
      s[r].x = fmaf(vn, kn.x, s[r].x); s[r].y = fmaf(vn, kn.y, s[r].y);
      s[r].z = fmaf(vn, kn.z, s[r].z); s[r].w = fmaf(vn, kn.w, s[r].w);
      part[r] = s[r].x * qn.x + s[r].y * qn.y + s[r].z * qn.z + s[r].w * qn.w;
    }
    const float od = warp_sum_rows<ROWS>(part, lane);     // o of row lane >> SH
    if ((lane & ((1 << SH) - 1)) == 0) op[t * p.o_s[1] + (lane >> SH)] = __float2bfloat16(p.scale * od);
  }

  if (p.ht != nullptr && p.k_first) {
    float* ht = p.ht + (static_cast<size_t>(bh) * D + k0) * D + v0;
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
      for (int r = 0; r < ROWS; r += PIECE) {
        auto comp = [&](int rr) { return c == 0 ? s[rr].x : (c == 1 ? s[rr].y : (c == 2 ? s[rr].z : s[rr].w)); };
        if (PIECE == 4) *reinterpret_cast<float4*>(ht + c * D + r) = make_float4(comp(r), comp(r + 1), comp(r + 2), comp(r + 3));
        else *reinterpret_cast<float2*>(ht + c * D + r) = make_float2(comp(r), comp(r + 1));
      }
  } else if (p.ht != nullptr) {
    float* ht = p.ht + (static_cast<size_t>(bh) * D + v0) * D + k0;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) *reinterpret_cast<float4*>(ht + r * D) = s[r];
  }
}

// K-first state h[K][V] with enough heads to fill the GPU: lanes along v.
// A CTA owns all 128 k of a 32-wide slice of v (one full 128-byte line per k); thread (vq = tid % 8,
// kg = tid / 8) keeps rows k = 8 kg .. 8 kg + 7 of columns v = 4 vq .. 4 vq + 3 of that slice in
// registers (eight 16-byte accesses, four whole lines per warp instruction -- the access pattern of
// the V-first kernel above on the transposed state).  The two dot products per token run over k:
// serial over the thread's eight rows, two shuffles over the four k-groups of a warp, and a
// 512-byte exchange through shared memory over the four warps (two CTA barriers per token).
// Same arithmetic and rounding points as the kernel above; the fp32 sums run in another order.
template <bool G_BF16>
__global__ void __launch_bounds__(128) kda_recurrent_kfirst_kernel(const RecurrentParams p) {
  __shared__ float4 red[2][4][8];   // [prediction | output][warp][v quad]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int vq = tid & 7, kg = tid >> 3;
  const int bh = blockIdx.x >> 2, slice = blockIdx.x & 3;
  const int b = bh / p.H, h = bh % p.H;
  const int v0 = slice * 32 + vq * 4;   // first state column of this thread
  const int k0 = kg * 8;                // first state row of this thread

  float4 s[8];
  if (p.h0 != nullptr) {
    const float* h0 = p.h0 + (static_cast<size_t>(bh) * D + k0) * D + v0;
#pragma unroll
    for (int i = 0; i < 8; ++i) s[i] = *reinterpret_cast<const float4*>(h0 + i * D);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) s[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }

  const float expA = expf(p.A_log[h]);
  float bias[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) bias[i] = (p.dt_bias != nullptr) ? p.dt_bias[h * D + k0 + i] : 0.f;
  const float lbr = p.lower_bound * RCP_LN2;

  const int hq = h / p.group;   // grouped value heads share a q/k head
  const __nv_bfloat16* qp = p.q + b * p.q_s[0] + hq * p.q_s[2];
  const __nv_bfloat16* kp = p.k + b * p.k_s[0] + hq * p.k_s[2];
  const __nv_bfloat16* vp = p.v + b * p.v_s[0] + h * p.v_s[2] + v0;
  const uint8_t* gp = static_cast<const uint8_t*>(p.g) + (b * p.g_s[0] + h * p.g_s[2] + k0) * (G_BF16 ? 2 : 4);
  const float* bp = p.beta + b * p.beta_s[0] + h * p.beta_s[2];
  __nv_bfloat16* op = p.o + b * p.o_s[0] + h * p.o_s[2] + v0;

  auto load4 = [](const __nv_bfloat16* src) {
    const uint2 raw = *reinterpret_cast<const uint2*>(src);
    return make_float4(bf16_lo_to_f32(raw.x), bf16_hi_to_f32(raw.x), bf16_lo_to_f32(raw.y), bf16_hi_to_f32(raw.y));
  };
  auto load8 = [](const __nv_bfloat16* src, float (&x)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(src);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { x[2 * i] = bf16_lo_to_f32(w[i]); x[2 * i + 1] = bf16_hi_to_f32(w[i]); }
  };
  // sum over the k-groups of this warp (lanes with the same vq), then over the warps
  auto reduce_k = [&](float4 x, int which) {
#pragma unroll
    for (int m = 8; m <= 16; m <<= 1) {
      x.x += __shfl_xor_sync(0xffffffffu, x.x, m); x.y += __shfl_xor_sync(0xffffffffu, x.y, m);
      x.z += __shfl_xor_sync(0xffffffffu, x.z, m); x.w += __shfl_xor_sync(0xffffffffu, x.w, m);
    }
    if (lane < 8) red[which][warp][vq] = x;
    __syncthreads();
    const float4 a = red[which][0][vq], c = red[which][1][vq], d = red[which][2][vq], e = red[which][3][vq];
    return make_float4((a.x + c.x) + (d.x + e.x), (a.y + c.y) + (d.y + e.y), (a.z + c.z) + (d.z + e.z), (a.w + c.w) + (d.w + e.w));
  };

  for (int t = 0; t < p.T; ++t) {
    // l2 norms over all 128 k: every warp computes them (lane l: k = 4 l .. 4 l + 3), rounded to bf16 like the chunk path
    const float4 qa = load4(qp + t * p.q_s[1] + lane * 4);
    const float4 ka = load4(kp + t * p.k_s[1] + lane * 4);
    const float rq = rsqrtf(warp_sum(qa.x * qa.x + qa.y * qa.y + qa.z * qa.z + qa.w * qa.w) + L2NORM_EPS);
    const float rk = rsqrtf(warp_sum(ka.x * ka.x + ka.y * ka.y + ka.z * ka.z + ka.w * ka.w) + L2NORM_EPS);
    float qn[8], kn[8], gr[8];
    load8(qp + t * p.q_s[1] + k0, qn);
    load8(kp + t * p.k_s[1] + k0, kn);
    if (G_BF16) load8(reinterpret_cast<const __nv_bfloat16*>(gp + t * p.g_s[1] * 2), gr);
    else {
      const float4 g0 = *reinterpret_cast<const float4*>(gp + t * p.g_s[1] * 4);
      const float4 g1 = *reinterpret_cast<const float4*>(gp + t * p.g_s[1] * 4 + 16);
      gr[0] = g0.x; gr[1] = g0.y; gr[2] = g0.z; gr[3] = g0.w; gr[4] = g1.x; gr[5] = g1.y; gr[6] = g1.z; gr[7] = g1.w;
    }
    const float4 v4 = load4(vp + t * p.v_s[1]);
    float beta = bp[t * p.beta_s[1]];
    beta = 1.0f / (1.0f + __expf(-beta));

    float4 part = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      qn[i] = bf16_round(qn[i] * rq);
      kn[i] = bf16_round(kn[i] * rk);
      // decay 2^(lb * sigmoid(e^A (g + bias)) / ln 2) of row k0 + i
      const float z = expA * (gr[i] + bias[i]);
      const float dc = ex2f(lbr / (1.0f + __expf(-z)));
      s[i].x *= dc; s[i].y *= dc; s[i].z *= dc; s[i].w *= dc;
      part.x = fmaf(s[i].x, kn[i], part.x); part.y = fmaf(s[i].y, kn[i], part.y);
      part.z = fmaf(s[i].z, kn[i], part.z); part.w = fmaf(s[i].w, kn[i], part.w);
    }
    const float4 pred = reduce_k(part, 0);
    const float4 vn = make_float4(beta * (v4.x - pred.x), beta * (v4.y - pred.y), beta * (v4.z - pred.z), beta * (v4.w - pred.w));
    part = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      s[i].x = fmaf(vn.x, kn[i], s[i].x); s[i].y = fmaf(vn.y, kn[i], s[i].y);
      s[i].z = fmaf(vn.z, kn[i], s[i].z); s[i].w = fmaf(vn.w, kn[i], s[i].w);
      part.x = fmaf(s[i].x, qn[i], part.x); part.y = fmaf(s[i].y, qn[i], part.y);
      part.z = fmaf(s[i].z, qn[i], part.z); part.w = fmaf(s[i].w, qn[i], part.w);
    }
    const float4 od = reduce_k(part, 1);
    if (tid < 8) {
      uint2 out;
      out.x = pack_bf16(p.scale * od.x, p.scale * od.y);
      out.y = pack_bf16(p.scale * od.z, p.scale * od.w);
      *reinterpret_cast<uint2*>(op + t * p.o_s[1]) = out;
    }
  }

  if (p.ht != nullptr) {
    float* ht = p.ht + (static_cast<size_t>(bh) * D + k0) * D + v0;
#pragma unroll
    for (int i = 0; i < 8; ++i) *reinterpret_cast<float4*>(ht + i * D) = s[i];
  }
}

template <int ROWS>
cudaError_t launch_rows(const RecurrentParams& p, bool g_bf16, cudaStream_t stream) {
  const int grid = p.B * p.H * (D / (ROWS * REC_WARPS));
  if (g_bf16) kda_recurrent_kernel<ROWS, true><<<grid, REC_WARPS * 32, 0, stream>>>(p);
  else kda_recurrent_kernel<ROWS, false><<<grid, REC_WARPS * 32, 0, stream>>>(p);
  return cudaGetLastError();
}
}  // namespace

// rows per warp: 8 (four CTAs per head) once there are enough heads to fill the GPU, else 2
// (sixteen CTAs per head) so that a handful of heads still spreads over many SMs
cudaError_t launch_recurrent(const RecurrentParams& p, bool g_bf16, int sms, cudaStream_t stream) {
  const long long bh = static_cast<long long>(p.B) * p.H;
  if (p.k_first && bh * 4 >= 2LL * sms) {
    // four CTAs per head with the lanes along v; with fewer heads the calls are latency-bound and the
    // row-per-warp kernel's strided state accesses cost nothing measurable
    const int grid = static_cast<int>(bh) * 4;
    if (g_bf16) kda_recurrent_kfirst_kernel<true><<<grid, 128, 0, stream>>>(p);
    else kda_recurrent_kfirst_kernel<false><<<grid, 128, 0, stream>>>(p);
    return cudaGetLastError();
  }
  if (bh * 4 >= 2LL * sms) return launch_rows<8>(p, g_bf16, stream);
  if (bh * 8 >= 2LL * sms) return launch_rows<4>(p, g_bf16, stream);
  return launch_rows<2>(p, g_bf16, stream);
}

}  // namespace kda
