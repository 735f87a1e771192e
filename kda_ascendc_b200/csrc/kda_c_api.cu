// C-ABI layer of libkda_b200.so: argument checks, workspace arithmetic, stage launches.
// Interface and the reference entry points it stands in for: include/kda_b200.h.
#include <cstddef>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <vector>

#include <cuda.h>

#include "../../include/kda_b200.h"
#include "kda_common.cuh"
#include "kda_kernels.h"

static_assert(sizeof(KdaFwdArgs) == 312 && offsetof(KdaFwdArgs, chunk_table) == 288 && offsetof(KdaFwdArgs, Hq) == 308,
              "KdaFwdArgs layout is part of the ABI (bindings mirror it field by field)");

namespace {

thread_local char g_err[512] = "";
thread_local int g_launches = 0;

int fail(int code, const char* fmt, const char* a = "", long long x = 0, long long y = 0) {
  snprintf(g_err, sizeof(g_err), fmt, a, x, y);
  return code;
}

int check_common(const KdaFwdArgs* a) {
  if (a == nullptr) return fail(KDA_ERR_INVALID_ARG, "kda: args is NULL%s", "");
  if (a->B <= 0 || a->T <= 0 || a->H <= 0)
    return fail(KDA_ERR_INVALID_ARG, "kda: B, T, H must be positive%s (T=%lld, H=%lld)", "", a->T, a->H);
  if (a->workspace == nullptr) return fail(KDA_ERR_INVALID_ARG, "kda: workspace is NULL%s", "");
  if (reinterpret_cast<uintptr_t>(a->workspace) % 256 != 0)
    return fail(KDA_ERR_INVALID_ARG, "kda: workspace must be 256-byte aligned%s", "");
  if (a->Hq < 0 || (a->Hq > 0 && a->H % a->Hq != 0))
    return fail(KDA_ERR_INVALID_ARG, "kda: H%s (%lld) must be a multiple of Hq (%lld)", "", a->H, a->Hq);
  if (a->n_seqs < 0) return fail(KDA_ERR_INVALID_ARG, "kda: n_seqs must not be negative%s", "");
  if (a->n_seqs > 0) {
    if (a->B != 1) return fail(KDA_ERR_INVALID_ARG, "kda: packed sequences need B = 1%s (got %lld)", "", a->B);
    if (a->chunk_table == nullptr || a->seq_table == nullptr || a->n_chunks <= 0)
      return fail(KDA_ERR_INVALID_ARG, "kda: packed sequences need chunk_table, seq_table and n_chunks%s", "");
    if (reinterpret_cast<uintptr_t>(a->chunk_table) % 16 != 0 || reinterpret_cast<uintptr_t>(a->seq_table) % 16 != 0)
      return fail(KDA_ERR_INVALID_ARG, "kda: chunk_table and seq_table must be 16-byte aligned%s", "");
    if (a->g_out != nullptr || a->ainv_out != nullptr)
      return fail(KDA_ERR_INVALID_ARG, "kda: the debug outputs are not available with packed sequences%s", "");
  }
  return KDA_OK;
}

bool row_aligned(const void* p, const int64_t s[3], int elem_bytes) {
  if (reinterpret_cast<uintptr_t>(p) % 16 != 0) return false;
  for (int i = 0; i < 3; ++i)
    if ((s[i] * elem_bytes) % 16 != 0) return false;
  return true;
}

int check_k1(const KdaFwdArgs* a) {
  if (int rc = check_common(a)) return rc;
  if (!a->q || !a->k || !a->v || !a->g || !a->beta)
    return fail(KDA_ERR_INVALID_ARG, "kda: q, k, v, g and beta are required%s", "");
  if (a->g_dtype != KDA_G_FP32 && a->g_dtype != KDA_G_BF16)
    return fail(KDA_ERR_INVALID_ARG, "kda: g_dtype must be KDA_G_FP32 or KDA_G_BF16%s (got %lld)", "", a->g_dtype);
  if ((a->flags & KDA_FLAG_GATE_IN_KERNEL) && a->A_log == nullptr)
    return fail(KDA_ERR_INVALID_ARG, "kda: the in-kernel gate requires A_log%s", "");
  if ((a->flags & KDA_FLAG_GATE_IN_KERNEL) && !(a->lower_bound > -11.0f && a->lower_bound < 0.0f))
    return fail(KDA_ERR_INVALID_ARG, "kda: lower_bound must be in (-11, 0)%s", "");
  if (!row_aligned(a->q, a->q_stride, 2) || !row_aligned(a->k, a->k_stride, 2) || !row_aligned(a->v, a->v_stride, 2) ||
      !row_aligned(a->g, a->g_stride, a->g_dtype == KDA_G_BF16 ? 2 : 4))
    return fail(KDA_ERR_INVALID_ARG, "kda: q/k/v/g rows must start on 16-byte boundaries%s", "");
  // an expanded view (stride 0 on a dimension larger than 1) cannot be described to the TMA unit
  const int hq = a->Hq > 0 ? a->Hq : a->H;
  const struct { const int64_t* s; int heads; const char* name; } views[4] = {
      {a->q_stride, hq, "q"}, {a->k_stride, hq, "k"}, {a->v_stride, a->H, "v"}, {a->g_stride, a->H, "g"}};
  for (const auto& v : views) {
    const int sizes[3] = {a->B, a->T, v.heads};
    for (int i = 0; i < 3; ++i)
      if (sizes[i] > 1 && v.s[i] <= 0)
        return fail(KDA_ERR_INVALID_ARG, "kda: %s has a zero or negative stride on a dimension of size %lld (expanded views are not supported)",
                    v.name, sizes[i]);
  }
  return KDA_OK;
}

int check_k2(const KdaFwdArgs* a, bool state_only) {
  if (int rc = check_common(a)) return rc;
  if (!state_only && a->o == nullptr) return fail(KDA_ERR_INVALID_ARG, "kda: o is NULL%s", "");
  if (!state_only && !row_aligned(a->o, a->o_stride, 2))
    return fail(KDA_ERR_INVALID_ARG, "kda: o rows must start on 16-byte boundaries%s", "");
  for (const void* ptr : {static_cast<const void*>(a->h0), static_cast<const void*>(a->ht)})
    if (ptr != nullptr && reinterpret_cast<uintptr_t>(ptr) % 16 != 0)
      return fail(KDA_ERR_INVALID_ARG, "kda: h0 and ht must be 16-byte aligned%s", "");
  const int vs = a->k2_vsplit, var = a->k2_variant;
  if (var < 0 || var > 5 || var == 2)
    return fail(KDA_ERR_INVALID_ARG, "kda: k2_variant must be 0, 1, 3, 4 or 5%s (got %lld)", "", var);
  if (var == 4 && state_only)
    return fail(KDA_ERR_INVALID_ARG, "kda: the tensor-memory K2 (k2_variant 4) has no state-only form%s", "");
  if (var == 4) return KDA_OK;
  if (vs != 0 && vs != 2 && vs != 4 && vs != 8 && vs != 16)
    return fail(KDA_ERR_INVALID_ARG, "kda: k2_vsplit must be 0, 2, 4, 8 or 16%s (got %lld)", "", vs);
  if (vs != 0 && var != 0 && ((var == 1 || var == 5) ? (vs < 4) : (vs > 8)))
    return fail(KDA_ERR_INVALID_ARG, "kda: k2_vsplit %lld%s does not go with k2_variant %lld", "", vs, var);
  return KDA_OK;
}

// How one head's 128x128 state is spread over warps.  The recurrence is a serial chain per head;
// a warp alone on an SM sub-partition cannot overlap its own MMA issue with its other
// instructions, so a step costs about 8 cycles per MMA plus its non-MMA instructions, and every
// warp re-reads the shared operand tiles from shared memory.  Measured on B200 (T = 8192):
// up to ~37 (batch x head) chains the 8-rows-per-warp "n8" form wins (two warps per SM while
// chains x 8 CTAs fit the SMs, else four); beyond that the 16-rows-per-warp "m16" form with four
// warps per CTA, which reads half the shared-memory bytes per MMA.  With more chains than SMs the
// tensor-memory form (one CTA per chain, two per SM, tcgen05) is 10-35 % faster still once the
// chains are a few chunks long: its set-up (TMEM allocation, the state in and out through
// registers) costs about as much as two steps.  2,048 chains x 1 chunk: 81 us against 80 us,
// x 4: 126 against 134, x 16: 243 against 343; 1,024 chains x 64: 404 against 601; 256 chains
// x 4: 17 against 21 -- hence from four chunks per chain on.  Between half as many chains as SMs and as many
// (where the 16-row form needs two CTAs per chain and so more than one CTA per SM) it wins from
// about 32 chunks per chain: 96 chains x 64 chunks 85 us against 92, x 16 equal.  It has no
// state-only variant.
void pick_split(const KdaFwdArgs* a, bool state_only, int* vsplit, int* variant, int sms = 0, int chain_mult = 1) {
  if (sms <= 0) {   // the current device's SM count
    int dev = 0;
    sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const long long bh = static_cast<long long>(a->n_seqs > 0 ? a->n_seqs : a->B) * a->H * chain_mult;
  // chunks per chain (the mean, for packed sequences)
  const long long steps = a->n_seqs > 0 ? a->n_chunks / a->n_seqs : (a->T + kda::BT - 1) / kda::BT;
  int var = a->k2_variant;
  int vs = a->k2_vsplit;
  if (var == 0) {
    if (vs == 16) var = 1;
    else if (vs == 2) var = 3;
    else if (!state_only && vs == 0 && ((bh > sms && steps >= 4) || (bh * 2 > sms && steps >= 32))) var = 4;
    else var = (bh * 4 <= sms) ? 1 : 3;
  }
  if (vs == 0) {
    if (var == 1 || var == 5) vs = (bh * 16 <= sms) ? 16 : (bh * 8 <= sms) ? 8 : 4;
    else vs = (bh * 4 <= sms) ? 4 : 2;
  }
  if ((var == 1 || var == 5) && vs < 4) vs = 4;
  if (var != 1 && var != 5 && vs > 8) vs = 8;
  *vsplit = vs;
  *variant = var;
}

int* status_ptr(const KdaFwdArgs* a) { return static_cast<int*>(a->workspace); }
uint8_t* rec_ptr(const KdaFwdArgs* a) { return static_cast<uint8_t*>(a->workspace) + kda::WS_HEADER_BYTES; }

int do_k1(const KdaFwdArgs* a, cudaStream_t st) {
  kda::K1Params p;
  memset(&p, 0, sizeof(p));
  p.q = static_cast<const __nv_bfloat16*>(a->q);
  p.k = static_cast<const __nv_bfloat16*>(a->k);
  p.v = static_cast<const __nv_bfloat16*>(a->v);
  p.g = a->g;
  p.beta = a->beta;
  p.A_log = a->A_log;
  p.dt_bias = a->dt_bias;
  p.rec = rec_ptr(a);
  p.status = status_ptr(a);
  p.g_out = a->g_out;
  p.ainv_out = a->ainv_out;
  p.B = a->B; p.T = a->T; p.H = a->H; p.NT = (a->T + kda::BT - 1) / kda::BT;
  p.div_h.set(static_cast<uint32_t>(p.H));
  p.div_nt.set(static_cast<uint32_t>(p.NT));
  for (int i = 0; i < 3; ++i) {
    p.q_s[i] = a->q_stride[i]; p.k_s[i] = a->k_stride[i]; p.v_s[i] = a->v_stride[i];
    p.g_s[i] = a->g_stride[i]; p.beta_s[i] = a->beta_stride[i];
  }
  p.scale = a->scale;
  p.lower_bound = a->lower_bound;
  p.flags = a->flags;
  if (a->n_seqs > 0) {
    p.chunk_table = reinterpret_cast<const int4*>(a->chunk_table);
    p.n_chunks = a->n_chunks;
  }
  p.Hq = a->Hq > 0 ? a->Hq : a->H;
  p.div_g.set(static_cast<uint32_t>(p.H / p.Hq));
  // 2^g may be factored as 2^(g-g_mid) * 2^(g_mid) only while no factor can underflow:
  // 16 tokens * |lower_bound| * RCP_LN2 must stay inside the fp32 exponent range.
  const bool fast_exp = (a->flags & KDA_FLAG_GATE_IN_KERNEL) && (16.0f * -a->lower_bound * kda::RCP_LN2 <= 120.0f);
  // The four tensor maps depend only on the input pointers, sizes and strides: a loop that calls with
  // the same buffers (a serving loop, a benchmark) re-uses the maps of its previous call.
  struct MapKey {
    const void *q, *k, *v, *g;
    int32_t B, T, H, Hq, g_dtype;
    int64_t s[12];
  };
  thread_local MapKey last_key;
  thread_local CUtensorMap last_maps[4];
  thread_local bool have_maps = false;
  MapKey key;
  memset(&key, 0, sizeof(key));
  key.q = a->q; key.k = a->k; key.v = a->v; key.g = a->g;
  key.B = a->B; key.T = a->T; key.H = a->H; key.Hq = p.Hq; key.g_dtype = a->g_dtype;
  for (int i = 0; i < 3; ++i) {
    key.s[i] = a->q_stride[i]; key.s[3 + i] = a->k_stride[i]; key.s[6 + i] = a->v_stride[i]; key.s[9 + i] = a->g_stride[i];
  }
  cudaError_t e = cudaSuccess;
  if (have_maps && memcmp(&key, &last_key, sizeof(key)) == 0) {
    p.tm_q = last_maps[0]; p.tm_k = last_maps[1]; p.tm_v = last_maps[2]; p.tm_g = last_maps[3];
  } else {
    const char* what = "";
    e = kda::k1_encode_tensor_maps(p, a->g_dtype == KDA_G_BF16, &what);
    if (e != cudaSuccess) return fail(KDA_ERR_CUDA, "kda: building the TMA descriptor failed for: %s", what);
    last_key = key;
    last_maps[0] = p.tm_q; last_maps[1] = p.tm_k; last_maps[2] = p.tm_v; last_maps[3] = p.tm_g;
    have_maps = true;
  }
  e = kda::launch_k1(p, a->g_dtype == KDA_G_BF16, fast_exp, st);
  if (e != cudaSuccess) return fail(KDA_ERR_CUDA, "kda: K1 launch failed: %s", cudaGetErrorString(e));
  ++g_launches;
  return KDA_OK;
}

struct H0Flags { const int32_t* flags; int n, epoch; };

int do_k2(const KdaFwdArgs* a, bool state_only, int zero_u, cudaStream_t st, const KdaPeerPushArgs* push = nullptr,
          const H0Flags* h0f = nullptr) {
  kda::K2Params p;
  memset(&p, 0, sizeof(p));
  p.rec = rec_ptr(a);
  p.h0 = a->h0;
  p.o = static_cast<__nv_bfloat16*>(a->o);
  p.ht = a->ht;
  p.status = status_ptr(a);
  p.B = a->B; p.T = a->T; p.H = a->H; p.NT = (a->T + kda::BT - 1) / kda::BT;
  for (int i = 0; i < 3; ++i) p.o_s[i] = a->o_stride[i];
  p.scale = a->scale;
  p.zero_u = zero_u == 1;
  p.k_first = (a->flags & KDA_FLAG_STATE_K_FIRST) ? 1 : 0;
  p.pair_mode = (state_only && zero_u == 2) ? 1 : 0;
  if (a->n_seqs > 0) {
    p.seq_table = reinterpret_cast<const int4*>(a->seq_table);
    p.n_seqs = a->n_seqs;
  }
  int vsplit = 4, variant = 3;
  pick_split(a, state_only, &vsplit, &variant);
  if (p.pair_mode) {
    p.k_first = 0;   // the transforms are always written [chains][2][V][K]
    // Both transforms of a segment in one launch.  Few chains (two recurrences per chain still give
    // every warp an SM sub-partition to itself): the 8-row form over twice as many chains.  Up to
    // the 8-row form's own limit: the two recurrences share a warp and its operand loads.  Beyond:
    // the 16-row form over twice as many chains.
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long bh = static_cast<long long>(a->n_seqs > 0 ? a->n_seqs : a->B) * a->H;
    if (2 * bh > 0x3fffffffLL) return fail(KDA_ERR_INVALID_ARG, "kda: too many chains%s", "");
    cudaError_t pe;
    if (push != nullptr) {
      // the tiles go straight into the owners' receive buffers: only the 8-row pair form does that
      if (!(variant == 1 || variant == 5))
        return fail(KDA_ERR_UNSUPPORTED, "kda: the fused push needs the 8-row pair form%s (too many chains: %lld)", "", bh);
      const long long hp = push->slice_floats / (2LL * kda::D * kda::D);
      if (hp <= 0 || hp * push->world != bh || push->slice_floats % (2LL * kda::D * kda::D) != 0)
        return fail(KDA_ERR_INVALID_ARG, "kda: slice_floats must be chains / world whole (M, Q) pairs%s (chains %lld)", "", bh);
      p.push_on = 1;
      p.push_hp = static_cast<int>(hp);
      p.push_epoch = push->epoch;
      p.push_dst_offset = push->dst_offset_floats;
      p.push_counter = push->counter;
      for (int d = 0; d < push->world; ++d) { p.push_dst[d] = push->dst[d]; p.push_flag[d] = push->flag[d]; }
      p.pair_mode = 0;
      pe = kda::launch_k2n_pair(p, vsplit, st);
    } else if (a->k2_variant == 0 && a->k2_vsplit == 0 && 2 * bh * 4 <= sms) {
      p.n_chains = static_cast<int>(2 * bh);
      pe = kda::launch_k2n(p, 2 * bh * 16 <= sms ? 16 : 2 * bh * 8 <= sms ? 8 : 4, 1, true, st);
    } else if (variant == 1 || variant == 5) {
      p.pair_mode = 0;   // the pair is compiled into the kernel
      pe = kda::launch_k2n_pair(p, vsplit, st);
    } else {
      p.n_chains = static_cast<int>(2 * bh);
      pick_split(a, state_only, &vsplit, &variant, 0, 2);
      pe = (variant == 3) ? kda::launch_k2m(p, vsplit, true, st) : cudaErrorInvalidValue;
    }
    if (pe != cudaSuccess) return fail(KDA_ERR_CUDA, "kda: K2 (transform pair) launch failed: %s", cudaGetErrorString(pe));
    ++g_launches;
    return KDA_OK;
  }
  if (h0f != nullptr) {
    // the entry state is stored by other GPUs: the kernels that can wait for it themselves are the 8-row and
    // the 16-row form
    if (!(variant == 1 || variant == 3))
      return fail(KDA_ERR_UNSUPPORTED, "kda: this K2 form cannot wait for the entry state%s (variant %lld)", "", variant);
    p.h0_flags = h0f->flags; p.h0_n_flags = h0f->n; p.h0_epoch = h0f->epoch;
  }
  cudaError_t e;
  if (variant == 4) {
    const long long n_records = a->n_seqs > 0 ? static_cast<long long>(a->n_chunks) * a->H
                                              : static_cast<long long>(a->B) * a->H * p.NT;
    // Tail wave.  The tensor-memory form holds two chains per SM at once; when the chains left over
    // after the full waves are at most half as many as SMs, they run faster in an mma.sync form
    // (16-row: two CTAs per chain, one per SM, 0.8 us per step; 8-row for at most SMs/4 chains,
    // 0.55 us per step; against 1.3 us for a lone tensor-memory CTA), launched behind the full
    // waves.  Only for the automatic choice.
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long bh = static_cast<long long>(a->n_seqs > 0 ? a->n_seqs : a->B) * a->H;
    const long long tail = bh % (2LL * sms);
    if (a->k2_variant == 0 && bh > 2LL * sms && tail > 0 && tail * 2 <= sms) {
      p.chain0 = 0;
      p.n_chains = static_cast<int>(bh - tail);
      e = kda::launch_k2t(p, n_records, st);
      if (e == cudaSuccess) {
        ++g_launches;
        p.chain0 = static_cast<int>(bh - tail);
        p.n_chains = static_cast<int>(tail);
        // the few-chain rule of pick_split applied to the tail alone
        if (tail * 4 <= sms) e = kda::launch_k2n(p, tail * 16 <= sms ? 16 : tail * 8 <= sms ? 8 : 4, 1, false, st);
        else e = kda::launch_k2m(p, 2, false, st);
      }
    } else {
      e = kda::launch_k2t(p, n_records, st);
    }
  } else {
    e = (variant == 3) ? kda::launch_k2m(p, vsplit, state_only, st)
        : (variant == 5) ? kda::launch_k2la(p, vsplit, state_only, st)
                         : kda::launch_k2n(p, vsplit, 1, state_only, st);
  }
  if (e != cudaSuccess) return fail(KDA_ERR_CUDA, "kda: K2 launch failed: %s", cudaGetErrorString(e));
  ++g_launches;
  return KDA_OK;
}

}  // namespace

namespace kda {
// lets the other translation units of the library report through kda_last_error()
void set_last_error(const char* msg) { snprintf(g_err, sizeof(g_err), "%s", msg); }
}  // namespace kda

extern "C" {

size_t kda_fwd_workspace_bytes(int32_t B, int32_t T, int32_t H) {
  if (B <= 0 || T <= 0 || H <= 0) return 0;
  const size_t nt = (static_cast<size_t>(T) + kda::BT - 1) / kda::BT;
  return kda::WS_HEADER_BYTES + static_cast<size_t>(B) * H * nt * kda::REC_BYTES;
}

int kda_fwd(const KdaFwdArgs* a, void* stream) {
  g_launches = 0;
  if (int rc = check_k1(a)) return rc;
  if (int rc = check_k2(a, false)) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(a->workspace, 0, kda::WS_HEADER_BYTES, st);
  if (e != cudaSuccess) return fail(KDA_ERR_CUDA, "kda: status clear failed: %s", cudaGetErrorString(e));
  if (int rc = do_k1(a, st)) return rc;
  return do_k2(a, false, 0, st);
}

int kda_fwd_k1(const KdaFwdArgs* a, void* stream) {
  g_launches = 0;
  if (int rc = check_k1(a)) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(a->workspace, 0, kda::WS_HEADER_BYTES, st);
  if (e != cudaSuccess) return fail(KDA_ERR_CUDA, "kda: status clear failed: %s", cudaGetErrorString(e));
  return do_k1(a, st);
}

int kda_fwd_k2(const KdaFwdArgs* a, void* stream) {
  g_launches = 0;
  if (int rc = check_k2(a, false)) return rc;
  return do_k2(a, false, 0, static_cast<cudaStream_t>(stream));
}

int kda_fwd_k2_state(const KdaFwdArgs* a, int zero_u, void* stream) {
  g_launches = 0;
  if (int rc = check_k2(a, true)) return rc;
  if (a->ht == nullptr) return fail(KDA_ERR_INVALID_ARG, "kda: the state-only pass needs ht%s", "");
  if (zero_u < 0 || zero_u > 2) return fail(KDA_ERR_INVALID_ARG, "kda: zero_u must be 0, 1 or 2%s (got %lld)", "", zero_u);
  return do_k2(a, true, zero_u, static_cast<cudaStream_t>(stream));
}

int kda_recurrent_fwd(const KdaFwdArgs* a, void* stream) {
  g_launches = 0;
  if (a == nullptr) return fail(KDA_ERR_INVALID_ARG, "kda: args is NULL%s", "");
  if (a->B <= 0 || a->T <= 0 || a->H <= 0)
    return fail(KDA_ERR_INVALID_ARG, "kda: B, T, H must be positive%s (T=%lld, H=%lld)", "", a->T, a->H);
  if (a->n_seqs != 0) return fail(KDA_ERR_INVALID_ARG, "kda: the recurrent step takes a fixed-length batch%s (n_seqs must be 0)", "");
  if (a->Hq < 0 || (a->Hq > 0 && a->H % a->Hq != 0))
    return fail(KDA_ERR_INVALID_ARG, "kda: H%s (%lld) must be a multiple of Hq (%lld)", "", a->H, a->Hq);
  if (!a->q || !a->k || !a->v || !a->g || !a->beta || !a->o || !a->A_log)
    return fail(KDA_ERR_INVALID_ARG, "kda: the recurrent step needs q, k, v, g, beta, A_log and o%s", "");
  const uint32_t all = KDA_FLAG_GATE_IN_KERNEL | KDA_FLAG_QK_L2NORM | KDA_FLAG_BETA_SIGMOID;
  if ((a->flags & all) != all)
    return fail(KDA_ERR_INVALID_ARG, "kda: the recurrent step computes gate, l2-norm and beta sigmoid in the kernel%s; set all three flags", "");
  if (a->g_dtype != KDA_G_FP32 && a->g_dtype != KDA_G_BF16)
    return fail(KDA_ERR_INVALID_ARG, "kda: g_dtype must be KDA_G_FP32 or KDA_G_BF16%s (got %lld)", "", a->g_dtype);
  if (!(a->lower_bound > -11.0f && a->lower_bound < 0.0f))
    return fail(KDA_ERR_INVALID_ARG, "kda: lower_bound must be in (-11, 0)%s", "");
  if (!row_aligned(a->q, a->q_stride, 2) || !row_aligned(a->k, a->k_stride, 2) || !row_aligned(a->v, a->v_stride, 2) ||
      !row_aligned(a->g, a->g_stride, a->g_dtype == KDA_G_BF16 ? 2 : 4) || !row_aligned(a->o, a->o_stride, 2))
    return fail(KDA_ERR_INVALID_ARG, "kda: q/k/v/g/o rows must start on 16-byte boundaries%s", "");
  for (const void* ptr : {static_cast<const void*>(a->h0), static_cast<const void*>(a->ht), static_cast<const void*>(a->dt_bias)})
    if (ptr != nullptr && reinterpret_cast<uintptr_t>(ptr) % 16 != 0)
      return fail(KDA_ERR_INVALID_ARG, "kda: h0, ht and dt_bias must be 16-byte aligned%s", "");
  kda::RecurrentParams p;
  memset(&p, 0, sizeof(p));
  p.q = static_cast<const __nv_bfloat16*>(a->q);
  p.k = static_cast<const __nv_bfloat16*>(a->k);
  p.v = static_cast<const __nv_bfloat16*>(a->v);
  p.g = a->g; p.beta = a->beta; p.A_log = a->A_log; p.dt_bias = a->dt_bias;
  p.h0 = a->h0; p.ht = a->ht; p.o = static_cast<__nv_bfloat16*>(a->o);
  p.B = a->B; p.T = a->T; p.H = a->H;
  p.group = a->Hq > 0 ? a->H / a->Hq : 1;
  p.k_first = (a->flags & KDA_FLAG_STATE_K_FIRST) ? 1 : 0;
  for (int i = 0; i < 3; ++i) {
    p.q_s[i] = a->q_stride[i]; p.k_s[i] = a->k_stride[i]; p.v_s[i] = a->v_stride[i];
    p.g_s[i] = a->g_stride[i]; p.beta_s[i] = a->beta_stride[i]; p.o_s[i] = a->o_stride[i];
  }
  p.scale = a->scale;
  p.lower_bound = a->lower_bound;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaError_t e = kda::launch_recurrent(p, a->g_dtype == KDA_G_BF16, sms, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(KDA_ERR_CUDA, "kda: recurrent launch failed: %s", cudaGetErrorString(e));
  ++g_launches;
  return KDA_OK;
}

static_assert(KDA_MAX_PEERS == kda::MAX_PEERS, "header and kernel limits differ");
static_assert(sizeof(KdaPeerPushArgs) == 296 && offsetof(KdaPeerPushArgs, epoch) == 292 && sizeof(KdaFoldPeerArgs) == 296 &&
                  offsetof(KdaFoldPeerArgs, counter) == 288,
              "the ctypes mirrors of these structures pin their layout");

static int fold_impl(const KdaFoldArgs* f, const KdaFoldPeerArgs* peer, void* stream) {
  g_launches = 0;
  if (f == nullptr) return fail(KDA_ERR_INVALID_ARG, "kda: fold args is NULL%s", "");
  if (f->mq == nullptr || (peer == nullptr && f->s_in == nullptr && f->final_out == nullptr))
    return fail(KDA_ERR_INVALID_ARG, "kda: the fold needs mq and at least one of s_in / final_out%s", "");
  if (peer != nullptr) {
    if (peer->n_wait < 0 || peer->n_wait > KDA_MAX_PEERS || peer->n_signal < 0 || peer->n_signal > KDA_MAX_PEERS ||
        f->n_seg > KDA_MAX_PEERS)
      return fail(KDA_ERR_INVALID_ARG, "kda: the peer fold takes at most %s16 segments, flags and signals", "");
    if ((peer->n_wait > 0 && peer->wait_flags == nullptr) || (peer->n_signal > 0 && peer->counter == nullptr) || peer->epoch <= 0)
      return fail(KDA_ERR_INVALID_ARG, "kda: the peer fold needs wait_flags, counter and a positive epoch%s", "");
    for (int i = 0; i <= f->n_seg && i <= KDA_MAX_PEERS; ++i)
      if (peer->s_in_seg[i] != nullptr && reinterpret_cast<uintptr_t>(peer->s_in_seg[i]) % 16 != 0)
        return fail(KDA_ERR_INVALID_ARG, "kda: s_in_seg entries must be 16-byte aligned%s", "");
    for (int i = 0; i < peer->n_signal; ++i)
      if (peer->signal[i] == nullptr) return fail(KDA_ERR_INVALID_ARG, "kda: signal[%s%lld] is NULL", "", i);
  }
  if (f->n_chains <= 0 || f->n_seg < 0)
    return fail(KDA_ERR_INVALID_ARG, "kda: the fold needs n_chains > 0 and n_seg >= 0%s (got %lld, %lld)", "", f->n_chains, f->n_seg);
  const int64_t state = static_cast<int64_t>(kda::D) * kda::D;
  const int64_t span = f->use_q ? 2 * state : state;   // without Q only the M block has to lie inside a stride
  if (f->n_seg > 0 && ((f->n_chains > 1 && f->chain_stride < span) || (f->n_seg > 1 && f->seg_stride < span)))
    return fail(KDA_ERR_INVALID_ARG, "kda: the fold's strides must span the 128 x 128 blocks they step over%s", "");
  if (f->seg_stride % 4 != 0 || f->chain_stride % 4 != 0)
    return fail(KDA_ERR_INVALID_ARG, "kda: the fold's strides must be multiples of 4 floats%s (every M_j is copied 16 bytes at a time)", "");
  const int64_t h0_stride = f->h0_stride != 0 ? f->h0_stride : state;
  const int64_t final_stride = f->final_stride != 0 ? f->final_stride : state;
  if (h0_stride < state || final_stride < state)
    return fail(KDA_ERR_INVALID_ARG, "kda: h0_stride and final_stride must be 0 (dense) or at least 128 x 128%s", "");
  if (f->status != nullptr && reinterpret_cast<uintptr_t>(f->status) % 4 != 0)
    return fail(KDA_ERR_INVALID_ARG, "kda: status must be 4-byte aligned%s", "");
  for (const void* ptr : {static_cast<const void*>(f->mq), static_cast<const void*>(f->h0), static_cast<const void*>(f->s_in),
                          static_cast<const void*>(f->final_out)})
    if (ptr != nullptr && reinterpret_cast<uintptr_t>(ptr) % 16 != 0)
      return fail(KDA_ERR_INVALID_ARG, "kda: mq, h0, s_in and final_out must be 16-byte aligned%s", "");
  if (static_cast<long long>(f->n_chains) * (kda::D / 4) > 0x7fffffffLL)
    return fail(KDA_ERR_INVALID_ARG, "kda: too many chains for one fold launch%s", "");
  kda::FoldParams p;
  memset(&p, 0, sizeof(p));
  p.mq = f->mq; p.seg_stride = f->seg_stride; p.chain_stride = f->chain_stride;
  p.h0 = f->h0; p.h0_stride = h0_stride;
  p.s_in = f->s_in; p.final_out = f->final_out; p.final_stride = final_stride;
  p.n_chains = f->n_chains; p.n_seg = f->n_seg; p.use_q = f->use_q ? 1 : 0;
  p.status = f->status;
  if (peer != nullptr) {
    p.s_in = nullptr;
    p.wait_flags = peer->wait_flags; p.n_wait = peer->n_wait; p.epoch = peer->epoch;
    p.s_in_seg_on = 1;
    for (int i = 0; i <= f->n_seg; ++i) p.s_in_seg[i] = peer->s_in_seg[i];
    p.n_signal = peer->n_signal;
    for (int i = 0; i < peer->n_signal; ++i) p.signal[i] = peer->signal[i];
    p.counter = peer->counter;
  }
  cudaError_t e = kda::launch_state_fold(p, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(KDA_ERR_CUDA, "kda: fold launch failed: %s", cudaGetErrorString(e));
  ++g_launches;
  return KDA_OK;
}

int kda_state_fold_ex(const KdaFoldArgs* f, void* stream) { return fold_impl(f, nullptr, stream); }

int kda_state_fold_peer(const KdaFoldArgs* f, const KdaFoldPeerArgs* peer, void* stream) {
  if (peer == nullptr) return fail(KDA_ERR_INVALID_ARG, "kda: peer args is NULL%s", "");
  return fold_impl(f, peer, stream);
}

static int check_push_targets(const KdaPeerPushArgs* a) {
  if (a == nullptr) return fail(KDA_ERR_INVALID_ARG, "kda: push args is NULL%s", "");
  if (a->world < 1 || a->world > KDA_MAX_PEERS || a->epoch <= 0)
    return fail(KDA_ERR_INVALID_ARG, "kda: the push needs 1..16 ranks and a positive epoch%s (world %lld)", "", a->world);
  if (a->counter == nullptr || a->slice_floats <= 0 || a->slice_floats % 4 != 0 || a->dst_offset_floats < 0 ||
      a->dst_offset_floats % 4 != 0)
    return fail(KDA_ERR_INVALID_ARG, "kda: the push needs a counter and 16-byte multiples for slice and offset%s", "");
  for (int d = 0; d < a->world; ++d)
    if (a->dst[d] == nullptr || a->flag[d] == nullptr || reinterpret_cast<uintptr_t>(a->dst[d]) % 16 != 0)
      return fail(KDA_ERR_INVALID_ARG, "kda: dst[%s%lld] and its flag must be set, dst 16-byte aligned", "", d);
  return KDA_OK;
}

int kda_fwd_k2_state_push(const KdaFwdArgs* a, const KdaPeerPushArgs* push, void* stream) {
  g_launches = 0;
  if (int rc = check_common(a)) return rc;
  if (int rc = check_k2(a, true)) return rc;
  if (int rc = check_push_targets(push)) return rc;
  return do_k2(a, true, 2, static_cast<cudaStream_t>(stream), push);
}

int kda_fwd_k2_after_flags(const KdaFwdArgs* a, const int32_t* flags, int32_t n, int32_t epoch, void* stream) {
  g_launches = 0;
  if (int rc = check_common(a)) return rc;
  if (int rc = check_k2(a, false)) return rc;
  if (flags == nullptr || n < 1 || n > KDA_MAX_PEERS || epoch <= 0 || a->h0 == nullptr)
    return fail(KDA_ERR_INVALID_ARG, "kda: the call needs h0, 1..16 flags and a positive epoch%s (n %lld)", "", n);
  const H0Flags h0f{flags, n, epoch};
  return do_k2(a, false, 0, static_cast<cudaStream_t>(stream), nullptr, &h0f);
}

int kda_peer_push(const KdaPeerPushArgs* a, void* stream) {
  g_launches = 0;
  if (a == nullptr) return fail(KDA_ERR_INVALID_ARG, "kda: push args is NULL%s", "");
  if (a->world < 1 || a->world > KDA_MAX_PEERS || a->epoch <= 0)
    return fail(KDA_ERR_INVALID_ARG, "kda: the push needs 1..16 ranks and a positive epoch%s (world %lld)", "", a->world);
  if (a->src == nullptr || a->counter == nullptr || a->slice_floats <= 0 || a->slice_floats % 4 != 0 ||
      a->dst_offset_floats < 0 || a->dst_offset_floats % 4 != 0 || reinterpret_cast<uintptr_t>(a->src) % 16 != 0)
    return fail(KDA_ERR_INVALID_ARG, "kda: the push needs src, counter and 16-byte multiples for slice and offset%s", "");
  kda::PeerPushParams p;
  memset(&p, 0, sizeof(p));
  for (int d = 0; d < a->world; ++d) {
    if (a->dst[d] == nullptr || a->flag[d] == nullptr || reinterpret_cast<uintptr_t>(a->dst[d]) % 16 != 0)
      return fail(KDA_ERR_INVALID_ARG, "kda: dst[%s%lld] and its flag must be set, dst 16-byte aligned", "", d);
    p.dst[d] = reinterpret_cast<float4*>(a->dst[d]);
    p.flag[d] = a->flag[d];
  }
  p.src = reinterpret_cast<const float4*>(a->src);
  p.dst_offset = a->dst_offset_floats / 4;
  p.slice = a->slice_floats / 4;
  p.counter = a->counter;
  p.world = a->world; p.epoch = a->epoch;
  cudaError_t e = kda::launch_peer_push(p, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(KDA_ERR_CUDA, "kda: push launch failed: %s", cudaGetErrorString(e));
  ++g_launches;
  return KDA_OK;
}

int kda_peer_enable(int32_t peer_device) {
  int dev = 0, can = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(KDA_ERR_CUDA, "kda: cudaGetDevice failed: %s", cudaGetErrorString(e));
  if (peer_device == dev) return KDA_OK;
  e = cudaDeviceCanAccessPeer(&can, dev, peer_device);
  if (e != cudaSuccess || !can) {
    cudaGetLastError();
    return fail(KDA_ERR_CUDA, "kda: this GPU cannot map the memory of GPU %s%lld", "", peer_device);
  }
  e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();
    e = cudaSuccess;
  }
  if (e != cudaSuccess) return fail(KDA_ERR_CUDA, "kda: enabling peer access failed: %s", cudaGetErrorString(e));
  return KDA_OK;
}

// ---- CUDA IPC for the peer exchange -------------------------------------------------------------
// The importing side opens a handle with ITS OWN device current, which is what maps the exporting
// GPU's memory for kernels of the importing GPU (a mapping made with another device current is
// not reachable from this one).  A handle is opened once per process and stays mapped.
namespace {
struct IpcOpened { cudaIpcMemHandle_t h; int dev; void* base; int refs; };
std::mutex g_ipc_mu;
std::vector<IpcOpened> g_ipc_opened;
}  // namespace

int kda_ipc_export(const void* ptr, void* handle_out, int64_t* offset_out) {
  if (ptr == nullptr || handle_out == nullptr || offset_out == nullptr)
    return fail(KDA_ERR_INVALID_ARG, "kda: ptr, handle_out and offset_out are required%s", "");
  typedef CUresult (*RangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
  static RangeFn range_fn = nullptr;
  if (range_fn == nullptr) {
    void* fp = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fp, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
      return fail(KDA_ERR_CUDA, "kda: cuMemGetAddressRange is not available from this driver%s", "");
    range_fn = reinterpret_cast<RangeFn>(fp);
  }
  CUdeviceptr base = 0;
  size_t size = 0;
  if (range_fn(&base, &size, reinterpret_cast<CUdeviceptr>(ptr)) != CUDA_SUCCESS)
    return fail(KDA_ERR_CUDA, "kda: the pointer does not belong to a device allocation%s", "");
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base));
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(KDA_ERR_CUDA, "kda: cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e));
  }
  memcpy(handle_out, &h, sizeof(h));
  *offset_out = static_cast<int64_t>(reinterpret_cast<CUdeviceptr>(ptr) - base);
  return KDA_OK;
}

int kda_ipc_open(const void* handle, int64_t offset, void** ptr_out) {
  if (handle == nullptr || ptr_out == nullptr || offset < 0)
    return fail(KDA_ERR_INVALID_ARG, "kda: handle and ptr_out are required%s", "");
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(KDA_ERR_CUDA, "kda: cudaGetDevice failed: %s", cudaGetErrorString(e));
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  std::lock_guard<std::mutex> lock(g_ipc_mu);
  for (IpcOpened& o : g_ipc_opened)
    if (o.dev == dev && memcmp(&o.h, &h, sizeof(h)) == 0) {
      ++o.refs;
      *ptr_out = static_cast<char*>(o.base) + offset;
      return KDA_OK;
    }
  void* base = nullptr;
  e = cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(KDA_ERR_CUDA, "kda: cudaIpcOpenMemHandle failed: %s", cudaGetErrorString(e));
  }
  g_ipc_opened.push_back(IpcOpened{h, dev, base, 1});
  *ptr_out = static_cast<char*>(base) + offset;
  return KDA_OK;
}

int kda_ipc_close(const void* handle) {
  if (handle == nullptr) return fail(KDA_ERR_INVALID_ARG, "kda: handle is required%s", "");
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(KDA_ERR_CUDA, "kda: cudaGetDevice failed: %s", cudaGetErrorString(e));
  std::lock_guard<std::mutex> lock(g_ipc_mu);
  for (size_t i = 0; i < g_ipc_opened.size(); ++i) {
    IpcOpened& o = g_ipc_opened[i];
    if (o.dev != dev || memcmp(&o.h, handle, sizeof(o.h)) != 0) continue;
    if (--o.refs > 0) return KDA_OK;
    e = cudaIpcCloseMemHandle(o.base);
    g_ipc_opened.erase(g_ipc_opened.begin() + static_cast<long>(i));
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fail(KDA_ERR_CUDA, "kda: cudaIpcCloseMemHandle failed: %s", cudaGetErrorString(e));
    }
    return KDA_OK;
  }
  return fail(KDA_ERR_INVALID_ARG, "kda: this handle is not open on the current device%s", "");
}

int kda_flag_wait(const int32_t* flags, int32_t n, int32_t epoch, int32_t* status, void* stream) {
  g_launches = 0;
  if (flags == nullptr || n < 1 || n > 32 || epoch <= 0)
    return fail(KDA_ERR_INVALID_ARG, "kda: the flag wait needs 1..32 flags and a positive epoch%s (n %lld)", "", n);
  cudaError_t e = kda::launch_flag_wait(flags, n, epoch, status, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(KDA_ERR_CUDA, "kda: flag wait launch failed: %s", cudaGetErrorString(e));
  ++g_launches;
  return KDA_OK;
}

int kda_state_fold(const float* mq, int64_t seg_stride, int64_t chain_stride, const float* h0, float* s_in,
                   int32_t n_chains, int32_t n_seg, int32_t* status, void* stream) {
  if (s_in == nullptr) return fail(KDA_ERR_INVALID_ARG, "kda: the fold needs mq and s_in%s", "");
  KdaFoldArgs f;
  memset(&f, 0, sizeof(f));
  f.mq = mq; f.seg_stride = seg_stride; f.chain_stride = chain_stride; f.h0 = h0; f.s_in = s_in;
  f.n_chains = n_chains; f.n_seg = n_seg; f.use_q = 1; f.status = status;
  return kda_state_fold_ex(&f, stream);
}

int kda_varlen_fill_tables(const int32_t* cu, int32_t n_seqs, int32_t H, int32_t* chunk_table, int32_t* seq_table) {
  if (cu == nullptr || n_seqs <= 0 || H <= 0)
    return fail(KDA_ERR_INVALID_ARG, "kda: cu_seqlens, n_seqs and H are required%s", "");
  if (cu[0] != 0) return fail(KDA_ERR_INVALID_ARG, "kda: cu_seqlens must start at 0%s (got %lld)", "", cu[0]);
  long long chunks = 0;
  for (int i = 0; i < n_seqs; ++i) {
    const long long len = static_cast<long long>(cu[i + 1]) - cu[i];
    if (len <= 0) return fail(KDA_ERR_INVALID_ARG, "kda: sequence %s%lld is empty or cu_seqlens decreases", "", i);
    const long long nt = (len + kda::BT - 1) / kda::BT;
    if ((chunks + nt) * H > 0x7fffffffLL) return fail(KDA_ERR_INVALID_ARG, "kda: too many chunk records%s", "");
    if (chunk_table != nullptr && seq_table != nullptr) {
      seq_table[4 * i + 0] = cu[i];
      seq_table[4 * i + 1] = static_cast<int32_t>(nt);
      seq_table[4 * i + 2] = static_cast<int32_t>(chunks * H);
      seq_table[4 * i + 3] = static_cast<int32_t>(len);
      for (long long n = 0; n < nt; ++n) {
        int32_t* e = chunk_table + 4 * (chunks + n);
        e[0] = cu[i] + static_cast<int32_t>(n * kda::BT);
        e[1] = static_cast<int32_t>(len - n * kda::BT < kda::BT ? len - n * kda::BT : kda::BT);
        e[2] = static_cast<int32_t>(chunks * H + n);
        e[3] = static_cast<int32_t>(nt);
      }
    }
    chunks += nt;
  }
  return static_cast<int>(chunks);
}

int kda_fwd_status(const void* workspace, void* stream, int32_t* status_out) {
  if (workspace == nullptr || status_out == nullptr)
    return fail(KDA_ERR_INVALID_ARG, "kda: workspace and status_out are required%s", "");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int32_t v = 0;
  cudaError_t e = cudaMemcpyAsync(&v, workspace, sizeof(v), cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return fail(KDA_ERR_CUDA, "kda: status read failed: %s", cudaGetErrorString(e));
  *status_out = v;
  if (v != 0) return fail(KDA_ERR_DEVICE_STATUS, "kda: a bounded device-side wait gave up%s (status %lld)", "", v);
  return KDA_OK;
}

int kda_fwd_k2_choice(const KdaFwdArgs* args, int state_only, int sm_count, int32_t* variant_out, int32_t* vsplit_out) {
  if (args == nullptr || variant_out == nullptr || vsplit_out == nullptr)
    return fail(KDA_ERR_INVALID_ARG, "kda: null pointer%s", "");
  if (args->k2_variant < 0 || args->k2_variant > 5 || args->k2_variant == 2)
    return fail(KDA_ERR_INVALID_ARG, "kda: k2_variant%s %lld is not one of 0, 1, 3, 4, 5", "", static_cast<long long>(args->k2_variant));
  int vs = 0, var = 0;
  pick_split(args, state_only != 0, &vs, &var, sm_count);
  *variant_out = var;
  *vsplit_out = (var == 4) ? 1 : vs;   // the tensor-memory form runs one CTA per chain
  return KDA_OK;
}

int kda_last_launch_count(void) { return g_launches; }

const char* kda_last_error(void) { return g_err; }

const char* kda_version(void) { return "0.1 sm_100a"; }

}  // extern "C"
