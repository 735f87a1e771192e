// Internal launch interface between the C-ABI layer and the two kernels.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace kda {

// division by a runtime constant as multiply-high + shift (n < 2^31): q = n / d
struct FastDiv {
  uint32_t mul, shr, d;
  __host__ void set(uint32_t div) {
    d = div;
    if (div <= 1) { mul = 0; shr = 0; return; }
    uint32_t lg = 0;
    while ((1u << lg) < div) ++lg;                       // ceil(log2(d))
    const unsigned p = 31 + lg;
    mul = static_cast<uint32_t>(((1ull << p) + div - 1) / div);
    shr = p - 32;
  }
  __device__ __forceinline__ uint32_t div(uint32_t n) const { return d <= 1 ? n : (__umulhi(n, mul) >> shr); }
};

struct K1Params {
  // tiled TMA descriptors of q, k, v, g viewed as 4-D tensors (d, head, token, batch) with the
  // caller's strides; one 16-token x 128 box per (tensor, chunk).  Rows past T read as zero.
  CUtensorMap tm_q, tm_k, tm_v, tm_g;
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  const void* g;
  const float* beta;
  const float* A_log;
  const float* dt_bias;
  uint8_t* rec;      // first chunk record (workspace + header)
  int* status;       // device status word
  float* g_out;      // optional
  float* ainv_out;   // optional
  int B, T, H, NT;
  FastDiv div_h, div_nt;   // item index -> (batch, chunk, head) without integer division
  int64_t q_s[3], k_s[3], v_s[3], g_s[3], beta_s[3];  // element strides (batch, token, head)
  float scale, lower_bound;
  uint32_t flags;
  // packed variable-length input: one entry per chunk (first token, valid tokens, first record,
  // chunks of its sequence), B == 1; null for a fixed-length batch
  const int4* chunk_table;
  int n_chunks;
  // grouped value heads: q and k have Hq heads, head h of everything else reads q/k head h / (H/Hq)
  int Hq;
  FastDiv div_g;   // divides by H / Hq
};

constexpr int MAX_PEERS = 16;   // = KDA_MAX_PEERS of the public header

struct K2Params {
  const uint8_t* rec;
  const float* h0;   // [B,H,128,128] or null
  __nv_bfloat16* o;  // may be null in state-only mode
  float* ht;         // may be null
  int* status;
  int B, T, H, NT;
  int64_t o_s[3];
  float scale;
  int k_first;       // h0 and ht are [B,H,K,V] (element (v, k) at k*128 + v) instead of [B,H,V,K]
  int zero_u;        // state-only mode: drop the u term
  // state-only "transform pair" mode of the m16 form: the launch runs 2 x chains; chain 2c starts from
  // the identity with u dropped (M of the segment), chain 2c+1 from zero with u (Q); h0 is not read
  // and ht is [chains][2][128][128]
  int pair_mode;
  // packed variable-length input: one entry per sequence (first token, chunks, first record,
  // length); the grid then runs over (sequence, head); null for a fixed-length batch
  const int4* seq_table;
  int n_seqs;
  // a launch may cover a sub-range of the (batch, head) chains: first chain and count (0 = all)
  int chain0, n_chains;
  // Transform-pair pass of a sequence split over peer memory (the 8-row pair form only): the (M, Q) tiles
  // of chain c go straight into the receive buffer of the rank that owns the chain,
  // push_dst[c / push_hp] + push_dst_offset + (c % push_hp) * 2 * 128 * 128, instead of ht, and the CTA that
  // completes a destination raises its flag (as kda_peer_push_kernel does).
  int push_on, push_hp, push_epoch, push_ctas_per_dst;
  long long push_dst_offset;
  float* push_dst[MAX_PEERS];
  int* push_flag[MAX_PEERS];
  int* push_counter;
  // Final pass of a sequence split over peer memory (the 8-row and 16-row forms): h0 is stored by other
  // GPUs; the consumer warps read it once the h0_n_flags local flags have reached h0_epoch (bounded wait,
  // status code 7), while the producer warp already streams the first records in.
  const int* h0_flags;
  int h0_n_flags, h0_epoch;
};

cudaError_t launch_k1(const K1Params& p, bool g_bf16, bool fast_exp, cudaStream_t stream);
// Fills the four tensor maps of p from its pointers, sizes and strides (host, no device work).
cudaError_t k1_encode_tensor_maps(K1Params& p, bool g_bf16, const char** what);
// Two organisations of K2 (same arithmetic, bit-identical results within one organisation):
//   "n8":       state rows on the MMA N dimension, ntile = 1 tile of 8 rows per warp,
//               16 / vsplit in {1, 2, 4} consumer warps per CTA                 (kda_k2_sm100.cu)
//   "m16":      state rows on the MMA M dimension, 16 rows per warp,
//               8 / vsplit in {1, 2, 4} consumer warps per CTA                 (kda_k2m_sm100.cu)
// vsplit = CTAs per (batch, head).
cudaError_t launch_k2n(const K2Params& p, int vsplit, int ntile, bool state_only, cudaStream_t stream);
cudaError_t launch_k2m(const K2Params& p, int vsplit, bool state_only, cudaStream_t stream);
//   "n8 look-ahead": the 8-row form with the products of chunk n+1 taken from the decayed state of
//               step n plus a 16x16 cross-Gram correction, so that a step has no dependent hand-over;
//               16 / vsplit in {1, 2, 4} consumer warps per CTA; measured slower than "n8", never
//               chosen automatically                                           (kda_k2la_sm100.cu)
cudaError_t launch_k2la(const K2Params& p, int vsplit, bool state_only, cudaStream_t stream);
// the transform-pair pass of the sequence split in the "n8" form: both recurrences (M: identity entry
// state without u; Q: zero entry state with u) on the same eight rows of one warp, so every operand
// fragment read from shared memory feeds two MMAs; ht is [chains][2][128][128]
cudaError_t launch_k2n_pair(const K2Params& p, int vsplit, cudaStream_t stream);
//   "tc":       the whole 128-row state of a head in tensor memory, tcgen05 MMAs, one CTA per
//               (batch, head), two CTAs per SM; outputs + final state only              (kda_k2t_sm100.cu)
cudaError_t launch_k2t(const K2Params& p, long long n_records, cudaStream_t stream);

// Walk of the per-segment affine state transforms of a sequence split (kda_fold_sm100.cu).
struct FoldParams {
  const float* mq;             // M_j[c] at mq + j*seg_stride + c*chain_stride (floats), Q_j[c] 128*128 floats behind it
  long long seg_stride, chain_stride;
  const float* h0;             // entry state of chain c at h0 + c*h0_stride, or null (zeros)
  long long h0_stride;
  float* s_in;                 // [n_seg + 1][n_chains][128][128] or null: the state before every segment and after the last
  float* final_out;            // or null: the state after the last segment of chain c at final_out + c*final_stride
  long long final_stride;
  int n_chains, n_seg;
  int use_q;                   // 0: the walk is S <- S * M_j (composition of transition matrices)
  int* status;
  // Exchange over peer memory (all zero for the plain fold).  The walk starts once the n_wait local
  // flags have reached `epoch` (peers have stored the transforms into mq); the state before segment j
  // goes to s_in_seg[j] + chain * 128 * 128 (a peer's buffer; a null entry is skipped) instead of s_in;
  // after the last CTA has finished, *signal[i] = epoch for i < n_signal (system scope).
  const int* wait_flags;
  int n_wait, epoch;
  int s_in_seg_on;
  float* s_in_seg[MAX_PEERS + 1];
  int* signal[MAX_PEERS];
  int n_signal;
  int* counter;                // local int, zero between launches
};
cudaError_t launch_state_fold(const FoldParams& p, cudaStream_t stream);

// Peer-memory pieces of the sequence split's exchange (kda_peer_sm100.cu).
struct PeerPushParams {
  const float4* src;           // [world][slice] 16-byte units: slice d goes to rank d
  float4* dst[MAX_PEERS];  // rank d's receive buffer (peer-mapped; the own one for d = rank)
  long long dst_offset;        // 16-byte units into dst[d]: this rank's slot
  long long slice;             // 16-byte units per destination
  int* flag[MAX_PEERS];    // raised to `epoch` on rank d once the slice has been stored
  int* counter;                // local int[world], zero between launches
  int world, epoch;
  int ctas_per_dst;            // set by the launcher
};
cudaError_t launch_peer_push(const PeerPushParams& p, cudaStream_t stream);
cudaError_t launch_flag_wait(const int* flags, int n, int epoch, int* status, cudaStream_t stream);

// Token recurrence (decode / short sequences): no chunking, no workspace (kda_recurrent_sm100.cu).
struct RecurrentParams {
  const __nv_bfloat16 *q, *k, *v;
  const void* g;            // raw gate, bf16 or fp32
  const float *beta, *A_log, *dt_bias;   // dt_bias may be null
  const float* h0;          // [B,H,128,128] or null; may alias ht (each CTA reads its rows before it writes them)
  float* ht;                // may be null
  __nv_bfloat16* o;
  int B, T, H;
  int group;                // value heads per q/k head (1 = plain multi-head)
  int k_first;              // h0 / ht are [B,H,K,V] instead of [B,H,V,K]
  int64_t q_s[3], k_s[3], v_s[3], g_s[3], beta_s[3], o_s[3];
  float scale, lower_bound;
};
cudaError_t launch_recurrent(const RecurrentParams& p, bool g_bf16, int sms, cudaStream_t stream);

}  // namespace kda
