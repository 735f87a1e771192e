/* C ABI of libkda_b200.so -- the KDA (Kimi Delta Attention) chunked forward, chunk
 * size 16, K = V = 128, hand-written CUDA for sm_100a (B200).
 *
 * The library is the drop-in for the device side of the reference project's
 * forward path.  Reference interfaces each entry point replaces (paths inside
 * the reference project):
 *
 *   kda_fwd            <- the two Triton launches of `_run`
 *                         (src/kda_bt16/kernels.py:581-602) and the Ascend stage
 *                         sequence of `_kda_fwd_impl`
 *                         (python/kda_ascendc_v1/api.py:890-1191), which reach the
 *                         device through `launch_argsarray_engine`
 *                         (aclab/launcher/launcher.cpp:271-294).
 *   kda_fwd_k1         <- `kda_bt16_kernel_k1` (src/kda_bt16/kernels.py:53-184)
 *   kda_fwd_k2         <- `kda_bt16_kernel_k2` (src/kda_bt16/kernels.py:187-302)
 *   kda_fwd_workspace_bytes
 *                      <- the per-call `torch.empty` intermediates of `_run`
 *                         (src/kda_bt16/kernels.py:572-579)
 *   kda_last_error     <- the launcher's exception text
 *                         (aclab/launcher/launcher.cpp:35-39)
 *
 * Conventions: the library never calls an allocation routine; the caller owns every
 * buffer and passes raw device pointers (NULL = tensor absent).  What the library holds by
 * itself: a thread-local error string and tensor-map cache, per-device one-time kernel
 * attribute set-up, and the fixed KDA_STATIC_SCRATCH_BYTES device array (with its cached
 * address per device) behind kda_fwd_static_scratch.  All launches are
 * asynchronous on the given stream (a cudaStream_t passed as void*), exactly as
 * the reference launches on the caller's current stream.  Functions return 0 on
 * success and a negative KDA_ERR_* code otherwise; kda_last_error() returns the
 * thread-local message of the last failure.
 */
#ifndef KDA_B200_H_
#define KDA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KDA_OK 0
#define KDA_ERR_INVALID_ARG (-1)
#define KDA_ERR_CUDA (-2)
#define KDA_ERR_DEVICE_STATUS (-3)
#define KDA_ERR_UNSUPPORTED (-4)   /* the call is valid but this entry point has no kernel for it */

#define KDA_G_FP32 0
#define KDA_G_BF16 1

/* flags (all three set = the reference's production bucket) */
#define KDA_FLAG_GATE_IN_KERNEL 1u    /* g is the raw gate; apply A_log/dt_bias/sigmoid/cumsum */
#define KDA_FLAG_QK_L2NORM 2u         /* l2-normalise q and k (eps 1e-6) */
#define KDA_FLAG_BETA_SIGMOID 4u      /* beta holds logits */
#define KDA_FLAG_STATE_K_FIRST 8u     /* h0 / ht are [B, H, K, V] (the reference's state_v_first=False,
                                         src/kda_bt16/kernels.py:497-510, where it is a host-side transpose);
                                         read and written in that layout by kda_fwd, kda_fwd_k2,
                                         kda_fwd_k2_state(zero_u 0 / 1) and kda_recurrent_fwd; the transform
                                         pair (zero_u = 2) keeps [B, H, V, K] */

typedef struct KdaFwdArgs {
  /* inputs: [B, T, H, 128], innermost dimension contiguous; strides in ELEMENTS.
   * A head-shard or sequence-segment view of a larger tensor is passed by strides,
   * without a copy.  Every row start must be 16-byte aligned. */
  const void* q;        /* bf16 */
  const void* k;        /* bf16 */
  const void* v;        /* bf16 */
  const void* g;        /* raw gate (or, without KDA_FLAG_GATE_IN_KERNEL, the chunk-local
                           log2 cumsum); fp32 or bf16 per g_dtype */
  const float* beta;    /* [B, T, H] fp32 */
  const float* A_log;   /* [H] fp32; required with KDA_FLAG_GATE_IN_KERNEL */
  const float* dt_bias; /* [H*128] fp32 or NULL */
  const float* h0;      /* initial state [B, H, V=128, K=128] fp32 contiguous, or NULL (zeros) */
  void* o;              /* out: bf16 [B, T, H, 128] */
  float* ht;            /* out: final state [B, H, 128, 128] fp32 contiguous, or NULL */
  void* workspace;      /* kda_fwd_workspace_bytes(B, T, H) bytes, 256-byte aligned */
  float* g_out;         /* optional debug out: log2 cumsum, fp32 [B, T, H, 128] contiguous */
  float* ainv_out;      /* optional debug out: (I+Akk)^-1, fp32 [B, T, H, 16] contiguous */
  int32_t B, T, H;
  int32_t g_dtype;      /* KDA_G_FP32 / KDA_G_BF16 */
  int64_t q_stride[3];  /* batch, token, head strides of q (elements) */
  int64_t k_stride[3];
  int64_t v_stride[3];
  int64_t g_stride[3];
  int64_t o_stride[3];
  int64_t beta_stride[3];
  float scale;
  float lower_bound;
  uint32_t flags;
  int32_t k2_vsplit;    /* 0 = choose; else CTAs per (batch, head) that share the rows of its state */
  int32_t k2_variant;   /* 0 = choose; how K2 maps state rows to warps:
                           1 "n8":  8 rows per warp  (k2_vsplit 4, 8 or 16), rows on the MMA N dimension
                           3 "m16": 16 rows per warp (k2_vsplit 2, 4 or 8), rows on the MMA M dimension
                           4 "tc":  all 128 rows of a head in tensor memory, tcgen05 MMAs (k2_vsplit ignored;
                                    not for kda_fwd_k2_state)
                           5 "la":  the 8-row form with a one-chunk look-ahead (no dependent hand-over inside
                                    a step; k2_vsplit 4, 8 or 16); measured slower than "n8" and never chosen
                                    automatically */
  /* Packed variable-length sequences (optional; not in the reference, whose README.md:509 lists
   * it as future work).  n_seqs > 0 selects it: B must be 1, T is the total number of packed
   * tokens, h0 / ht are [n_seqs, H, 128, 128], and the two tables (DEVICE memory, int32, made by
   * kda_varlen_fill_tables) say where every sequence and every 16-token chunk lies.  The workspace
   * then holds one record per (chunk, head): kda_fwd_workspace_bytes(1, 16 * n_chunks, H). */
  int32_t n_seqs;
  const int32_t* chunk_table;  /* [n_chunks][4]: first token, valid tokens, first record, chunks of its sequence */
  const int32_t* seq_table;    /* [n_seqs][4]:   first token, chunks, first record, length */
  int32_t n_chunks;
  /* Grouped value heads (optional; the reference's kernels carry the index arithmetic,
   * src/kda_bt16/kernels.py:88, but its API rejects HV != H, :729-730): q and k have Hq heads,
   * everything else (v, g, beta, A_log, dt_bias, o, states, records) has H heads, H a multiple
   * of Hq, value head h reads q/k head h / (H / Hq).  0 = Hq equals H. */
  int32_t Hq;
} KdaFwdArgs;

/* Bytes of K1 -> K2 scratch for a (B, T, H) problem: a 256-byte status block
 * followed by one 26,112-byte record per (batch, head, chunk). */
size_t kda_fwd_workspace_bytes(int32_t B, int32_t T, int32_t H);

/* Whole forward: clears the status block, launches K1 then K2 on `stream`. */
int kda_fwd(const KdaFwdArgs* args, void* stream);

/* Stage launches (per-stage timing / profiling, and the sequence-parallel path,
 * which runs K2 more than once on the records of one K1 pass). */
int kda_fwd_k1(const KdaFwdArgs* args, void* stream);
int kda_fwd_k2(const KdaFwdArgs* args, void* stream);

/* State-only K2 pass for the sequence-parallel split: walks the records and
 * returns only the final state.  zero_u = 0: the ordinary recurrence from h0.  zero_u = 1: the u
 * term is dropped, so that feeding h0 = I yields the segment's transition matrix.  zero_u = 2:
 * both transforms of the segment in ONE launch -- h0 is not read, ht is
 * [B*H][2][128][128]: for every (batch, head) the transition matrix M (identity entry state, u
 * dropped) followed by the offset Q (zero entry state), the layout kda_state_fold reads. */
int kda_fwd_k2_state(const KdaFwdArgs* args, int zero_u, void* stream);

/* Exchange step of the sequence split: walks the affine transforms S_out = S_in * M_j + Q_j of the
 * n_seg segments of each of n_chains (batch, head) chains, in fp32:
 *   S = h0[c] (zeros when h0 is NULL);  for j = 0..n_seg-1: s_in[j][c] = S;  S = S * M_j[c] + Q_j[c];
 *   s_in[n_seg][c] = S
 * mq: M_j[c] = 128 x 128 floats at mq + j * seg_stride + c * chain_stride, Q_j[c] directly behind it
 * (strides in floats, so the buffer of an all-gather or of an all-to-all is read in place);
 * s_in: [n_seg + 1][n_chains][128][128] fp32 contiguous; h0: [n_chains][128][128] or NULL.
 * M_j is what kda_fwd_k2_state(zero_u = 1) returns from an identity entry state, Q_j what
 * kda_fwd_k2_state(zero_u = 0) returns from a zero one (zero_u = 2 returns both in this layout).
 * status: device word (NULL = none) that receives a non-zero code if a bounded wait inside the
 * kernel gives up -- pass the start of a workspace and read it with kda_fwd_status.  No reference
 * kernel: the reference only analyses the route (tools/probe_segment_affine.py:100-125,
 * docs/SEGMENT_SCAN_ROUTE_A_EVAL.md:92-118). */
int kda_state_fold(const float* mq, int64_t seg_stride, int64_t chain_stride, const float* h0, float* s_in,
                   int32_t n_chains, int32_t n_seg, int32_t* status, void* stream);

/* The same walk with every layout choice exposed (what the two-level sequence split uses: a rank
 * first composes the transforms of its own sub-segments, then walks its sub-segments from the entry
 * state the exchange returns).  h0_stride / final_stride: floats between the states of consecutive
 * chains, 0 = dense (128 x 128).  s_in and final_out are both optional (at least one): final_out
 * receives only the state after the last segment, with its own chain stride, so that it can be
 * written straight into an (M, Q) buffer.  use_q = 0 drops the offsets: S <- S * M_j, which with
 * h0 = M_0 composes transition matrices (M_0 M_1 ... ); use_q = 1 with h0 = Q_0 over segments 1..
 * composes the offsets (((Q_0 M_1 + Q_1) M_2 + Q_2) ...).  No reference counterpart. */
typedef struct KdaFoldArgs {
  const float* mq;        /* M_j[c] at mq + j * seg_stride + c * chain_stride; Q_j[c] 128 x 128 floats behind it */
  int64_t seg_stride, chain_stride;
  const float* h0;        /* or NULL (zeros) */
  int64_t h0_stride;
  float* s_in;            /* [n_seg + 1][n_chains][128][128] contiguous, or NULL */
  float* final_out;       /* or NULL */
  int64_t final_stride;
  int32_t n_chains, n_seg;
  int32_t use_q;
  int32_t* status;        /* device word, or NULL */
} KdaFoldArgs;
int kda_state_fold_ex(const KdaFoldArgs* args, void* stream);

/* The all-to-all exchange of the sequence split over peer memory (no reference counterpart: the
 * reference analyses the route only, tools/probe_segment_affine.py:100-125).  The caller maps every
 * rank's receive buffers and flag words into every process (CUDA IPC) and passes device pointers;
 * the library issues plain loads and stores on them -- no multicast, no TMA on peer memory -- and
 * every wait is bounded (status code 7 in *status when a flag does not arrive within a second).
 * Flags are int32 epoch counters in the WAITING rank's memory, zero at start, raised to the run's
 * epoch (1, 2, ...) by the rank that has stored the data.
 *
 * kda_peer_push: slice d (slice_floats fp32, a multiple of 4) of src goes to dst[d] +
 * dst_offset_floats; once the slice is complete *flag[d] = epoch.  counter: `world` zeroed int32 in
 * local memory, left zeroed.  One launch. */
#define KDA_MAX_PEERS 16
typedef struct KdaPeerPushArgs {
  const float* src;
  float* dst[KDA_MAX_PEERS];
  int32_t* flag[KDA_MAX_PEERS];
  int32_t* counter;
  int64_t slice_floats, dst_offset_floats;
  int32_t world, epoch;
} KdaPeerPushArgs;
int kda_peer_push(const KdaPeerPushArgs* args, void* stream);

/* kda_fwd_k2_state_push: kda_fwd_k2_state(args, 2, stream) and kda_peer_push in ONE launch -- the
 * transform-pair pass writes the (M, Q) tiles of chain c straight into rank (c / hp)'s buffer,
 * push->dst[c / hp] + dst_offset_floats + (c % hp) * 2 * 128 * 128 with hp = slice_floats / (2 * 128 * 128)
 * = chains / world, and raises push->flag[d] when destination d is complete; args->ht and push->src are
 * not used.  Only the 8-row pair form does this: KDA_ERR_UNSUPPORTED when the problem has more chains
 * than that form takes (the caller then runs the two calls separately). */
int kda_fwd_k2_state_push(const KdaFwdArgs* args, const KdaPeerPushArgs* push, void* stream);

/* kda_state_fold_peer: kda_state_fold_ex on transforms that peers have stored into args->mq.  The
 * walk starts when the n_wait flags at wait_flags have reached epoch; the state before segment j
 * (j = n_seg: after the last) of chain c is written to s_in_seg[j] + c * 128 * 128 (typically
 * rank j's entry-state buffer; NULL entries are skipped; args->s_in is ignored); when all of it
 * has been stored, *signal[i] = epoch for i < n_signal.  counter: one zeroed int32, left zeroed. */
typedef struct KdaFoldPeerArgs {
  const int32_t* wait_flags;
  int32_t n_wait, epoch;
  float* s_in_seg[KDA_MAX_PEERS + 1];
  int32_t* signal[KDA_MAX_PEERS];
  int32_t n_signal;
  int32_t* counter;
} KdaFoldPeerArgs;
int kda_state_fold_peer(const KdaFoldArgs* args, const KdaFoldPeerArgs* peer, void* stream);

/* kda_fwd_k2_after_flags: kda_fwd_k2 whose entry state args->h0 is stored by other GPUs -- the kernel itself
 * waits (bounded, status code 7) until the n flags have reached epoch before it reads h0, while it
 * already loads the first records: kda_flag_wait + kda_fwd_k2 in one launch.  The 8-row and 16-row
 * forms do this; KDA_ERR_UNSUPPORTED for problems that run in the tensor-memory form. */
int kda_fwd_k2_after_flags(const KdaFwdArgs* args, const int32_t* flags, int32_t n, int32_t epoch, void* stream);

/* kda_peer_enable: lets kernels of the current device load from and store to memory of GPU
 * peer_device that this process has mapped (cudaDeviceEnablePeerAccess; already enabled is fine).
 * KDA_ERR_CUDA when the two GPUs have no peer path.  Call it once per peer before the first
 * kda_peer_push / kda_state_fold_peer that is given pointers into that GPU's memory. */
int kda_peer_enable(int32_t peer_device);

/* CUDA IPC helpers for that set-up.  kda_ipc_export: the 64-byte handle of the device allocation
 * that contains ptr and ptr's offset inside it (send both to the other processes).  kda_ipc_open:
 * maps such a handle for kernels of the CURRENT device (call it with the importing GPU current)
 * and returns base + offset; a handle is mapped once per process and device (further opens
 * of it are counted). */
int kda_ipc_export(const void* ptr, void* handle_out_64_bytes, int64_t* offset_out);
int kda_ipc_open(const void* handle_64_bytes, int64_t offset, void** ptr_out);
/* kda_ipc_close: gives back one kda_ipc_open of that handle on the current device; the mapping goes
 * with the last one.  The exporting process may free the allocation only after every importer has
 * closed it (or exited). */
int kda_ipc_close(const void* handle_64_bytes);

/* kda_flag_wait: a one-warp kernel that returns when the n (<= 32) flags have reached epoch, or
 * writes status code 7 to *status (may be NULL) after the wait limit.  Orders the launches behind
 * it on `stream` after the peers' stores. */
int kda_flag_wait(const int32_t* flags, int32_t n, int32_t epoch, int32_t* status, void* stream);

/* Token-by-token recurrence for decode steps and short sequences (T of one to a few dozen
 * tokens): reads the state from args->h0 (NULL = zeros), applies args->T tokens, writes the
 * outputs to args->o and the new state to args->ht (may be NULL; may be the same buffer as h0
 * for an in-place update; [B, H, V, K], or [B, H, K, V] with KDA_FLAG_STATE_K_FIRST, moved in that
 * layout).  Needs the gate, l2-norm and beta-sigmoid flag bits; args->workspace is not used.
 * The reference has no decode kernel (README.md:503-505 lists it as future work); the
 * arithmetic is the token recurrence its tests take as the gold (fused_recurrent_kda,
 * tests/test_kda_bt16.py:26-39) with the chunk path's rounding of the normalised q and k, so a
 * prefill by kda_fwd followed by steps of this function continues the same sequence. */
int kda_recurrent_fwd(const KdaFwdArgs* args, void* stream);

/* Host helper for packed variable-length input: from cu_seqlens[0..n_seqs] (HOST memory,
 * non-decreasing, cu_seqlens[0] = 0, no empty sequence) fills chunk_table ([n_chunks][4]) and
 * seq_table ([n_seqs][4]) in HOST memory for H heads; the caller copies them to the device.
 * Called with chunk_table == NULL it only counts.  Returns n_chunks, or a negative error. */
int kda_varlen_fill_tables(const int32_t* cu_seqlens, int32_t n_seqs, int32_t H, int32_t* chunk_table,
                           int32_t* seq_table);

/* Self-test of the failure path (no reference counterpart): launches a one-warp kernel that waits,
 * with the same bounded wait every kernel of the library uses, on a barrier nothing arrives on.  The
 * wait gives up after its limit (one second), the kernel writes status code 100 into the status word
 * at the start of `workspace` (at least 256 bytes of device memory) and returns normally;
 * kda_fwd_status then reports KDA_ERR_DEVICE_STATUS, and the GPU context stays usable. */
int kda_selftest_bounded_wait(void* workspace, void* stream);

/* Whole forward with the K1 -> K2 scratch taken from a fixed array inside the library instead
 * of args->workspace (which is ignored).  It has no counterpart in the reference, whose host
 * code always allocates its intermediates itself.  It exists for callers that cannot obtain
 * device memory at call time -- a serving loop that gave all free GPU memory to its own pool and
 * keeps the CUDA allocator off the request path, or a plugin whose host passes tensors but no
 * allocator.  Limits: the problem must satisfy
 * kda_fwd_workspace_bytes(B, T, H) <= KDA_STATIC_SCRATCH_BYTES (else KDA_ERR_INVALID_ARG, nothing
 * runs); the array occupies that much memory on every GPU that loads the library, until exit; all
 * calls on a device share it, so calls that may overlap on the GPU must be ordered by the caller;
 * the first call on a device resolves the array's address and should be made outside stream
 * capture.  No allocation routine is called. */
#define KDA_STATIC_SCRATCH_BYTES (32 * 1024 * 1024)
int kda_fwd_static_scratch(const KdaFwdArgs* args, void* stream);

/* Synchronising read of the status word that kda_fwd_static_scratch's kernels report through (it
 * sits at the start of the library's own array on the current device, whose address no caller
 * has): 0 = every bounded device-side wait of the last call completed; otherwise the code is
 * stored and KDA_ERR_DEVICE_STATUS returned, as by kda_fwd_status.  No reference counterpart. */
int kda_fwd_static_scratch_status(void* stream, int32_t* status_out);

/* Synchronising read of the device status word of a workspace (0 = every bounded
 * wait inside the kernels completed). */
int kda_fwd_status(const void* workspace, void* stream, int32_t* status_out);

/* Which organisation of K2 a call with these arguments runs, without running it: k2_variant
 * (1 n8, 3 m16, 4 tc; with tc chosen automatically, a last partial wave of at most SMs/2 chains runs in
 * the m16 form as a second launch) and k2_vsplit (CTAs per chain; 1 for tc) as kda_fwd / kda_fwd_k2 (state_only = 0) or kda_fwd_k2_state
 * (state_only = 1) resolve the zeros ("automatic") in args.  Reads B, T, H, n_seqs, n_chunks,
 * k2_variant and k2_vsplit only; no pointer in args is touched and no CUDA work is issued.
 * sm_count = 0 takes the SM count of the current device (148 without one).  No reference
 * counterpart: the reference has one K2 (src/kda_bt16/kernels.py:188-318). */
int kda_fwd_k2_choice(const KdaFwdArgs* args, int state_only, int sm_count, int32_t* variant_out, int32_t* vsplit_out);

/* Number of kernels the last kda_fwd* call on this thread launched. */
int kda_last_launch_count(void);

const char* kda_last_error(void);

/* "major.minor" of the library and the SM architecture it was built for. */
const char* kda_version(void);

#ifdef __cplusplus
}
#endif
#endif /* KDA_B200_H_ */
