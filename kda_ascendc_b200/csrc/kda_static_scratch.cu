// kda_fwd_static_scratch: the whole forward for callers that have no device allocator to turn to.
//
// kda_fwd needs a K1 -> K2 scratch buffer from its caller.  Some callers cannot supply one at
// the moment of the call: a serving loop that handed every free byte of the GPU to its own
// memory pool at start-up and must not touch the CUDA allocator on the request path (an
// allocation can synchronise the whole device and may simply fail), or a plugin hosted by a
// runtime that gives it tensors but no allocation hook.  For them the scratch lives inside
// this library, in the fixed-size device array below.  Every GPU on which the library's code is
// loaded carries these KDA_STATIC_SCRATCH_BYTES until the process exits, whether or not the
// entry point is ever called; that is the price, and the reason the size is modest.
//
// Things a caller has to know:
//   * Problems whose scratch need (kda_fwd_workspace_bytes) exceeds the array are refused with
//     KDA_ERR_INVALID_ARG; nothing is launched.
//   * The first call on each device looks the array's device address up (cudaGetSymbolAddress;
//     the name `g_kda_scratch` in host code is only a handle, not an address a kernel could
//     use).  Make that first call outside of any stream capture.
//   * All calls on a device share the one array.  Two calls whose kernels can overlap on the
//     GPU (different streams without an ordering between them) corrupt each other; calls on
//     one stream, or otherwise ordered, are fine.  What a call left behind stays in the array:
//     the status block at its start is cleared by every call, and the chunk records are always
//     written by K1 before K2 reads them, so stale contents are never consumed.
//   * A bounded device-side wait that gave up leaves its code in the status word at the start of
//     the array; since the array's address never leaves the library, kda_fwd_static_scratch_status
//     reads that word for the current device (kda_fwd_status needs a caller-owned workspace).
//   * Neither this function nor anything it calls uses cudaMalloc, cudaFree, or an allocating
//     library routine.
#include <atomic>
#include <cstdio>

#include "../../include/kda_b200.h"
#include "kda_common.cuh"

namespace kda {
void set_last_error(const char* msg);   // kda_c_api.cu
}

namespace {

static __device__ __align__(256) unsigned char g_kda_scratch[KDA_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
// device address of g_kda_scratch, per device ordinal.  Two host threads that make their first
// call on one device at the same time both resolve the same address; the atomic only makes that
// race well defined.
std::atomic<void*> g_scratch_addr[kMaxDevices];

// Address of the array on the current device (resolved once per device, with that device
// current), or nullptr after setting the error text.
void* scratch_on_current_device(int* rc) {
  char msg[256];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    kda::set_last_error("kda: cannot determine the current CUDA device");
    *rc = KDA_ERR_CUDA;
    return nullptr;
  }
  void* ptr = g_scratch_addr[dev].load(std::memory_order_acquire);
  if (ptr == nullptr) {
    // turn the host-side handle into the address the kernels can use
    e = cudaGetSymbolAddress(&ptr, g_kda_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      snprintf(msg, sizeof(msg), "kda: cudaGetSymbolAddress(static scratch) failed: %s", cudaGetErrorString(e));
      kda::set_last_error(msg);
      *rc = KDA_ERR_CUDA;
      return nullptr;
    }
    g_scratch_addr[dev].store(ptr, std::memory_order_release);
  }
  return ptr;
}

}  // namespace

extern "C" int kda_fwd_static_scratch(const KdaFwdArgs* args, void* stream) {
  char msg[256];
  if (args == nullptr) {
    kda::set_last_error("kda: args is NULL");
    return KDA_ERR_INVALID_ARG;
  }
  // The number of chunk records, in 64 bits: packed sequences hold one record per (chunk, head) of
  // their chunk table, a fixed-length batch one per (batch, head, 16-token chunk).
  unsigned long long chunks = 0;
  if (args->n_seqs < 0) {
    kda::set_last_error("kda: n_seqs must not be negative");
    return KDA_ERR_INVALID_ARG;
  }
  if (args->n_seqs > 0) {
    if (args->n_chunks <= 0 || args->H <= 0) {
      kda::set_last_error("kda: packed sequences need positive n_chunks and H");
      return KDA_ERR_INVALID_ARG;
    }
    chunks = static_cast<unsigned long long>(args->n_chunks);
  } else {
    if (args->B <= 0 || args->T <= 0 || args->H <= 0) {
      kda::set_last_error("kda: B, T, H must be positive");
      return KDA_ERR_INVALID_ARG;
    }
    chunks = static_cast<unsigned long long>(args->B) * ((static_cast<unsigned long long>(args->T) + kda::BT - 1) / kda::BT);
  }
  constexpr unsigned long long kMaxRecords =
      (static_cast<unsigned long long>(KDA_STATIC_SCRATCH_BYTES) - kda::WS_HEADER_BYTES) / kda::REC_BYTES;
  // chunks < 2^58 and H < 2^31 here; comparing chunks first keeps the product below 2^64
  if (chunks > kMaxRecords || chunks * static_cast<unsigned long long>(args->H) > kMaxRecords) {
    snprintf(msg, sizeof(msg),
             "kda: kda_fwd_static_scratch holds %lld bytes of scratch (%llu chunk records), this problem "
             "(B=%d T=%d H=%d n_chunks=%d) needs %llu x %d records; use kda_fwd with a caller-provided workspace",
             static_cast<long long>(KDA_STATIC_SCRATCH_BYTES), kMaxRecords, args->B, args->T, args->H, args->n_chunks,
             chunks, args->H);
    kda::set_last_error(msg);
    return KDA_ERR_INVALID_ARG;
  }
  int rc = KDA_OK;
  void* scratch = scratch_on_current_device(&rc);
  if (scratch == nullptr) return rc;
  KdaFwdArgs local = *args;          // the caller's block is left untouched
  local.workspace = scratch;         // whatever the caller put there is ignored
  return kda_fwd(&local, stream);    // clears the status block, then K1 and K2
}

extern "C" int kda_fwd_static_scratch_status(void* stream, int32_t* status_out) {
  if (status_out == nullptr) {
    kda::set_last_error("kda: status_out is required");
    return KDA_ERR_INVALID_ARG;
  }
  int rc = KDA_OK;
  void* scratch = scratch_on_current_device(&rc);
  if (scratch == nullptr) return rc;
  return kda_fwd_status(scratch, stream, status_out);
}
