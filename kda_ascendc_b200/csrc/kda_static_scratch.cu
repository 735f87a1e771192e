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
//   * Neither this function nor anything it calls uses cudaMalloc, cudaFree, or an allocating
//     library routine.
#include <cstdio>

#include "../../include/kda_b200.h"
#include "kda_common.cuh"

namespace kda {
void set_last_error(const char* msg);   // kda_c_api.cu
}

namespace {

static __device__ __align__(256) unsigned char g_kda_scratch[KDA_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
void* g_scratch_addr[kMaxDevices] = {};   // device address of g_kda_scratch, per device ordinal

}  // namespace

extern "C" int kda_fwd_static_scratch(const KdaFwdArgs* args, void* stream) {
  char msg[256];
  if (args == nullptr) {
    kda::set_last_error("kda: args is NULL");
    return KDA_ERR_INVALID_ARG;
  }
  // packed sequences hold one record per (chunk, head) of their chunk table
  const size_t need = args->n_seqs > 0 ? kda_fwd_workspace_bytes(1, 16 * args->n_chunks, args->H)
                                       : kda_fwd_workspace_bytes(args->B, args->T, args->H);
  if (need == 0) {
    kda::set_last_error("kda: B, T, H must be positive");
    return KDA_ERR_INVALID_ARG;
  }
  if (need > static_cast<size_t>(KDA_STATIC_SCRATCH_BYTES)) {
    snprintf(msg, sizeof(msg),
             "kda: kda_fwd_static_scratch holds %lld bytes of scratch, this problem (B=%d T=%d H=%d) needs %lld; "
             "use kda_fwd with a caller-provided workspace",
             static_cast<long long>(KDA_STATIC_SCRATCH_BYTES), args->B, args->T, args->H, static_cast<long long>(need));
    kda::set_last_error(msg);
    return KDA_ERR_INVALID_ARG;
  }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    kda::set_last_error("kda: cannot determine the current CUDA device");
    return KDA_ERR_CUDA;
  }
  if (g_scratch_addr[dev] == nullptr) {
    // once per device, with that device current: turn the host-side handle into the address
    // the kernels can use
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_kda_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      snprintf(msg, sizeof(msg), "kda: cudaGetSymbolAddress(static scratch) failed: %s", cudaGetErrorString(e));
      kda::set_last_error(msg);
      return KDA_ERR_CUDA;
    }
    g_scratch_addr[dev] = ptr;
  }
  KdaFwdArgs local = *args;                  // the caller's block is left untouched
  local.workspace = g_scratch_addr[dev];     // whatever the caller put there is ignored
  return kda_fwd(&local, stream);            // clears the status block, then K1 and K2
}
