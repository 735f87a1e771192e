// Self-test of the failure path every kernel of the library relies on: a bounded device-side wait
// that runs out, the status word it leaves behind, and a context that stays usable afterwards.
// The kernel waits on an mbarrier that nothing ever arrives on; the wait gives up after its time
// limit (WAIT_LIMIT_NS, one second), the kernel records a status code and returns normally -- no
// trap, no assert, no endless loop.
#include "../../include/kda_b200.h"
#include "kda_common.cuh"

namespace kda {
void set_last_error(const char* msg);

namespace {
constexpr int ST_SELFTEST_TIMEOUT = 100;

__global__ void kda_selftest_wait_kernel(int* status) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ int flag;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  // all 32 threads wait, as the consumer warps of K2 do; nobody ever arrives
  const bool ok = mbar_wait_bounded(smem_u32(&bar), 0, &flag);
  if (!ok && threadIdx.x == 0) atomicExch(status, ST_SELFTEST_TIMEOUT);
}
}  // namespace
}  // namespace kda

extern "C" int kda_selftest_bounded_wait(void* workspace, void* stream) {
  if (workspace == nullptr) {
    kda::set_last_error("kda: workspace is NULL");
    return KDA_ERR_INVALID_ARG;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(workspace, 0, kda::WS_HEADER_BYTES, st);
  if (e == cudaSuccess) {
    kda::kda_selftest_wait_kernel<<<1, 32, 0, st>>>(static_cast<int*>(workspace));
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) {
    kda::set_last_error(cudaGetErrorString(e));
    return KDA_ERR_CUDA;
  }
  return KDA_OK;
}
