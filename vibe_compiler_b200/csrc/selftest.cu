// Self-test of the bounded device-side waits: a kernel waits on an mbarrier that nothing will ever arrive on, with a
// caller-chosen cycle limit, gives up, records the timeout in the backend's status word and returns, so the context stays
// usable and the next wb200_backend_poll() reports WB200_ERR_DEVICE_TIMEOUT. This is how the waits of the tcgen05 kernels
// end when a producer never shows up (their limit is about a second); the test form runs out in microseconds.
#include "backend.h"
#include "ptx_sm100.cuh"

namespace wb200 {
namespace {

__global__ void bounded_wait_kernel(long long cycle_limit, int *status, long long *waited_cycles) {
  __shared__ uint64_t barrier;
  __shared__ int abort_word;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&barrier), 1);
    abort_word = 0;
    fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const long long start = clock64();
    const bool arrived = mbar_wait(smem_u32(&barrier), 0, &abort_word, kDeviceWaitTimeout, cycle_limit);
    *waited_cycles = clock64() - start;
    if (!arrived) atomicExch(status, abort_word);
  }
}

}  // namespace
}  // namespace wb200

extern "C" wb200_status wb200_selftest_bounded_wait(wb200_backend *backend, uint64_t cycle_limit, uint64_t *waited_cycles) {
  using namespace wb200;
  if (!backend) return fail(WB200_ERR_INVALID_ARGUMENT, "backend is null");
  if (cycle_limit == 0 || cycle_limit > 2000000000ull) return fail(WB200_ERR_INVALID_ARGUMENT, "cycle limit must lie in (0, 2e9]");
  DeviceGuard guard(backend->device);
  void *scratch;
  wb200_status st = backend->buffer(9, sizeof(long long), &scratch);
  if (st != WB200_OK) return st;
  bounded_wait_kernel<<<1, 32, 0, backend->stream>>>(static_cast<long long>(cycle_limit), backend->d_status, static_cast<long long *>(scratch));
  WB200_CUDA_CHECK(cudaGetLastError());
  backend->launches += 1;
  long long waited = 0;
  WB200_CUDA_CHECK(cudaMemcpyAsync(&waited, scratch, sizeof(waited), cudaMemcpyDeviceToHost, backend->stream));
  WB200_CUDA_CHECK(cudaStreamSynchronize(backend->stream));
  if (waited_cycles) *waited_cycles = static_cast<uint64_t>(waited);
  return WB200_OK;
}
