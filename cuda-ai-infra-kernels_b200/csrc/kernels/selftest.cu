// Self tests of the library's safety plumbing, callable through the C ABI. They exist so that the
// paths a healthy run never takes - a device-side wait that gives up, a launch the runtime refuses -
// can be exercised without faulting, trapping or hanging anything.
#include "host_common.h"
#include "ptx_sm100.cuh"

namespace b200 {

cudaError_t selftest_status_read_clear(uint32_t* word) { return status_word_read_clear(word); }

namespace {

// One CTA, one thread: waits on a barrier phase that nothing will ever complete, with the same
// bounded wait the GEMM kernels use but a cap of `max_polls`. The wait gives up, records its site
// in the status word and the kernel returns normally.
__global__ void wait_gives_up_kernel(uint32_t max_polls, uint32_t* outcome) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_init_fence();
    const bool completed = mbar_wait(&bar, 0, kSiteSelfTest, max_polls);
    if (outcome != nullptr) *outcome = completed ? 1u : 2u;
  }
}

}  // namespace
}  // namespace b200

extern "C" {

int b200_selftest_wait_gives_up(uint32_t max_polls, uint32_t* outcome, b200_stream_t stream) {
  if (max_polls == 0 || max_polls > (1u << 20)) return B200_ERR_INVALID_ARGUMENT;   // a short wait only
  b200::wait_gives_up_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(max_polls, outcome);
  return b200::launch_status();
}

int b200_selftest_refused_launch(b200_stream_t stream) {
  // 2048 threads per block exceed every device's limit: the runtime refuses the launch on the host
  // (cudaErrorInvalidConfiguration, not sticky) and nothing reaches the GPU.
  b200::wait_gives_up_kernel<<<1, 2048, 0, static_cast<cudaStream_t>(stream)>>>(1, nullptr);
  return b200::launch_status();
}

}  // extern "C"
