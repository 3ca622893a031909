// Self-test of the failure path: a wait that nothing will ever satisfy must give up after its time
// limit, record its code in the status word and let the kernel end normally, so that the host can
// read the code and the context stays usable.  Nothing here faults, traps or spins without a bound.
#include "forge_host.h"
#include "forge_ptx.cuh"

namespace forge {

constexpr int ERR_SELFTEST_WAIT = 190;

// One CTA.  Thread 0 waits, with the same bounded wait the update kernels use, on a barrier no one
// arrives on; the other threads wait on a second barrier that thread 0 would arrive on after a
// successful wait -- they see the abort word instead and return as well.
__global__ void forge_selftest_wait_kernel(int* status, unsigned long long limit_ns) {
  __shared__ uint64_t never;
  __shared__ uint64_t after;
  __shared__ int abort_word;
  if (threadIdx.x == 0) {
    mbar_init(&never, 1);
    mbar_init(&after, 1);
    abort_word = 0;
    mbar_fence_init();
  }
  __syncthreads();
  volatile int* aw = &abort_word;
  if (threadIdx.x == 0) {
    if (mbar_wait(&never, 0, aw, ERR_SELFTEST_WAIT, limit_ns)) mbar_arrive(&after);
  } else {
    // a longer limit: these threads must leave because thread 0 gave up, not on their own clock
    mbar_wait(&after, 0, aw, ERR_SELFTEST_WAIT + 1, 100 * limit_ns + 1000000ull);
  }
  __syncthreads();
  if (threadIdx.x == 0 && abort_word != 0 && status != nullptr) atomicCAS(status, 0, abort_word);
}

}  // namespace forge

extern "C" int forge_selftest_wait_timeout(int32_t* status, uint64_t limit_ns, void* cuda_stream) {
  using namespace forge;
  if (status == nullptr) return fail(FORGE_ERR_INVALID_ARG, "forge_selftest_wait_timeout: status is NULL");
  if (limit_ns == 0 || limit_ns > 1000000000ull)
    return fail(FORGE_ERR_INVALID_ARG, "forge_selftest_wait_timeout: limit must be 1 ns .. 1 s");
  forge_selftest_wait_kernel<<<1, 64, 0, static_cast<cudaStream_t>(cuda_stream)>>>(status, limit_ns);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(FORGE_ERR_CUDA, "self-test launch: %s", cudaGetErrorString(e));
  return FORGE_OK;
}
