// Self-test of the bounded-wait machinery every pipeline kernel of this library relies on.
//
// The GEMM and attention kernels wait on mbarriers through mbar_wait(), which gives up after
// B200AIT_WAIT_LIMIT_NS, records a code in the device status word, raises the CTA-wide abort flag and
// returns. In a healthy run that branch never executes, so this file compiles the very same
// mbar_wait() with a 1 ms limit and points it at a barrier nobody ever arrives on: one CTA, one
// waiting thread, which gives up after about a millisecond and returns. Nothing traps, faults or
// spins without bound; the host then sees the status code exactly as it would after a stuck
// pipeline (b200ait_device_status, or the error a synchronous Run raises).
#define B200AIT_WAIT_LIMIT_NS 1000000ull  // 1 ms
#include "common.h"
#include "ptx.cuh"

namespace b200ait {

__global__ void selftest_bounded_wait_kernel(int* status, unsigned long long* waited_ns, int* returned_flags) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&bar, 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint64_t t0 = globaltimer_ns();
    const bool ok = mbar_wait(&bar, 0, &abort_flag, status, kDevWaitOtherTimeout);  // nobody arrives: must give up
    *waited_ns = globaltimer_ns() - t0;
    returned_flags[0] = ok ? 1 : 0;
  }
  __syncthreads();
  // every other thread's wait now returns at once because the abort flag is up
  if (threadIdx.x == 32) returned_flags[1] = mbar_wait(&bar, 0, &abort_flag, status, kDevWaitFullTimeout) ? 1 : 0;
}

}  // namespace b200ait

using namespace b200ait;

// Launches the kernel above on `stream` and waits for it. out[0] = what the first wait returned
// (0 = gave up, as it must), out[1] = what a later wait in the same CTA returned (0 = skipped at
// once), out[2] = nanoseconds the first wait spent before giving up. The device status word is left
// holding kDevWaitOtherTimeout (5) for b200ait_device_status / a synchronous Run to find and clear.
B200AIT_EXPORT int b200ait_selftest_bounded_wait(int64_t* out, cudaStream_t stream) {
  return guarded("b200ait_selftest_bounded_wait", [&] {
    B200AIT_REQUIRE(out, "out is null");
    int* status = device_status_word();
    unsigned long long* d_ns = nullptr;
    int* d_flags = nullptr;
    B200AIT_CUDA_CHECK(cudaMalloc(&d_ns, sizeof(unsigned long long)));
    B200AIT_CUDA_CHECK(cudaMalloc(&d_flags, 2 * sizeof(int)));
    B200AIT_CUDA_CHECK(cudaMemsetAsync(d_flags, 0xff, 2 * sizeof(int), stream));
    ::b200ait::count_launch(), selftest_bounded_wait_kernel<<<1, 64, 0, stream>>>(status, d_ns, d_flags);
    unsigned long long ns = 0;
    int flags[2] = {-1, -1};
    cudaError_t e = cudaStreamSynchronize(stream);
    if (e == cudaSuccess) e = cudaMemcpy(&ns, d_ns, sizeof(ns), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess) e = cudaMemcpy(flags, d_flags, sizeof(flags), cudaMemcpyDeviceToHost);
    cudaFree(d_ns);
    cudaFree(d_flags);
    B200AIT_CUDA_CHECK(e);
    out[0] = flags[0];
    out[1] = flags[1];
    out[2] = static_cast<int64_t>(ns);
  });
}
