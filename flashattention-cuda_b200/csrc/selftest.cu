// Self-test of the bounded-wait machinery every tcgen05 kernel of the library relies on.
//
// The pipelines of the dense and MLA kernels wait on mbarriers; each wait gives up after a cycle bound,
// raises the CTA's abort flag and records a code in the device status word, so that a protocol error ends
// the launch with a readable status instead of a hung GPU.  This entry point runs that wait on a barrier
// that nothing ever arrives on, with a bound the caller chooses (a millisecond is plenty), so that the
// give-up path and the host side that reads the word can be exercised without disturbing a real pipeline.

#include "sm100.cuh"

namespace fa {
namespace {

__global__ void bounded_wait_probe_kernel(int* status, long long max_cycles, int code, int* gave_up) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    sm100::mbar_init(smem_u32(&bar), 1);
    sm100::fence_barrier_init();
  }
  __syncthreads();
  // phase 0 of a fresh barrier never completes without an arrival
  const bool ok = sm100::mbar_wait_cycles(smem_u32(&bar), 0, &abort_flag, status, code, max_cycles);
  __syncthreads();
  if (threadIdx.x == 0 && gave_up) *gave_up = ok ? 0 : 1;
}

}  // namespace
}  // namespace fa

extern "C" int fa_selftest_bounded_wait(int32_t* status, long long max_cycles, int code, int32_t* gave_up, void* stream) {
  FA_CHECK_ARG(status != nullptr, "fa_selftest_bounded_wait: null status word");
  FA_CHECK_ARG(max_cycles >= 0 && max_cycles <= 2000000000LL, "fa_selftest_bounded_wait: max_cycles must be in [0, 2e9]");
  FA_CHECK_ARG(code > 0 && code < 0x10000, "fa_selftest_bounded_wait: code must be in (0, 65536)");
  fa::bounded_wait_probe_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(status, max_cycles, code, gave_up);
  FA_CUDA_OK(cudaGetLastError());
  return FA_OK;
}
