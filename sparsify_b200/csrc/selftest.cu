// Self-test of the bounded device-side wait that every tensor-core kernel of
// this library uses (sc::tc::mbar_wait): a one-thread kernel waits, for a
// caller-chosen limit, on an mbarrier that nothing ever arrives on. Nothing
// asynchronous is outstanding when it gives up, so the kernel simply returns;
// the wait's code is left in the status word, exactly as a stalled pipeline
// stage of the encoder or GEMM kernels would leave it.
#include "tc.cuh"

namespace {

using namespace sc::tc;

constexpr int32_t kSelftestWaitCode = 199;

__global__ void wait_timeout_kernel(int32_t* status, uint64_t limit_ns) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    fence_barrier_init();
    mbar_wait(&bar, 0, status, kSelftestWaitCode, limit_ns);
  }
}

}  // namespace

extern "C" int sc_selftest_wait_timeout(int32_t* status_word, int64_t limit_ns, void* stream) {
  SC_REQUIRE(status_word != nullptr, "sc_selftest_wait_timeout: null status word");
  SC_REQUIRE(limit_ns > 0 && limit_ns <= 100000000LL, "sc_selftest_wait_timeout: limit must be in (0, 100 ms]");
  cudaStream_t st = sc::as_stream(stream);
  SC_CUDA(cudaMemsetAsync(status_word, 0, sizeof(int32_t), st));
  wait_timeout_kernel<<<1, 32, 0, st>>>(status_word, (uint64_t)limit_ns);
  SC_CHECK_LAUNCH("sc_selftest_wait_timeout");
  return SC_OK;
}
