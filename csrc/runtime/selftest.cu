// Bounded-wait self test: a kernel waits on a flag of the local signal pad that
// nothing ever sets.  The wait runs out after the communicator's timeout, the
// kernel records who waited for what in the status block and returns normally,
// so the context stays usable.
//
// Capability parity: the only bounded wait of the reference is its host-mapped
// signal micro-test (src/test/host_mapped_ready_microtest.cu:42-71).
#include <cuda_runtime.h>
#include "../api/oob.h"
#include "../device/sync.cuh"
#include "comm.h"
#include "errors.h"

namespace oob {
namespace {
__global__ void bounded_wait_kernel(CommCtx ctx_param) {
  const CommCtx ctx = resolve_ctx(ctx_param);
  if (threadIdx.x == 0) {
    // The last general counter is reserved for this test and stays zero.
    const uint32_t* flag = counter_ptr(ctx, ctx.rank, kNumCounters - 1);
    wait_word_ge(ctx, flag, 1u, kDevTimeoutCounter, ctx.rank, 99);
  }
}
}  // namespace
}  // namespace oob

extern "C" int oob_test_bounded_wait(oob_comm* c, void* stream) {
  using namespace oob;
  if (c == nullptr) return set_error(OOB_ERR_INVALID, "null communicator");
  CommCtx ctx = c->make_ctx();
  if (c->emulated) {
    void* argv[] = {(void*)&ctx};
    cudaError_t e = cudaLaunchCooperativeKernel((const void*)bounded_wait_kernel, dim3(1, c->world), dim3(32), argv, 0,
                                                static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(e, "bounded wait launch");
    return OOB_OK;
  }
  bounded_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(ctx);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "bounded wait launch");
  return OOB_OK;
}
