// Self-test of the bounded device-side wait that every tensor-core kernel of this library relies on (csrc/tc_util.cuh).
//
// A kernel that waits on a barrier nothing ever arrives on must give up after its poll limit, raise the wait-timeout bit of the
// device error word and return, leaving the context usable: vb_check_errors() then reports "a device-side wait ran out" and the
// next launches run normally.  This entry point makes exactly that happen, on purpose and in one CTA, with a short poll limit:
// no fault, no trap, no unbounded loop.  It also measures how long the polls take, which gives the give-up time of the
// production limit (2^20 polls).
#include "common.h"
#include "tc_util.cuh"

namespace vb {
namespace {
__global__ void k_wait_selftest(int* err, uint32_t limit) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    tc::mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // thread 0 plays a role whose partner never shows up; the others are the roles that learn of it through the abort flag
  if (threadIdx.x == 0) (void)tc::mbar_wait(&bar, 0, &abort_flag, limit);
  __syncthreads();
  if (threadIdx.x == 0 && abort_flag) atomicOr(err, ERRBIT_WAIT_TIMEOUT);
}
}  // namespace
}  // namespace vb

extern "C" int vb_selftest_wait_timeout(uint32_t polls, double* elapsed_ms) {
  using namespace vb;
  if (!ctx().ready) return set_error(VB_ERR_NOT_INIT, "vb_init has not been called");
  if (polls == 0 || polls > (1u << 16)) return set_error(VB_ERR_INVALID, "vb_selftest_wait_timeout: polls must be in 1..65536");
  cudaEvent_t e0, e1;
  VB_CUDA(cudaEventCreate(&e0)); VB_CUDA(cudaEventCreate(&e1));
  cudaStream_t st = ctx().stream;
  cudaEventRecord(e0, st);
  k_wait_selftest<<<1, 64, 0, st>>>(ctx().d_err, polls);
  cudaEventRecord(e1, st);
  cudaError_t rc = cudaEventSynchronize(e1);
  float ms = 0.0f;
  if (rc == cudaSuccess) rc = cudaEventElapsedTime(&ms, e0, e1);
  cudaEventDestroy(e0); cudaEventDestroy(e1);
  if (rc != cudaSuccess) return set_error(VB_ERR_CUDA, cudaGetErrorString(rc));
  if (elapsed_ms) *elapsed_ms = (double)ms;
  VB_LAUNCH_CHECK();
  return VB_OK;
}
