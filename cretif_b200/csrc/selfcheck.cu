// A launch that runs the library's bounded wait to its end, harmlessly.
//
// Every wait inside the kernels (on an mbarrier that a TMA copy or a tensor-core product
// completes) gives up after a number of polls, raises its CTA's abort flag, sets
// kFaultWaitExpired in the device status word and lets the kernel return; the host finds the
// bit at its next synchronisation.  That path cannot be reached by a healthy kernel, so this
// file offers one CTA that waits on a barrier nothing will ever complete, with a poll limit
// of the caller's choosing.  It lets tests (and an application's start-up check) see the
// whole chain — expired wait, status word, the host's error, a usable context afterwards —
// without a fault, a trap or an unbounded loop.
#include "api.h"
#include "tc_common.cuh"

namespace cretif {

__global__ void wait_that_expires_kernel(unsigned limit, unsigned int* fault, unsigned int* polls) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    tc::mbar_init(&bar, 1);
    tc::fence_barrier_init();
  }
  __syncthreads();
  // phase 0 of a barrier that expects one arrival which never comes
  const bool ok = tc::mbar_wait(&bar, 0, &abort_flag, limit);
  __syncthreads();
  if (threadIdx.x == 0) {
    if (!ok) atomicOr(fault, kFaultWaitExpired);
    if (polls) *polls = limit;
  }
}

}  // namespace cretif

extern "C" int cretif_wait_that_expires(unsigned int limit, unsigned int* fault,
                                        unsigned int* polls, void* stream) {
  if (!fault || limit == 0 || limit > (1u << 20)) return cretif::kBadArgument;
  cretif::wait_that_expires_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(limit, fault, polls);
  return cretif::launch_status();
}
