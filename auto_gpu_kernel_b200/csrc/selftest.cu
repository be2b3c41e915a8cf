// Self-test of the bounded device-side wait that every pipeline in this library is built on.
//
// All mbarrier waits go through ptx::mbar_wait, which gives up after a time limit; the kernels
// then set DSA_STATUS_WAIT_TIMEOUT, let their roles leave together and return.  In normal
// operation the limit is never reached, so this entry point makes it run out on purpose in the
// only harmless way: one thread waits, with a short limit, on a barrier that nothing will ever
// arrive on.  Nothing faults and nothing spins past the limit; the CUDA context stays usable.
#include "common.cuh"
#include "ptx.cuh"

namespace dsa {

__global__ void wait_expiry_selftest_kernel(uint64_t limit_ns, int32_t* status, uint64_t* waited_ns) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    ptx::mbar_init(smem_u32(&bar), 1);   // expects one arrival; none will come
    ptx::fence_barrier_init();
    const uint64_t t0 = ptx::global_timer_ns();
    const bool completed = ptx::mbar_wait(smem_u32(&bar), 0, limit_ns);
    const uint64_t t1 = ptx::global_timer_ns();
    if (!completed) raise_status(status, DSA_STATUS_WAIT_TIMEOUT);
    if (waited_ns != nullptr) *waited_ns = t1 - t0;
  }
}

}  // namespace dsa

extern "C" int dsa_selftest_wait_expiry(uint64_t limit_ns, int32_t* status_dev, uint64_t* waited_ns_dev,
                                        void* stream) {
  if (!status_dev) return DSA_ERR_NULL_POINTER;
  if (limit_ns == 0 || limit_ns > 1000000000ull) return DSA_ERR_BAD_SHAPE;   // at most one second
  dsa::wait_expiry_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(limit_ns, status_dev,
                                                                                    waited_ns_dev);
  return static_cast<int>(cudaGetLastError());
}
