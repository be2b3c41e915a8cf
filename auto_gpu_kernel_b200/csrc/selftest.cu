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

// ------------------------------------------------------------------------------------------------
// Issue-rate measurement of the two tensor-core instruction families, on operands that are all
// zero (one CTA, nothing read from or written to global memory but the two cycle counts).  It
// backs the choice of instruction for the sparse attention: with 16 heads the tcgen05 products have
// N = 16, and what a tcgen05.mma costs there -- about the same whatever M is -- against what
// mma.sync m16n8k16 costs per SM is the whole argument.
namespace dsa {

// `iters` tcgen05.mma (M x n x 16 bf16, or M x n x 32 e4m3) issued back to back by one thread into
// one accumulator; cycles[0] = until the last one is issued, cycles[1] = until all have completed.
template <bool kFp8>
__global__ void __launch_bounds__(128, 1)
tcgen05_rate_selftest_kernel(int m, int n, int iters, long long* cycles, int32_t* status) {
  extern __shared__ unsigned char dyn[];
  __shared__ uint32_t tmem_slot;
  __shared__ uint64_t bar;
  const uint32_t raw = smem_u32(dyn);
  const uint32_t base = (raw + 1023u) & ~1023u;     // A at base (128 rows x 128 B), B at base + 64 KB (256 rows)
  for (int i = threadIdx.x; i < (96 * 1024) / 4; i += blockDim.x)
    reinterpret_cast<uint32_t*>(dyn + (base - raw))[i] = 0u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == 0) {
    if (lane == 0) { ptx::mbar_init(smem_u32(&bar), 1); ptx::fence_barrier_init(); }
    __syncwarp();
    ptx::tmem_alloc(smem_u32(&tmem_slot), 256);
    ptx::tmem_relinquish();
  }
  ptx::fence_proxy_async_smem();
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tm = tmem_slot;
  if (threadIdx.x == 0) {
    const uint32_t fmt = kFp8 ? ptx::kFmtE4M3 : ptx::kFmtBF16;
    const uint32_t id = ptx::idesc(fmt, fmt, false, false, (uint32_t)m, (uint32_t)n);
    const uint64_t ad = ptx::smem_desc_sw128(base, 16, 1024), bd = ptx::smem_desc_sw128(base + 65536, 16, 1024);
    const long long t0 = clock64();
    for (int i = 0; i < iters; ++i) {               // four K slices of the 128-byte rows in turn
      const uint64_t a = ad + 2 * (i & 3), b = bd + 2 * (i & 3);
      if (kFp8) ptx::mma_f8(tm, a, b, id, true);
      else ptx::mma_bf16_split(tm, (uint32_t)a, (uint32_t)(a >> 32), (uint32_t)b, (uint32_t)(b >> 32), id, 1u);
    }
    const long long t1 = clock64();
    ptx::tc_commit(smem_u32(&bar));
    const bool ok = ptx::mbar_wait(smem_u32(&bar), 0);
    const long long t2 = clock64();
    if (!ok) raise_status(status, DSA_STATUS_WAIT_TIMEOUT);
    cycles[0] = t1 - t0;
    cycles[1] = t2 - t0;
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 0) ptx::tmem_dealloc(tm, 256);
}

// `iters` x 8 independent mma.sync.m16n8k16 (bf16, fp32 accumulate) per warp, `blockDim.x / 32`
// warps; cycles[0] = cycles[1] = duration seen by warp 0.
__global__ void mma_sync_rate_selftest_kernel(int iters, long long* cycles, float* sink) {
  uint32_t a0 = threadIdx.x, a1 = 1, a2 = 2, a3 = 3, b0 = 4, b1 = 5;
  float c[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i) c[i][0] = c[i][1] = c[i][2] = c[i][3] = 0.f;
  __syncthreads();
  const long long t0 = clock64();
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int i = 0; i < 8; ++i)
      asm volatile(
          "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
          : "+f"(c[i][0]), "+f"(c[i][1]), "+f"(c[i][2]), "+f"(c[i][3])
          : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
  const long long t1 = clock64();
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) s += c[i][0] + c[i][1] + c[i][2] + c[i][3];
  if (s == 12345.678f) sink[0] = s;                 // keeps the products alive
  if (threadIdx.x == 0) { cycles[0] = t1 - t0; cycles[1] = t1 - t0; }
}

}  // namespace dsa

extern "C" int dsa_selftest_mma_rate(int kind, int m, int n, int iters, long long* cycles_dev,
                                     float* sink_dev, int32_t* status_dev, void* stream) {
  if (!cycles_dev || !sink_dev) return DSA_ERR_NULL_POINTER;
  if (iters <= 0 || iters > (1 << 20)) return DSA_ERR_BAD_SHAPE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (kind == 2) {   // mma.sync: m = warps of the one CTA
    if (m < 1 || m > 32) return DSA_ERR_BAD_SHAPE;
    dsa::mma_sync_rate_selftest_kernel<<<1, 32 * m, 0, s>>>(iters, cycles_dev, sink_dev);
    return static_cast<int>(cudaGetLastError());
  }
  if (kind != 0 && kind != 1) return DSA_ERR_UNSUPPORTED;
  if ((m != 64 && m != 128) || n < 16 || n > 256 || (n % 16) != 0) return DSA_ERR_BAD_SHAPE;
  const size_t smem = 1024 + 96 * 1024;
  cudaError_t e = cudaSuccess;
  if (kind == 1) {
    e = cudaFuncSetAttribute(dsa::tcgen05_rate_selftest_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    dsa::tcgen05_rate_selftest_kernel<true><<<1, 128, smem, s>>>(m, n, iters, cycles_dev, status_dev);
  } else {
    e = cudaFuncSetAttribute(dsa::tcgen05_rate_selftest_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    dsa::tcgen05_rate_selftest_kernel<false><<<1, 128, smem, s>>>(m, n, iters, cycles_dev, status_dev);
  }
  return static_cast<int>(cudaGetLastError());
}
