// Exchange of the selected index rows between the GPUs of a head-sharded layer, without NCCL.
//
// In the head-sharded layout every rank runs the indexer for its own requests and the attention
// of ALL requests for its own heads, so each rank needs every rank's int32 [rows, 2048] index rows
// (the reference has no multi-GPU code; its two operators meet only through this tensor:
// indexer_baseline.py:82-90 -> sparse_baseline.py:22-28).  One kernel per rank and step does both
// directions with no fence and no separate flag:
//   * push: the CTA of a LOCAL row reads it from the rank's own index tensor and stores it into the
//     row's place of every peer's staging buffer as (id, epoch) pairs -- 16-byte stores of two
//     pairs over NVLink, each 8-byte pair written whole;
//   * take: the CTA of a REMOTE row polls that row of its OWN staging buffer until every pair
//     carries this call's epoch, and writes the ids into the rank's index tensor.
// A pair that carries the epoch is its own proof of arrival, so the latency is one NVLink trip
// instead of data + fence + flag.  The poll has a time limit that ends in DSA_STATUS_WAIT_TIMEOUT.
// The push half can also run at the end of the selection kernel (topk_select_hist_kernel sends
// every row as soon as it is complete, while other requests are still being selected); this kernel
// is then launched for the take half only (`mode`: 1 = push, 2 = take, 3 = both).
// Nothing is ever read from a peer's memory, and nothing on this GPU waits for another kernel of
// this GPU.  The host alternates two staging buffers with the epoch's parity: a rank can run at
// most one step ahead of a peer's take, so it never overwrites pairs that are still being read.
#include "common.cuh"
#include "ptx.cuh"
#include "tmap.cuh"

namespace dsa {

constexpr int kXchThreads = 256;

namespace {

__device__ __forceinline__ uint4 ld_volatile_v4(const uint4* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(kXchThreads)
index_rows_exchange_kernel(int32_t* __restrict__ rows, const __grid_constant__ RowSend xs, int rows_local, int rows_total,
                           int64_t row_stride, int mode, uint64_t limit_ns, int32_t* status) {
  const int rank = xs.rank, row_offset = xs.row_offset, row_width = xs.row_width;
  const uint32_t epoch = xs.epoch;
  const int tid = threadIdx.x;
  // the local rows come from the selection kernel before us in the stream
  ptx::grid_dependency_wait();
  ptx::launch_dependents();   // the attention behind us waits for this whole kernel by itself
  const int pairs2 = row_width / 2;   // 16-byte units (two pairs) per row
  // ---- push: local row b by CTA b, b + grid, ... (before any take: a CTA never polls while it
  //      still has rows to send); skipped when the selection kernel has sent them itself ----
  if (mode & 1) {
    for (int b = blockIdx.x; b < rows_local; b += gridDim.x)
      send_row_pairs(xs, rows + (size_t)(row_offset + b) * row_stride, row_offset + b);
  }
  if (!(mode & 2)) return;
  // ---- take: the k-th remote row by CTA k, k + grid, ... ----
  const int rows_remote = rows_total - rows_local;
  for (int k = blockIdx.x; k < rows_remote; k += gridDim.x) {
    const int i = k < row_offset ? k : k + rows_local;
    int32_t* row = rows + (size_t)i * row_stride;
    const uint4* src = reinterpret_cast<const uint4*>(own_stage(xs) + (size_t)i * row_width);
    uint64_t t0 = 0;
    bool gave_up = false;
    for (int u = tid; u < pairs2; u += kXchThreads) {
      uint4 v = ld_volatile_v4(src + u);
      for (uint32_t spins = 0; !gave_up && (v.y != epoch || v.w != epoch); ++spins) {
        if ((spins & 31u) == 31u) {
          const uint64_t now = ptx::global_timer_ns();
          if (t0 == 0) t0 = now;
          else if (now - t0 > limit_ns) gave_up = true;
        }
        v = ld_volatile_v4(src + u);
      }
      if (gave_up) break;
      reinterpret_cast<int2*>(row)[u] = make_int2((int32_t)v.x, (int32_t)v.z);
    }
    if (gave_up) raise_status(status, DSA_STATUS_WAIT_TIMEOUT);
  }
}

}  // namespace

cudaError_t launch_index_rows_exchange(int32_t* rows, const RowSend& xs, int rows_local, int rows_total,
                                       int64_t row_stride, int mode, uint64_t limit_ns, int32_t* status,
                                       cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  const int ctas = (mode & 2) ? rows_total : rows_local;
  cfg.gridDim = dim3((unsigned)min(max(ctas, 1), 1024));
  cfg.blockDim = dim3(kXchThreads);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled();
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, index_rows_exchange_kernel, rows, xs, rows_local, rows_total,
                            row_stride, mode, limit_ns, status);
}

}  // namespace dsa
