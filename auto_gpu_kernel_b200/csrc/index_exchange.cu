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
// Nothing is ever read from a peer's memory, and nothing on this GPU waits for another kernel of
// this GPU.  The host alternates two staging buffers with the epoch's parity: a rank can run at
// most one step ahead of a peer's take, so it never overwrites pairs that are still being read.
#include "common.cuh"
#include "ptx.cuh"
#include "tmap.cuh"

namespace dsa {

constexpr int kXchThreads = 256;
constexpr int kXchMaxWorld = 8;

struct XchPeers {
  uint2* stage[kXchMaxWorld];   // every rank's [rows_total][row_width] (id, epoch) staging buffer
};

namespace {

__device__ __forceinline__ uint4 ld_volatile_v4(const uint4* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(kXchThreads)
index_rows_exchange_kernel(int32_t* __restrict__ rows, XchPeers peers, int world, int rank,
                           int rows_local, int row_offset, int rows_total, int64_t row_stride,
                           int row_width, uint32_t epoch, uint64_t limit_ns, int32_t* status) {
  const int tid = threadIdx.x;
  // the local rows come from the selection kernel before us in the stream
  ptx::grid_dependency_wait();
  ptx::launch_dependents();   // the attention behind us waits for this whole kernel by itself
  const int pairs2 = row_width / 2;   // 16-byte units (two pairs) per row
  // ---- push: local row b by CTA b, b + grid, ... (before any take: a CTA never polls while it
  //      still has rows to send) ----
  for (int b = blockIdx.x; b < rows_local; b += gridDim.x) {
    const int i = row_offset + b;
    const int32_t* row = rows + (size_t)i * row_stride;
    for (int u = tid; u < pairs2; u += kXchThreads) {
      const int2 v = __ldcg(reinterpret_cast<const int2*>(row) + u);
      const uint4 packed = make_uint4((uint32_t)v.x, epoch, (uint32_t)v.y, epoch);
      for (int p = 0; p < world; ++p) {
        if (p == rank) continue;
        reinterpret_cast<uint4*>(peers.stage[p] + (size_t)i * row_width)[u] = packed;
      }
    }
  }
  // ---- take: the k-th remote row by CTA k, k + grid, ... ----
  const int rows_remote = rows_total - rows_local;
  for (int k = blockIdx.x; k < rows_remote; k += gridDim.x) {
    const int i = k < row_offset ? k : k + rows_local;
    int32_t* row = rows + (size_t)i * row_stride;
    const uint4* src = reinterpret_cast<const uint4*>(peers.stage[rank] + (size_t)i * row_width);
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

cudaError_t launch_index_rows_exchange(int32_t* rows, uint2* const* peer_stage, int world, int rank,
                                       int rows_local, int row_offset, int rows_total, int64_t row_stride,
                                       int row_width, uint32_t epoch, uint64_t limit_ns, int32_t* status,
                                       cudaStream_t stream) {
  XchPeers peers = {};
  for (int p = 0; p < world; ++p) peers.stage[p] = peer_stage[p];
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)min(max(rows_total, 1), 1024));
  cfg.blockDim = dim3(kXchThreads);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled();
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, index_rows_exchange_kernel, rows, peers, world, rank, rows_local,
                            row_offset, rows_total, row_stride, row_width, epoch, limit_ns, status);
}

}  // namespace dsa
