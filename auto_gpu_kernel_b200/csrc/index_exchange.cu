// Exchange of the selected index rows between the GPUs of a head-sharded layer, without NCCL.
//
// In the head-sharded layout every rank runs the indexer for its own requests and the attention
// of ALL requests for its own heads, so each rank needs every rank's int32 [rows, 2048] index rows
// (the reference has no multi-GPU code; its two operators meet only through this tensor:
// indexer_baseline.py:82-90 -> sparse_baseline.py:22-28).  Here the producer pushes: one CTA per
// local row copies the row (8 KB) into the same place of every peer's buffer with plain 16-byte
// stores over NVLink, fences, and stores the call's epoch into the row's ready word on that peer.
// The same kernel then waits, one thread per row, until every remote row of its own buffer carries
// this epoch (or a later one) -- a wait with a time limit that ends in DSA_STATUS_WAIT_TIMEOUT --
// so that the attention kernel behind it in the stream finds the whole tensor in local memory.
// Nothing is ever read from a peer's memory, and nothing on this GPU waits for another kernel of
// this GPU.  Buffers alternate with the epoch's parity on the host side: a rank can run at most one
// step ahead of a peer's attention, so it never overwrites rows that are still being read.
#include "common.cuh"
#include "ptx.cuh"
#include "tmap.cuh"

namespace dsa {

constexpr int kXchThreads = 256;
constexpr int kXchMaxWorld = 8;

struct XchPeers {
  int32_t* rows[kXchMaxWorld];    // every rank's [rows_total, row_stride] buffer (own one included)
  uint32_t* ready[kXchMaxWorld];  // every rank's [rows_total] ready words
};

namespace {

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(kXchThreads)
index_rows_exchange_kernel(XchPeers peers, int world, int rank, int rows_local, int row_offset,
                           int rows_total, int64_t row_stride, int row_width, uint32_t epoch,
                           uint64_t limit_ns, int32_t* status) {
  const int tid = threadIdx.x;
  // the local rows come from the selection kernel before us in the stream
  ptx::grid_dependency_wait();
  ptx::launch_dependents();   // the attention behind us waits for this whole kernel by itself

  // ---- push: CTA b owns local row b ----
  for (int b = blockIdx.x; b < rows_local; b += gridDim.x) {
    const size_t row_at = (size_t)(row_offset + b) * row_stride;
    const uint4* src = reinterpret_cast<const uint4*>(peers.rows[rank] + row_at);
    const int chunks = row_width / 4;   // 16-byte chunks per row
    for (int c = tid; c < chunks; c += kXchThreads) {
      const uint4 v = __ldcg(src + c);
      for (int p = 0; p < world; ++p) {
        if (p == rank) continue;
        reinterpret_cast<uint4*>(peers.rows[p] + row_at)[c] = v;
      }
    }
    __threadfence_system();
    __syncthreads();
    if (tid < world && tid != rank) st_release_sys(peers.ready[tid] + row_offset + b, epoch);
    if (tid == 0) st_release_sys(peers.ready[rank] + row_offset + b, epoch);
  }

  // ---- wait: one thread per row of the whole tensor ----
  for (int i = blockIdx.x * kXchThreads + tid; i < rows_total; i += gridDim.x * kXchThreads) {
    if (i >= row_offset && i < row_offset + rows_local) continue;   // own rows: stream order
    const uint32_t* word = peers.ready[rank] + i;
    bool ok = (int32_t)(ld_acquire_sys(word) - epoch) >= 0;
    if (!ok) {
      const uint64_t t0 = ptx::global_timer_ns();
      for (uint32_t spins = 0; !ok; ++spins) {
        ok = (int32_t)(ld_acquire_sys(word) - epoch) >= 0;
        if (!ok && (spins & 15u) == 15u) {
          if (ptx::global_timer_ns() - t0 > limit_ns) break;
          __nanosleep(200);
        }
      }
    }
    if (!ok) raise_status(status, DSA_STATUS_WAIT_TIMEOUT);
  }
}

}  // namespace

cudaError_t launch_index_rows_exchange(int32_t* const* peer_rows, uint32_t* const* peer_ready, int world,
                                       int rank, int rows_local, int row_offset, int rows_total,
                                       int64_t row_stride, int row_width, uint32_t epoch,
                                       uint64_t limit_ns, int32_t* status, cudaStream_t stream) {
  XchPeers peers = {};
  for (int p = 0; p < world; ++p) {
    peers.rows[p] = peer_rows[p];
    peers.ready[p] = peer_ready[p];
  }
  const int wait_ctas = (rows_total + kXchThreads - 1) / kXchThreads;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)max(1, max(rows_local, wait_ctas)));
  cfg.blockDim = dim3(kXchThreads);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled();
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, index_rows_exchange_kernel, peers, world, rank, rows_local, row_offset,
                            rows_total, row_stride, row_width, epoch, limit_ns, status);
}

}  // namespace dsa
