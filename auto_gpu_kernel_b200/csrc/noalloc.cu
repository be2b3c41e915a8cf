// dsa_indexer_topk_noalloc: the FP8 top-k indexer for callers that cannot allocate device memory.
//
// Who needs it: code that runs where cudaMalloc is off limits -- inside a CUDA-graph capture or a
// stream-ordered region of a serving loop whose memory pool is frozen after start-up, inside a
// plugin sandbox that only hands out the tensors of the call, or in a process whose allocator
// belongs to another runtime.  Such a caller cannot provide the score workspace that
// dsa_indexer_topk asks for, so this entry point brings its own: a fixed array in the library's
// device image.  The price is a size limit and a shared buffer (see below).
#include <atomic>

#include "common.cuh"

namespace dsa {
cudaError_t launch_indexer_score_tc(const void*, const void*, const float*, const int32_t*,
                                    const int32_t*, int64_t, float*, int64_t, int, int, int, int,
                                    uint32_t*, uint32_t*, int32_t*, cudaStream_t);
cudaError_t launch_topk_select(const float*, int64_t, const int32_t*, const int32_t*, int64_t,
                               int32_t*, int64_t, int, int, uint32_t*, int32_t*, cudaStream_t);
}  // namespace dsa

namespace {

// 2 Mi fp32 scores = 8 MiB, e.g. 64 requests x 32768 tokens.  Every GPU that loads the library
// keeps this array resident until the process exits.
constexpr size_t kNoAllocMaxScores = DSA_NOALLOC_MAX_SCORES;
static __device__ __align__(256) float g_noalloc_scores[kNoAllocMaxScores];

constexpr int kMaxDevices = 64;
// per device: device address of g_noalloc_scores (null = not yet asked); published atomically, so
// host threads making their first call at once agree on it
std::atomic<float*> g_scores_addr[kMaxDevices];

// In host code `g_noalloc_scores` is only a handle for the runtime, not a device address: the
// address a kernel can use comes from cudaGetSymbolAddress, asked once per device with that
// device current.
int scores_address(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDevices) return DSA_ERR_UNSUPPORTED;
  float* addr = g_scores_addr[dev].load(std::memory_order_acquire);
  if (addr == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scores);
    if (e != cudaSuccess) return static_cast<int>(e);
    addr = static_cast<float*>(p);
    g_scores_addr[dev].store(addr, std::memory_order_release);
  }
  *out = addr;
  return DSA_OK;
}

}  // namespace

extern "C" int dsa_indexer_topk_noalloc(const void* q_fp8, const void* k_cache, const float* weights,
                                        const int32_t* seq_lens, const int32_t* block_table,
                                        int64_t block_table_stride, int32_t* topk_out,
                                        int64_t topk_stride, int batch, int num_pages, int max_pages,
                                        int32_t* status_dev, void* stream) {
  if (batch == 0) return DSA_OK;
  if (!q_fp8 || !k_cache || !weights || !seq_lens || !block_table || !topk_out)
    return DSA_ERR_NULL_POINTER;
  if (batch < 0 || batch > 65535 || num_pages <= 0 || max_pages <= 0 || block_table_stride < 0 ||
      topk_stride < dsa::kTopK)
    return DSA_ERR_BAD_SHAPE;
  if ((reinterpret_cast<uintptr_t>(q_fp8) & 15u) || (reinterpret_cast<uintptr_t>(k_cache) & 15u))
    return DSA_ERR_MISALIGNED;
  const int64_t stride = ((int64_t)max_pages * dsa::kPage + 127) / 128 * 128;  // scores per request
  if ((uint64_t)batch * (uint64_t)stride > kNoAllocMaxScores) return DSA_ERR_SCRATCH_TOO_SMALL;
  float* scores = nullptr;
  int rc = scores_address(&scores);  // first call on a device: one cudaGetSymbolAddress, no allocation
  if (rc != DSA_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // Nothing in the scratch has to start at zero: the scorer writes every score the selection reads
  // (rows of at most 2048 tokens are neither scored nor read), so stale contents of an earlier call
  // are never observed.
  cudaError_t e = dsa::launch_indexer_score_tc(q_fp8, k_cache, weights, seq_lens, block_table,
                                               block_table_stride, scores, stride, batch, num_pages,
                                               max_pages, 1, nullptr, nullptr, status_dev, s);
  if (e != cudaSuccess) return static_cast<int>(e);
  e = dsa::launch_topk_select(scores, stride, seq_lens, block_table, block_table_stride, topk_out,
                              topk_stride, batch, max_pages, nullptr, status_dev, s);
  return static_cast<int>(e);
}
