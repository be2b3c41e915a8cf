// extern "C" boundary of libdsa_b200.so: argument checks on the host, then kernel launches on the
// caller's stream.  No allocation, no synchronisation, no exceptions cross this boundary.
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace dsa {
cudaError_t launch_indexer_score_simt(const void*, const void*, const float*, const int32_t*,
                                      const int32_t*, int64_t, float*, int64_t, int, int, int,
                                      int32_t*, cudaStream_t);
cudaError_t launch_indexer_score_tc(const void*, const void*, const float*, const int32_t*,
                                    const int32_t*, int64_t, float*, int64_t, int, int, int, int,
                                    uint32_t*, uint32_t*, int32_t*, cudaStream_t);
cudaError_t launch_topk_select_hist(const float*, int64_t, const int32_t*, const int32_t*, int64_t,
                                    int32_t*, int64_t, int, int, uint32_t*, const RowSend*, int32_t*,
                                    cudaStream_t);
bool topk_select_hist_supports(int batch, int max_pages);
cudaError_t launch_topk_select(const float*, int64_t, const int32_t*, const int32_t*, int64_t,
                               int32_t*, int64_t, int, int, uint32_t*, int32_t*, cudaStream_t);
cudaError_t launch_sparse_attn_simt(const void*, const void*, const void*, const void*,
                                    const int32_t*, int64_t, float, void*, float*, int, int, int64_t,
                                    int, void*, int32_t*, cudaStream_t);
cudaError_t launch_sparse_attn_tc(const void*, const void*, const void*, const void*,
                                  const int32_t*, int64_t, float, void*, float*, int, int, int64_t,
                                  void*, int32_t*, cudaStream_t);
size_t at_tc_workspace_bytes_auto(int tokens, int topk);
cudaError_t launch_index_rows_exchange(int32_t*, const RowSend&, int, int, int64_t, int, uint64_t, int32_t*,
                                       cudaStream_t);
cudaError_t launch_sparse_attn_mma(const void*, const void*, const void*, const void*,
                                   const int32_t*, int64_t, float, void*, float*, int, int, int64_t,
                                   void*, int32_t*, cudaStream_t);
int att_pick_splits(int tokens, int topk);
cudaError_t launch_indexer_score_prefill(const void*, const void*, const float*, const int32_t*,
                                         const int32_t*, float*, int64_t, int, int, int, int,
                                         int32_t*, cudaStream_t);
constexpr int kPrefillMinRows = 16;   // below this the per-row streaming kernel is as fast
cudaError_t launch_index_cache_write(const void*, int, int64_t, const int32_t*, void*, int, int64_t,
                                     int32_t*, cudaStream_t);
cudaError_t launch_kv_cache_append(const void*, int64_t, const void*, int64_t, const int32_t*, void*,
                                   void*, int, int64_t, int32_t*, cudaStream_t);
size_t att_workspace_bytes(int tokens, int splits);
}  // namespace dsa

namespace {
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline size_t round256(size_t n) { return (n + 255) / 256 * 256; }
// score rows are padded to a multiple of 128 tokens so a 2-page tile never crosses rows
inline int64_t score_row_stride(int max_pages) { return ((int64_t)max_pages * dsa::kPage + 127) / 128 * 128; }
}  // namespace

extern "C" {

int dsa_b200_version(void) { return DSA_B200_ABI_VERSION; }

const char* dsa_b200_error_string(int code) {
  switch (code) {
    case DSA_OK: return "ok";
    case DSA_ERR_NULL_POINTER: return "dsa_b200: null pointer argument";
    case DSA_ERR_BAD_SHAPE: return "dsa_b200: unsupported or inconsistent shape";
    case DSA_ERR_WORKSPACE_TOO_SMALL: return "dsa_b200: workspace too small";
    case DSA_ERR_MISALIGNED: return "dsa_b200: pointer or stride not 16-byte aligned";
    case DSA_ERR_UNSUPPORTED: return "dsa_b200: variant not available";
    case DSA_ERR_SCRATCH_TOO_SMALL:
      return "dsa_b200: batch x context exceeds the built-in scratch of dsa_indexer_topk_noalloc";
    default: break;
  }
  if (code > 0) return cudaGetErrorString(static_cast<cudaError_t>(code));
  return "dsa_b200: unknown error code";
}

// [ per request: max of the ordered score keys, max of their complements | per-request score
//   histograms | fp32 score rows ]
// The first two regions must be zero between calls (the kernels put back what they use), so each
// has one fixed size for every shape: no call's score rows ever land on another call's words.
constexpr size_t kMinmaxRegionBytes = 65536 * 2 * sizeof(uint32_t);   // batch <= 65535
constexpr size_t kScoreRowsOffset = kMinmaxRegionBytes + dsa::kHistRegionBytes;
size_t dsa_indexer_workspace_bytes(int batch, int max_pages) {
  if (batch <= 0 || max_pages <= 0) return 256;
  return kScoreRowsOffset + round256((size_t)batch * score_row_stride(max_pages) * sizeof(float));
}

// How dsa_indexer_topk scores and selects long rows (decode shapes, batch <= 1024):
//   "hist"   (default) the scorer also builds every request's score histogram; the selection
//            kernel starts from it (boundary bin, one counting and one writing sweep);
//   "minmax" the scorer hands over each row's min / max, the selection builds its own histogram
//            over the linear map of that range (also what larger batches and the shared-pages
//            scorer use).
// DSA_INDEXER_PATH in the environment picks one; read on every call so that a test can compare
// the paths in one process.
enum IndexerPath { kPathHist, kPathMinmax };
static IndexerPath indexer_path() {
  const char* e = getenv("DSA_INDEXER_PATH");
  return (e != nullptr && e[0] == 'm') ? kPathMinmax : kPathHist;
}

static int scores_impl(const void* q_fp8, const void* k_cache, const float* weights,
                       const int32_t* seq_lens, const int32_t* block_table,
                       int64_t block_table_stride, float* scores, int64_t score_stride, int batch,
                       int num_pages, int max_pages, int variant, int skip_short, uint32_t* minmax,
                       uint32_t* ghist, int32_t* status_dev, void* stream) {
  if (batch == 0) return DSA_OK;
  if (!q_fp8 || !k_cache || !weights || !seq_lens || !block_table || !scores)
    return DSA_ERR_NULL_POINTER;
  if (batch < 0 || batch > 65535 || num_pages <= 0 || max_pages <= 0 || block_table_stride < 0 ||
      score_stride < (int64_t)max_pages * dsa::kPage)
    return DSA_ERR_BAD_SHAPE;
  if (!aligned16(q_fp8) || !aligned16(k_cache) || !aligned16(scores) || (score_stride & 3))
    return DSA_ERR_MISALIGNED;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (variant == 1) {
    e = dsa::launch_indexer_score_simt(q_fp8, k_cache, weights, seq_lens, block_table,
                                       block_table_stride, scores, score_stride, batch, num_pages,
                                       max_pages, status_dev, s);
  } else if (variant == 0 && block_table_stride == 0 && batch >= dsa::kPrefillMinRows) {
    // every row reads the same pages (chunked prefill): four rows share each tcgen05.mma
    e = dsa::launch_indexer_score_prefill(q_fp8, k_cache, weights, seq_lens, block_table, scores,
                                          score_stride, batch, num_pages, max_pages, skip_short,
                                          status_dev, s);
  } else if (variant == 0 || variant == 2) {
    e = dsa::launch_indexer_score_tc(q_fp8, k_cache, weights, seq_lens, block_table,
                                     block_table_stride, scores, score_stride, batch, num_pages,
                                     max_pages, skip_short, minmax, ghist, status_dev, s);
  } else {
    return DSA_ERR_UNSUPPORTED;
  }
  return static_cast<int>(e);
}

int dsa_indexer_scores(const void* q_fp8, const void* k_cache, const float* weights,
                       const int32_t* seq_lens, const int32_t* block_table,
                       int64_t block_table_stride, float* scores, int64_t score_stride, int batch,
                       int num_pages, int max_pages, int variant, int32_t* status_dev,
                       void* stream) {
  return scores_impl(q_fp8, k_cache, weights, seq_lens, block_table, block_table_stride, scores,
                     score_stride, batch, num_pages, max_pages, variant, 0, nullptr, nullptr, status_dev,
                     stream);
}

int dsa_topk_select(const float* scores, int64_t score_stride, const int32_t* seq_lens,
                    const int32_t* block_table, int64_t block_table_stride, int32_t* topk_out,
                    int64_t topk_stride, int batch, int max_pages, int32_t* status_dev,
                    void* stream) {
  if (batch == 0) return DSA_OK;
  if (!scores || !seq_lens || !block_table || !topk_out) return DSA_ERR_NULL_POINTER;
  if (batch < 0 || max_pages <= 0 || topk_stride < dsa::kTopK || block_table_stride < 0)
    return DSA_ERR_BAD_SHAPE;
  return static_cast<int>(dsa::launch_topk_select(scores, score_stride, seq_lens, block_table,
                                                  block_table_stride, topk_out, topk_stride, batch,
                                                  max_pages, nullptr, status_dev,
                                                  static_cast<cudaStream_t>(stream)));
}

// `send` (may be null): where finished rows go in a head-sharded layer.  *sent tells whether the
// selection kernel has sent them itself (the histogram path) or the caller still has to.
static int indexer_topk_impl(const void* q_fp8, const void* k_cache, const float* weights,
                             const int32_t* seq_lens, const int32_t* block_table,
                             int64_t block_table_stride, int32_t* topk_out, int64_t topk_stride, int batch,
                             int num_pages, int max_pages, void* workspace, size_t workspace_bytes,
                             int32_t* status_dev, void* stream, const dsa::RowSend* send, bool* sent) {
  if (sent) *sent = false;
  if (batch == 0) return DSA_OK;
  if (!workspace) return DSA_ERR_NULL_POINTER;
  if (workspace_bytes < dsa_indexer_workspace_bytes(batch, max_pages))
    return DSA_ERR_WORKSPACE_TOO_SMALL;
  if (reinterpret_cast<uintptr_t>(workspace) & 255u) return DSA_ERR_MISALIGNED;
  if (batch > 65535) return DSA_ERR_BAD_SHAPE;
  float* scores = reinterpret_cast<float*>(static_cast<char*>(workspace) + kScoreRowsOffset);
  const int64_t stride = score_row_stride(max_pages);
  // The streaming scorer leaves every row's min / max in front of the score rows (the words start
  // at zero and the selection puts them back to zero); the shared-pages scorer does not.
  const bool shared_pages = block_table_stride == 0 && batch >= dsa::kPrefillMinRows;
  uint32_t* minmax = shared_pages ? nullptr : static_cast<uint32_t*>(workspace);
  const bool long_rows = (int64_t)max_pages * dsa::kPage > dsa::kTopK;
  const IndexerPath path = indexer_path();
  uint32_t* ghist = reinterpret_cast<uint32_t*>(static_cast<char*>(workspace) + kMinmaxRegionBytes);
  // rows of at most 2048 tokens are emitted whole by the selection: their scores are skipped, and
  // when no row can be longer (max_pages <= 32) the scorer is not launched at all (the reference's
  // GPU dispatch takes the same shortcut from the shape alone, indexer_fused.py:358-380)
  if (long_rows && !shared_pages && path != kPathMinmax &&
      dsa::topk_select_hist_supports(batch, max_pages)) {
    if (!topk_out) return DSA_ERR_NULL_POINTER;
    if (topk_stride < dsa::kTopK) return DSA_ERR_BAD_SHAPE;
    int rc = scores_impl(q_fp8, k_cache, weights, seq_lens, block_table, block_table_stride, scores,
                         stride, batch, num_pages, max_pages, 0, 1, nullptr, ghist, status_dev, stream);
    if (rc != DSA_OK) return rc;
    if (sent) *sent = send != nullptr;
    return static_cast<int>(dsa::launch_topk_select_hist(
        scores, stride, seq_lens, block_table, block_table_stride, topk_out, topk_stride, batch,
        max_pages, ghist, send, status_dev, static_cast<cudaStream_t>(stream)));
  }
  if (long_rows) {
    int rc = scores_impl(q_fp8, k_cache, weights, seq_lens, block_table, block_table_stride, scores,
                         stride, batch, num_pages, max_pages, 0, 1, minmax, nullptr, status_dev, stream);
    if (rc != DSA_OK) return rc;
  } else if (!q_fp8 || !k_cache || !weights || !seq_lens || !block_table) {
    return DSA_ERR_NULL_POINTER;
  }
  if (!seq_lens || !block_table || !topk_out) return DSA_ERR_NULL_POINTER;
  if (max_pages <= 0 || topk_stride < dsa::kTopK || block_table_stride < 0) return DSA_ERR_BAD_SHAPE;
  return static_cast<int>(dsa::launch_topk_select(scores, stride, seq_lens, block_table,
                                                  block_table_stride, topk_out, topk_stride, batch,
                                                  max_pages, minmax, status_dev,
                                                  static_cast<cudaStream_t>(stream)));
}

int dsa_indexer_topk(const void* q_fp8, const void* k_cache, const float* weights,
                     const int32_t* seq_lens, const int32_t* block_table,
                     int64_t block_table_stride, int32_t* topk_out, int64_t topk_stride, int batch,
                     int num_pages, int max_pages, void* workspace, size_t workspace_bytes,
                     int32_t* status_dev, void* stream) {
  return indexer_topk_impl(q_fp8, k_cache, weights, seq_lens, block_table, block_table_stride, topk_out,
                           topk_stride, batch, num_pages, max_pages, workspace, workspace_bytes,
                           status_dev, stream, nullptr, nullptr);
}

static int fill_row_send(dsa::RowSend* xs, void* const* peer_stage, int world, int rank, int row_offset,
                         int row_width, uint32_t epoch) {
  if (!peer_stage) return DSA_ERR_NULL_POINTER;
  if (world < 1 || world > dsa::kRowSendMaxWorld || rank < 0 || rank >= world || row_offset < 0 ||
      row_width <= 0 || row_width % 2 != 0 || epoch == 0)
    return DSA_ERR_BAD_SHAPE;
  *xs = dsa::RowSend{};
  for (int p = 0; p < world; ++p) {
    if (!peer_stage[p]) return DSA_ERR_NULL_POINTER;
    if (!aligned16(peer_stage[p])) return DSA_ERR_MISALIGNED;
    xs->stage[p] = static_cast<uint2*>(peer_stage[p]);
  }
  xs->world = world;
  xs->rank = rank;
  xs->row_offset = row_offset;
  xs->row_width = row_width;
  xs->epoch = epoch;
  return DSA_OK;
}

int dsa_indexer_topk_send(const void* q_fp8, const void* k_cache, const float* weights,
                          const int32_t* seq_lens, const int32_t* block_table,
                          int64_t block_table_stride, int32_t* topk_out, int64_t topk_stride, int batch,
                          int num_pages, int max_pages, void* workspace, size_t workspace_bytes,
                          void* const* peer_stage, int world, int rank, int row_offset, uint32_t epoch,
                          int32_t* status_dev, void* stream) {
  dsa::RowSend xs;
  int rc = fill_row_send(&xs, peer_stage, world, rank, row_offset, dsa::kTopK, epoch);
  if (rc != DSA_OK) return rc;
  if (topk_stride % 2 != 0 || (reinterpret_cast<uintptr_t>(topk_out) & 7u)) return DSA_ERR_MISALIGNED;
  bool sent = false;
  rc = indexer_topk_impl(q_fp8, k_cache, weights, seq_lens, block_table, block_table_stride, topk_out,
                         topk_stride, batch, num_pages, max_pages, workspace, workspace_bytes, status_dev,
                         stream, &xs, &sent);
  if (rc != DSA_OK || sent || batch == 0 || world == 1) return rc;
  // the other selection kernels do not send: a push-only pass over the finished rows
  int32_t* base = topk_out - (int64_t)row_offset * topk_stride;   // row i of the exchange = base + i * stride
  return static_cast<int>(dsa::launch_index_rows_exchange(base, xs, batch, row_offset + batch, topk_stride, 1,
                                                          1, status_dev, static_cast<cudaStream_t>(stream)));
}

size_t dsa_sparse_attn_workspace_bytes(int tokens, int heads, int topk) {
  if (tokens <= 0 || heads != dsa::kHeads || topk <= 0) return 256;
  size_t a = dsa::att_workspace_bytes(tokens, dsa::att_pick_splits(tokens, topk));
  size_t b = dsa::at_tc_workspace_bytes_auto(tokens, topk);
  return round256(a > b ? a : b);
}

static int attn_impl(const void* q_nope, const void* q_pe, const void* ckv, const void* kpe,
                     const int32_t* sparse_indices, int64_t index_stride, float sm_scale, void* out,
                     float* lse, int tokens, int heads, int topk, int64_t num_slots, void* workspace,
                     size_t workspace_bytes, int32_t* status_dev, void* stream, int variant) {
  if (tokens == 0) return DSA_OK;
  if (!q_nope || !q_pe || !ckv || !kpe || !sparse_indices || !out || !lse || !workspace)
    return DSA_ERR_NULL_POINTER;
  if (tokens < 0 || heads != dsa::kHeads || topk <= 0 || num_slots <= 0 || index_stride < topk)
    return DSA_ERR_BAD_SHAPE;
  if (!aligned16(q_nope) || !aligned16(q_pe) || !aligned16(ckv) || !aligned16(kpe) ||
      !aligned16(out) || (reinterpret_cast<uintptr_t>(workspace) & 255u))
    return DSA_ERR_MISALIGNED;
  if (workspace_bytes < dsa_sparse_attn_workspace_bytes(tokens, heads, topk))
    return DSA_ERR_WORKSPACE_TOO_SMALL;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (variant == 1) {
    const int splits = dsa::att_pick_splits(tokens, topk);
    return static_cast<int>(dsa::launch_sparse_attn_simt(q_nope, q_pe, ckv, kpe, sparse_indices,
                                                         index_stride, sm_scale, out, lse, tokens,
                                                         topk, num_slots, splits, workspace,
                                                         status_dev, s));
  }
  if (variant == 2) {
    return static_cast<int>(dsa::launch_sparse_attn_tc(q_nope, q_pe, ckv, kpe, sparse_indices,
                                                       index_stride, sm_scale, out, lse, tokens,
                                                       topk, num_slots, workspace, status_dev, s));
  }
  return static_cast<int>(dsa::launch_sparse_attn_mma(q_nope, q_pe, ckv, kpe, sparse_indices,
                                                      index_stride, sm_scale, out, lse, tokens, topk,
                                                      num_slots, workspace, status_dev, s));
}

int dsa_sparse_attn(const void* q_nope, const void* q_pe, const void* ckv, const void* kpe,
                    const int32_t* sparse_indices, int64_t index_stride, float sm_scale, void* out,
                    float* lse, int tokens, int heads, int topk, int64_t num_slots, void* workspace,
                    size_t workspace_bytes, int32_t* status_dev, void* stream) {
  return attn_impl(q_nope, q_pe, ckv, kpe, sparse_indices, index_stride, sm_scale, out, lse, tokens,
                   heads, topk, num_slots, workspace, workspace_bytes, status_dev, stream, 0);
}

int dsa_sparse_attn_cuda_core(const void* q_nope, const void* q_pe, const void* ckv,
                              const void* kpe, const int32_t* sparse_indices, int64_t index_stride,
                              float sm_scale, void* out, float* lse, int tokens, int heads, int topk,
                              int64_t num_slots, void* workspace, size_t workspace_bytes,
                              int32_t* status_dev, void* stream) {
  return attn_impl(q_nope, q_pe, ckv, kpe, sparse_indices, index_stride, sm_scale, out, lse, tokens,
                   heads, topk, num_slots, workspace, workspace_bytes, status_dev, stream, 1);
}

int dsa_sparse_attn_tcgen05(const void* q_nope, const void* q_pe, const void* ckv, const void* kpe,
                            const int32_t* sparse_indices, int64_t index_stride, float sm_scale,
                            void* out, float* lse, int tokens, int heads, int topk,
                            int64_t num_slots, void* workspace, size_t workspace_bytes,
                            int32_t* status_dev, void* stream) {
  return attn_impl(q_nope, q_pe, ckv, kpe, sparse_indices, index_stride, sm_scale, out, lse, tokens,
                   heads, topk, num_slots, workspace, workspace_bytes, status_dev, stream, 2);
}

// ---- buffers that the GPUs of one host can address in each other's memory (CUDA IPC) ----------
int dsa_peer_slab_create(size_t bytes, void** ptr, void* handle64) {
  if (!ptr || !handle64 || bytes == 0) return DSA_ERR_NULL_POINTER;
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaMemset(p, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return static_cast<int>(e);
  }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  memcpy(handle64, &h, 64);
  *ptr = p;
  return DSA_OK;
}

int dsa_peer_slab_open(const void* handle64, void** ptr) {
  if (!ptr || !handle64) return DSA_ERR_NULL_POINTER;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  // opened with the CALLER's device current: peer access from it to the owner is enabled with it
  return static_cast<int>(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
}

int dsa_peer_slab_close(void* ptr) {
  return ptr ? static_cast<int>(cudaIpcCloseMemHandle(ptr)) : DSA_OK;
}

int dsa_peer_slab_destroy(void* ptr) { return ptr ? static_cast<int>(cudaFree(ptr)) : DSA_OK; }

int dsa_index_rows_exchange(int32_t* rows, void* const* peer_stage, int world, int rank, int rows_local,
                            int row_offset, int rows_total, int64_t row_stride, int row_width,
                            uint32_t epoch, int mode, uint64_t wait_limit_ns, int32_t* status_dev,
                            void* stream) {
  if (!rows) return DSA_ERR_NULL_POINTER;
  dsa::RowSend xs;
  int rc = fill_row_send(&xs, peer_stage, world, rank, row_offset, row_width, epoch);
  if (rc != DSA_OK) return rc;
  if (rows_local < 0 || rows_total < row_offset + rows_local || row_stride < row_width ||
      row_stride % 2 != 0 || mode < 1 || mode > 3 || wait_limit_ns == 0 ||
      wait_limit_ns > 10000000000ull)
    return DSA_ERR_BAD_SHAPE;
  if (reinterpret_cast<uintptr_t>(rows) & 7u) return DSA_ERR_MISALIGNED;
  if (rows_total == 0) return DSA_OK;
  return static_cast<int>(dsa::launch_index_rows_exchange(rows, xs, rows_local, rows_total, row_stride,
                                                          mode, wait_limit_ns, status_dev,
                                                          static_cast<cudaStream_t>(stream)));
}

int dsa_index_cache_write(const void* keys, int key_dtype, int64_t key_stride, const int32_t* slots,
                          void* k_cache, int tokens, int num_pages, int32_t* status_dev,
                          void* stream) {
  if (tokens == 0) return DSA_OK;
  if (!keys || !slots || !k_cache) return DSA_ERR_NULL_POINTER;
  if (tokens < 0 || num_pages <= 0 || key_stride < dsa::kIdxDim || (key_dtype != 0 && key_dtype != 1))
    return DSA_ERR_BAD_SHAPE;
  const int64_t elem = key_dtype == 0 ? 4 : 2;
  if (!aligned16(keys) || (key_stride * elem) % 16 != 0 || !aligned16(k_cache))
    return DSA_ERR_MISALIGNED;
  return static_cast<int>(dsa::launch_index_cache_write(
      keys, key_dtype, key_stride, slots, k_cache, tokens,
      static_cast<int64_t>(num_pages) * dsa::kPage, status_dev, static_cast<cudaStream_t>(stream)));
}

int dsa_kv_cache_append(const void* ckv, int64_t ckv_stride, const void* kpe, int64_t kpe_stride,
                        const int32_t* slots, void* ckv_cache, void* kpe_cache, int tokens,
                        int64_t num_slots, int32_t* status_dev, void* stream) {
  if (tokens == 0) return DSA_OK;
  if (!ckv || !kpe || !slots || !ckv_cache || !kpe_cache) return DSA_ERR_NULL_POINTER;
  if (tokens < 0 || num_slots <= 0 || ckv_stride < dsa::kCkv || kpe_stride < dsa::kKpe)
    return DSA_ERR_BAD_SHAPE;
  if (!aligned16(ckv) || !aligned16(kpe) || !aligned16(ckv_cache) || !aligned16(kpe_cache) ||
      ckv_stride % 8 != 0 || kpe_stride % 8 != 0)
    return DSA_ERR_MISALIGNED;
  return static_cast<int>(dsa::launch_kv_cache_append(ckv, ckv_stride, kpe, kpe_stride, slots,
                                                      ckv_cache, kpe_cache, tokens, num_slots,
                                                      status_dev, static_cast<cudaStream_t>(stream)));
}

}  // extern "C"
