/*
 * dsa_b200 -- C ABI of the B200 (sm_100a) DeepSeek Sparse Attention hot path.
 *
 * The reference repository (Dogacel/auto-gpu-kernel) has no native code: its hot path is the pair
 * of Python entry points `kernel(...)` that flashinfer-bench calls with CUDA tensors.  Each entry
 * point below states which Python interface of the reference it stands behind.  All pointers are
 * DEVICE pointers unless a name ends in `_host`; the caller owns every buffer; nothing is allocated
 * per call; work is enqueued on `stream` (a cudaStream_t passed as void*) and the call returns
 * without synchronising.
 *
 * Return value: 0 = enqueued; negative = argument error found on the host (DSA_ERR_*); positive =
 * a cudaError_t raised by a launch.  Faults found on the device (a bounded wait that ran out, an
 * out-of-range page id in a checked build) are OR-ed into the int32 word `status_dev` points to
 * (may be NULL); the caller reads it when it chooses to synchronise.
 */
#ifndef DSA_B200_H_
#define DSA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DSA_B200_ABI_VERSION 1

#define DSA_PAGE_SIZE 64
#define DSA_INDEX_HEADS 64
#define DSA_INDEX_DIM 128
#define DSA_INDEX_PAGE_BYTES 8448 /* 64*128 e4m3 bytes, then 64 fp32 scales */
#define DSA_TOPK 2048
#define DSA_ATTN_HEADS 16
#define DSA_CKV_DIM 512
#define DSA_KPE_DIM 64

enum {
  DSA_OK = 0,
  DSA_ERR_NULL_POINTER = -1,
  DSA_ERR_BAD_SHAPE = -2,
  DSA_ERR_WORKSPACE_TOO_SMALL = -3,
  DSA_ERR_MISALIGNED = -4,
  DSA_ERR_UNSUPPORTED = -5,
  DSA_ERR_SCRATCH_TOO_SMALL = -6 /* dsa_indexer_topk_noalloc: batch x padded context > built-in scratch */
};

/* bits OR-ed into *status_dev by kernels */
#define DSA_STATUS_WAIT_TIMEOUT 0x1u   /* a bounded mbarrier / flag wait gave up */
#define DSA_STATUS_BAD_PAGE     0x2u   /* block_table entry outside [0, num_pages) (skipped) */
#define DSA_STATUS_BAD_SLOT     0x4u   /* sparse index outside [0, num_slots) (treated as -1) */
#define DSA_STATUS_TOPK_COUNT   0x8u   /* selection wrote a number of ids != min(2048, len) */

/* ABI version of the loaded library (DSA_B200_ABI_VERSION at build time). */
int dsa_b200_version(void);

/* Static text for a DSA_ERR_* code or a cudaError_t value returned by the calls below. */
const char* dsa_b200_error_string(int code);

/* ---------------------------------------------------------------------------------------------
 * FP8 top-k indexer.  Stands behind the reference's
 *   kernel(q_index_fp8, k_index_cache_fp8, weights, seq_lens, block_table, topk_indices)
 * (archive/dsa_topk_indexer_fp8_h64_d128_topk2048_ps64/solution/triton/indexer_baseline.py:39-90;
 *  GPU dispatch it replaces: .../indexer_fused.py:331-412).
 *
 *   q_fp8        [batch,64,128] e4m3, contiguous
 *   k_cache      [num_pages] pages of DSA_INDEX_PAGE_BYTES bytes (the [P,64,1,132] int8 tensor)
 *   weights      [batch,64] fp32, contiguous
 *   seq_lens     [batch] int32
 *   block_table  [batch,max_pages] int32, row stride `block_table_stride` elements (0 = every
 *                request shares one row: chunked prefill)
 *   topk_out     [batch,2048] int32, row stride `topk_stride` elements; receives
 *                min(2048,seq_len) global slot ids (page*64+offset) then -1
 *   workspace    >= dsa_indexer_workspace_bytes(batch,max_pages) bytes, 256-byte aligned, zero-filled
 *                once when created: two words per request (min / max of the row; 512 KB whatever
 *                the batch), then 1024 score histograms of 4096 words (16 MB whatever the batch),
 *                then the fp32 score rows.  The scorer leaves either the row's histogram (decode
 *                shapes up to 1024 requests) or its min / max for the selection, which puts what
 *                it used back to zero; the histograms must be zero when a call starts
 * ------------------------------------------------------------------------------------------- */
size_t dsa_indexer_workspace_bytes(int batch, int max_pages);

int dsa_indexer_topk(const void* q_fp8, const void* k_cache, const float* weights,
                     const int32_t* seq_lens, const int32_t* block_table,
                     int64_t block_table_stride, int32_t* topk_out, int64_t topk_stride,
                     int batch, int num_pages, int max_pages, void* workspace,
                     size_t workspace_bytes, int32_t* status_dev, void* stream);

/* The same indexer for callers that cannot allocate device memory (no counterpart in the
 * reference: its callers always own an allocator).  Use it from places where cudaMalloc is not an
 * option -- a frozen memory pool of a serving loop, a plugin that may only touch the tensors it was
 * handed, a process whose allocator belongs to another runtime -- and the score workspace of
 * dsa_indexer_topk therefore cannot be provided.  The scores go to a fixed array inside the
 * library's device image instead (DSA_NOALLOC_MAX_SCORES fp32 values = 8 MiB, resident on every
 * GPU that loads the library until the process exits).
 *   - limit: batch * round_up(max_pages * 64, 128) <= DSA_NOALLOC_MAX_SCORES, e.g. 64 requests of
 *     32768 tokens; larger calls return DSA_ERR_SCRATCH_TOO_SMALL and launch nothing;
 *   - the call allocates nothing: no cudaMalloc/cudaFree, no allocating library routine;
 *   - the first call on each device looks the array's device address up once
 *     (cudaGetSymbolAddress); make that first call outside any stream capture;
 *   - every call on a device shares the one array: two calls that overlap on the GPU (different
 *     streams, no dependency) race on it and corrupt each other's result; calls on one stream, or
 *     ordered by events, are fine.  The array keeps the previous call's scores; nothing relies on
 *     its initial contents.
 * Arguments as for dsa_indexer_topk, minus the workspace. */
#define DSA_NOALLOC_MAX_SCORES (2u * 1024u * 1024u)
int dsa_indexer_topk_noalloc(const void* q_fp8, const void* k_cache, const float* weights,
                             const int32_t* seq_lens, const int32_t* block_table,
                             int64_t block_table_stride, int32_t* topk_out, int64_t topk_stride,
                             int batch, int num_pages, int max_pages, int32_t* status_dev,
                             void* stream);

/* Stage 1 alone: fp32 score rows, scores[b*score_stride + t] for t < seq_len[b] (the quantity
 * `final_scores` of indexer_baseline.py:80).  Entries t >= seq_len[b] are left untouched.
 * `variant`: 0 = tensor-core (tcgen05) scorer -- the streaming kernel (one row per product), or,
 * when block_table_stride == 0 and batch >= 16 (chunked prefill: every row reads the same pages),
 * the kernel that shares each key tile among eight rows; 1 = plain CUDA-core scorer kept as an
 * on-device cross-check; 2 = the streaming tcgen05 kernel whatever the shape. */
int dsa_indexer_scores(const void* q_fp8, const void* k_cache, const float* weights,
                       const int32_t* seq_lens, const int32_t* block_table,
                       int64_t block_table_stride, float* scores, int64_t score_stride,
                       int batch, int num_pages, int max_pages, int variant,
                       int32_t* status_dev, void* stream);

/* Stage 2 alone: top-2048 selection + page remap over given fp32 score rows
 * (torch.topk + remap of indexer_baseline.py:82-90). */
int dsa_topk_select(const float* scores, int64_t score_stride, const int32_t* seq_lens,
                    const int32_t* block_table, int64_t block_table_stride, int32_t* topk_out,
                    int64_t topk_stride, int batch, int max_pages, int32_t* status_dev,
                    void* stream);

/* ---------------------------------------------------------------------------------------------
 * Sparse MLA attention.  Stands behind the reference's
 *   kernel(q_nope, q_pe, ckv_cache, kpe_cache, sparse_indices, sm_scale, output, lse)
 * (archive/dsa_sparse_attention_h16_ckv512_kpe64_topk2048_ps64/solution/triton/
 *  sparse_baseline.py:12-45; GPU dispatch it replaces: .../sparse_fused.py:305-375).
 *
 *   q_nope  [tokens,heads,512] bf16   q_pe [tokens,heads,64] bf16      (contiguous)
 *   ckv     [num_slots,512] bf16      kpe  [num_slots,64] bf16         (flat paged caches)
 *   sparse_indices [tokens,topk] int32, row stride `index_stride`; -1 = masked
 *   out     [tokens,heads,512] bf16   lse [tokens,heads] fp32 (base-2 log-sum-exp)
 * A row with no valid index gets out = 0 and lse = -inf.  `heads` must be 16.
 * ------------------------------------------------------------------------------------------- */
size_t dsa_sparse_attn_workspace_bytes(int tokens, int heads, int topk);

int dsa_sparse_attn(const void* q_nope, const void* q_pe, const void* ckv, const void* kpe,
                    const int32_t* sparse_indices, int64_t index_stride, float sm_scale,
                    void* out, float* lse, int tokens, int heads, int topk, int64_t num_slots,
                    void* workspace, size_t workspace_bytes, int32_t* status_dev, void* stream);

/* Same contract as dsa_sparse_attn (which runs the warp-level mma.sync kernel: with 16 heads it is
 * the fastest formulation on B200), computed with the tcgen05/TMEM kernel that issues the
 * products transposed (heads as N = 16).  Same reference interface; kept selectable because it is
 * the formulation that wins once more heads share a gathered row. */
int dsa_sparse_attn_tcgen05(const void* q_nope, const void* q_pe, const void* ckv, const void* kpe,
                            const int32_t* sparse_indices, int64_t index_stride, float sm_scale,
                            void* out, float* lse, int tokens, int heads, int topk,
                            int64_t num_slots, void* workspace, size_t workspace_bytes,
                            int32_t* status_dev, void* stream);

/* Same contract as dsa_sparse_attn, computed with plain CUDA-core FMAs: an on-device cross-check
 * at sizes where the CPU oracle is slow.  Same reference interface. */
int dsa_sparse_attn_cuda_core(const void* q_nope, const void* q_pe, const void* ckv,
                              const void* kpe, const int32_t* sparse_indices, int64_t index_stride,
                              float sm_scale, void* out, float* lse, int tokens, int heads, int topk,
                              int64_t num_slots, void* workspace, size_t workspace_bytes,
                              int32_t* status_dev, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Cache writers: the producers of the two paged caches, run on the step before the path.
 * The reference has no writer (its inputs arrive packed); the layouts are the ones its readers
 * unpack: index-key pages by dequant_fp8_kv_cache (archive/dsa_topk_indexer_fp8_h64_d128_topk2048_ps64/
 * solution/triton/indexer_baseline.py:16-36; layout notes in that directory's CLAUDE.md:65), ckv/kpe
 * rows by the flat views of .../sparse_baseline.py:18-28.
 *
 * dsa_index_cache_write: per token t with slot = slots[t] (page * 64 + position; -1 = skip):
 *   scale = max(max_d |key[t,d]|, 1e-12) / 448;  byte[d] = e4m3(key[t,d] / scale) (round to nearest
 *   even, saturating);  the 128 bytes go to page*8448 + position*128, the fp32 scale to
 *   page*8448 + 8192 + position*4.
 *   keys [tokens,128], row stride `key_stride` elements, key_dtype 0 = fp32, 1 = bf16.
 * dsa_kv_cache_append: ckv_cache[slot,:] = ckv[t,:] (512 bf16), kpe_cache[slot,:] = kpe[t,:]
 *   (64 bf16); row strides in elements (multiples of 8).
 * Slots outside the cache are skipped and reported as DSA_STATUS_BAD_SLOT.  Two tokens with the
 * same slot in one call race (the result is one of them).
 * ------------------------------------------------------------------------------------------- */
int dsa_index_cache_write(const void* keys, int key_dtype, int64_t key_stride, const int32_t* slots,
                          void* k_cache, int tokens, int num_pages, int32_t* status_dev,
                          void* stream);

int dsa_kv_cache_append(const void* ckv, int64_t ckv_stride, const void* kpe, int64_t kpe_stride,
                        const int32_t* slots, void* ckv_cache, void* kpe_cache, int tokens,
                        int64_t num_slots, int32_t* status_dev, void* stream);

/* ---------------------------------------------------------------------------------------------
 * One decode step with HOST buffers: copies in, dsa_indexer_topk, dsa_sparse_attn over the
 * indexer's own indices, copies out, synchronised on return.  No counterpart in the reference,
 * whose callers pass CUDA tensors (kbench/flashinfer.py:109-120); it replaces the nine copies and
 * two operator calls such a caller would issue itself.
 *
 * host_in / dev_in : one pinned slab and its device mirror,
 *     [ indexer inputs: in_indexer_bytes ][ attention inputs: in_attention_bytes ];
 *     q_index_fp8, weights, seq_lens, block_table point into the first part of dev_in, q_nope and
 *     q_pe into the second (any 16-byte aligned packing).
 * host_out / dev_out : [ output | lse : out_attention_bytes ][ topk_indices : out_indices_bytes ];
 *     output, lse and topk_indices point into dev_out accordingly (topk rows dense, stride 2048).
 * Caches, workspaces and status word as for the two operator calls.  `stream` carries the kernels,
 * `side_stream` the overlapped copies; the three events are the caller's (created once, reused).
 * ------------------------------------------------------------------------------------------- */
typedef struct dsa_host_step_args {
  const void* host_in;
  void* dev_in;
  size_t in_indexer_bytes, in_attention_bytes;
  void* host_out;
  const void* dev_out;
  size_t out_attention_bytes, out_indices_bytes;
  /* device views into dev_in / dev_out */
  const void* q_index_fp8;
  const float* weights;
  const int32_t* seq_lens;
  const int32_t* block_table;
  int64_t block_table_stride;
  const void* q_nope;
  const void* q_pe;
  void* output;
  float* lse;
  int32_t* topk_indices;
  /* device-resident state */
  const void* k_index_cache;
  const void* ckv_cache;
  const void* kpe_cache;
  int batch, num_pages, max_pages;
  int64_t num_slots;
  float sm_scale;
  void* indexer_workspace;
  size_t indexer_workspace_bytes;
  void* attention_workspace;
  size_t attention_workspace_bytes;
  int32_t* status_dev;
  void* stream;
  void* side_stream;
  void* ev_first_copy;
  void* ev_q_ready;
  void* ev_indices_ready;
} dsa_host_step_args;

int dsa_decode_step_host(const dsa_host_step_args* args);

/* Device buffers that the other GPUs of the host can address (no counterpart in the reference).
 * The library allocates nothing on its own; these four calls are the explicit exception, made by
 * the caller once when a head-sharded layer is set up.  `create` allocates `bytes` of zeroed device
 * memory on the current device and writes its 64-byte CUDA IPC handle to `handle64`; the handle
 * travels to the peer processes by whatever channel the caller has; `open`, made there with the
 * peer's own device current, returns the address of that memory as seen from it (peer access to the
 * owner is enabled with it); `close` unmaps it; `destroy` frees the owner's memory, after every peer
 * has closed it.  One process per GPU.  Return values as everywhere: 0, DSA_ERR_*, or cudaError_t. */
int dsa_peer_slab_create(size_t bytes, void** ptr, void* handle64);
int dsa_peer_slab_open(const void* handle64, void** ptr);
int dsa_peer_slab_close(void* ptr);
int dsa_peer_slab_destroy(void* ptr);

/* Exchange of index rows between the GPUs of a head-sharded layer (no counterpart in the reference,
 * which is single-GPU: its operators meet only through the index tensor, indexer_baseline.py:82-90 ->
 * sparse_baseline.py:22-28).  `rows` is the caller's own [rows_total][row_stride] int32 index tensor
 * (ordinary device memory) whose rows [row_offset, row_offset + rows_local) the selection has just
 * written.  Every rank also owns a staging buffer of rows_total x row_width 8-byte (id, epoch)
 * pairs, zero when created, that its peers can address (dsa_peer_slab_create / _open);
 * `peer_stage` is a HOST array of `world` device pointers to those buffers as seen from this GPU
 * (entry `rank`: the caller's own).  One kernel stores the local rows as pairs into the same rows
 * of every peer's staging buffer (plain 16-byte stores; nothing is read from a peer), and polls
 * the other rows of its own staging buffer until every pair carries `epoch`, writing the ids into
 * `rows`.  When it has completed, `rows` holds all rows_total rows.  `epoch` (never 0) must differ
 * from the epoch of the call two steps earlier on every rank: count calls from 1.  Use two staging
 * buffers alternately (by the epoch's parity): a rank can run one step ahead of a peer, not two.
 * The poll ends after `wait_limit_ns` (1 .. 1e10) with DSA_STATUS_WAIT_TIMEOUT in *status_dev and
 * the rows it could not complete left as they were; the context stays usable.  `mode`: 1 = only
 * store the local rows (push), 2 = only take the peers' rows (after dsa_indexer_topk_send, which has
 * sent the local ones), 3 = both.  row_width and row_stride even, `rows` 8-byte aligned.  One
 * process per GPU; never run two ranks on one GPU at the same time. */
int dsa_index_rows_exchange(int32_t* rows, void* const* peer_stage, int world, int rank, int rows_local,
                            int row_offset, int rows_total, int64_t row_stride, int row_width,
                            uint32_t epoch, int mode, uint64_t wait_limit_ns, int32_t* status_dev,
                            void* stream);

/* dsa_indexer_topk for a rank of a head-sharded layer: the same call (same arguments, same results in
 * `topk_out`, which here is the rank's slice -- rows [row_offset, row_offset + batch) -- of its
 * [rows_total][topk_stride] index tensor), and in addition every finished row is stored as
 * (id, epoch) pairs into row row_offset + b of every peer's staging buffer (`peer_stage`, `world`,
 * `rank`, `epoch` as for dsa_index_rows_exchange; row width 2048).  On decode shapes the selection
 * kernel sends each row itself as soon as it is complete, while other requests are still being
 * selected; on the other shapes a push-only pass follows the selection.  Either way the caller
 * then calls dsa_index_rows_exchange with mode = 2 (take) and the same epoch.  topk_stride even,
 * topk_out 8-byte aligned. */
int dsa_indexer_topk_send(const void* q_fp8, const void* k_cache, const float* weights,
                          const int32_t* seq_lens, const int32_t* block_table,
                          int64_t block_table_stride, int32_t* topk_out, int64_t topk_stride, int batch,
                          int num_pages, int max_pages, void* workspace, size_t workspace_bytes,
                          void* const* peer_stage, int world, int rank, int row_offset, uint32_t epoch,
                          int32_t* status_dev, void* stream);

/* Self-test of the bounded device-side waits (no counterpart in the reference, whose kernels spin
 * without a limit: sparse_fused.py:135-137).  One thread waits for at most `limit_ns` nanoseconds
 * (1 .. 1e9) on a barrier that receives no arrival, then sets DSA_STATUS_WAIT_TIMEOUT in
 * *status_dev and stores the time it waited in *waited_ns_dev (may be NULL).  Nothing faults or
 * hangs; the context stays usable.  This is the path every pipeline of the library takes when an
 * arrival is lost. */
int dsa_selftest_wait_expiry(uint64_t limit_ns, int32_t* status_dev, uint64_t* waited_ns_dev,
                             void* stream);

/* Issue-rate measurement of the tensor-core instructions the attention kernels choose between (no
 * counterpart in the reference; its own attempt at tcgen05 for this operator is recorded in
 * archive/dsa_sparse_attention_h16_ckv512_kpe64_topk2048_ps64/experiments/exp_40/result.md:7-19).
 * One CTA on all-zero shared-memory operands; nothing but the two cycle counts touches global memory.
 *   kind 0 / 1: `iters` tcgen05.mma back to back from one thread, bf16 (m x n x 16) / e4m3
 *               (m x n x 32), m in {64, 128}, n a multiple of 16 up to 256;
 *               cycles_dev[0] = until the last is issued, cycles_dev[1] = until all have completed;
 *   kind 2:     `iters` x 8 independent mma.sync.m16n8k16 per warp on `m` warps (1..32);
 *               cycles_dev[0] = cycles_dev[1] = duration.
 * sink_dev: one float the kernel may write (keeps the products alive). */
int dsa_selftest_mma_rate(int kind, int m, int n, int iters, long long* cycles_dev, float* sink_dev,
                          int32_t* status_dev, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DSA_B200_H_ */
