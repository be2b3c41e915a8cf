// Top-2048 selection over one fp32 score row per request, fused with the page -> global slot
// remap and the -1 padding (reference: torch.topk + remap, indexer_baseline.py:60, :82-90).
//
// One CTA per request.  Scores are mapped to order-preserving 32-bit keys; an 11+11+10 bit
// most-significant-digit radix descent over shared-memory histograms finds the exact key T of the
// 2048-th largest score and how many elements equal to T must be taken; a last sweep emits every
// element above T (warp-aggregated slot allocation) and the required number of elements equal to T
// (lowest positions first, so the selected SET is deterministic).  The row is staged in shared
// memory when it fits (<= 49152 scores), otherwise each sweep streams it from L2/global.
// Nothing here waits on another CTA.
#include "common.cuh"

namespace dsa {

constexpr int kSelThreads = 1024;
constexpr int kSelRowCap = 49152;  // keys staged in dynamic shared memory (192 KB)
constexpr int kSelBins = 2048;

struct SelShared {
  uint32_t hist[kSelBins];
  uint32_t warp_sums[32];
  uint32_t digit, above, ties, cnt_gt, cnt_eq;
};

// Inclusive prefix sum over the CTA in thread order.
__device__ __forceinline__ uint32_t block_inclusive_scan(uint32_t v, uint32_t* warp_sums) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    uint32_t n = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += n;
  }
  if (lane == 31) warp_sums[warp] = v;
  __syncthreads();
  if (warp == 0) {
    uint32_t w = warp_sums[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      uint32_t n = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += n;
    }
    warp_sums[lane] = w;
  }
  __syncthreads();
  if (warp > 0) v += warp_sums[warp - 1];
  __syncthreads();  // warp_sums may be reused by the caller
  return v;
}

__global__ void __launch_bounds__(kSelThreads, 1)
topk_select_kernel(const float* __restrict__ scores, int64_t score_stride,
                   const int32_t* __restrict__ seq_lens, const int32_t* __restrict__ block_table,
                   int64_t bt_stride, int32_t* __restrict__ out, int64_t out_stride, int max_pages,
                   int32_t* status) {
  extern __shared__ uint32_t row_keys[];
  __shared__ SelShared sh;

  const int b = blockIdx.x;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  int len = seq_lens[b];
  len = max(0, min(len, max_pages * kPage));
  int32_t* out_row = out + (size_t)b * out_stride;
  const int32_t* table = block_table + (size_t)b * bt_stride;
  const float* row = scores + (size_t)b * score_stride;

  if (len <= kTopK) {  // every token is selected: no scores needed
    for (int i = tid; i < kTopK; i += kSelThreads)
      out_row[i] = i < len ? table[i >> 6] * kPage + (i & 63) : -1;
    return;
  }

  const bool staged = len <= kSelRowCap;
  if (staged) {
    for (int i = tid; i < len; i += kSelThreads) row_keys[i] = float_to_ordered(row[i]);
  }
  if (tid == 0) { sh.cnt_gt = 0; sh.cnt_eq = 0; }
  auto key_at = [&](int i) -> uint32_t {
    return staged ? row_keys[i] : float_to_ordered(__ldg(row + i));
  };

  uint32_t prefix = 0, mask = 0, k_rem = kTopK;
#pragma unroll 1
  for (int pass = 0; pass < 3; ++pass) {
    const int shift = pass == 0 ? 21 : (pass == 1 ? 10 : 0);
    const int bits = pass == 2 ? 10 : 11;
    const uint32_t nb = 1u << bits;
    for (int i = tid; i < kSelBins; i += kSelThreads) sh.hist[i] = 0;
    __syncthreads();
    for (int i = tid; i < len; i += kSelThreads) {
      uint32_t k = key_at(i);
      if ((k & mask) == prefix) atomicAdd(&sh.hist[(k >> shift) & (nb - 1)], 1u);
    }
    __syncthreads();
    // Thread t owns the bins nb-1-per*t ... (descending), so a prefix scan in thread order is a
    // suffix sum over digits.
    const int per = nb / kSelThreads;  // 2 or 1
    uint32_t c_hi = sh.hist[nb - 1 - per * tid];
    uint32_t c_lo = per == 2 ? sh.hist[nb - 2 - per * tid] : 0u;
    uint32_t incl = block_inclusive_scan(c_hi + c_lo, sh.warp_sums);
    uint32_t excl = incl - (c_hi + c_lo);
    if (excl < k_rem && k_rem <= incl) {
      if (excl + c_hi >= k_rem) {
        sh.digit = nb - 1 - per * tid; sh.above = excl; sh.ties = c_hi;
      } else {
        sh.digit = nb - 2 - per * tid; sh.above = excl + c_hi; sh.ties = c_lo;
      }
    }
    __syncthreads();
    prefix |= sh.digit << shift;
    mask |= (nb - 1) << shift;
    k_rem -= sh.above;
    __syncthreads();
  }
  const uint32_t thresh = prefix;         // key of the 2048-th largest score
  const uint32_t n_gt = kTopK - k_rem;    // elements strictly above it
  const uint32_t ties = sh.ties;          // elements equal to it (>= k_rem)
  const bool take_all_ties = ties == k_rem;

  const int sweeps = (len + kSelThreads - 1) / kSelThreads;
  for (int s = 0; s < sweeps; ++s) {
    const int i = s * kSelThreads + tid;
    uint32_t k = i < len ? key_at(i) : 0u;
    const bool gt = i < len && k > thresh;
    const bool eq = i < len && k == thresh;
    uint32_t m = __ballot_sync(0xffffffffu, gt);
    if (m) {
      uint32_t base = 0;
      if (lane == 0) base = atomicAdd(&sh.cnt_gt, __popc(m));
      base = __shfl_sync(0xffffffffu, base, 0);
      if (gt) {
        uint32_t pos = base + __popc(m & ((1u << lane) - 1));
        if (pos < kTopK) out_row[pos] = table[i >> 6] * kPage + (i & 63);
      }
    }
    if (take_all_ties && eq) {
      uint32_t pos = n_gt + atomicAdd(&sh.cnt_eq, 1u);
      if (pos < kTopK) out_row[pos] = table[i >> 6] * kPage + (i & 63);
    }
  }
  if (!take_all_ties) {
    // More elements tie with the threshold than are needed: keep the lowest positions.
    uint32_t running = 0;
    for (int s = 0; s < sweeps && running < k_rem; ++s) {
      const int i = s * kSelThreads + tid;
      const bool eq = i < len && key_at(i) == thresh;
      uint32_t incl = block_inclusive_scan(eq ? 1u : 0u, sh.warp_sums);
      uint32_t rank = running + incl - 1;
      if (eq && rank < k_rem) out_row[n_gt + rank] = table[i >> 6] * kPage + (i & 63);
      if (tid == kSelThreads - 1) sh.above = incl;
      __syncthreads();
      running += sh.above;
      __syncthreads();
    }
  }
  __syncthreads();
  if (tid == 0 && sh.cnt_gt != n_gt) raise_status(status, DSA_STATUS_TOPK_COUNT);
}

cudaError_t launch_topk_select(const float* scores, int64_t score_stride, const int32_t* seq_lens,
                               const int32_t* block_table, int64_t bt_stride, int32_t* out,
                               int64_t out_stride, int batch, int max_pages, int32_t* status,
                               cudaStream_t stream) {
  size_t smem = sizeof(uint32_t) * (size_t)min(kSelRowCap, max(max_pages * kPage, 1));
  cudaError_t e = cudaFuncSetAttribute(topk_select_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)(sizeof(uint32_t) * kSelRowCap));
  if (e != cudaSuccess) return e;
  topk_select_kernel<<<batch, kSelThreads, smem, stream>>>(scores, score_stride, seq_lens,
                                                           block_table, bt_stride, out, out_stride,
                                                           max_pages, status);
  return cudaGetLastError();
}

}  // namespace dsa
