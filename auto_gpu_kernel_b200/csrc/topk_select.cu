// Top-2048 selection over one fp32 score row per request, fused with the page -> global slot
// remap and the -1 padding (reference: torch.topk + remap, indexer_baseline.py:60, :82-90).
//
// One CTA (1024 threads) per request; the row is staged in shared memory when it fits (<= 49152
// scores), otherwise every sweep streams it from L2/global.
//
// Fast path (three sweeps): (A) min and max of the row; (B) a 2048-bin histogram over the LINEAR
// map of [min,max] -- scores of one request are spread over hundreds of bins, so shared-memory
// atomics rarely collide, unlike a histogram of the leading float bits where a few exponent bins
// take everything; (C) every element in a bin above the boundary bin is emitted (warp-aggregated
// slot allocation), the few elements inside the boundary bin become candidates.  The linear map
// is monotone, so the bins order the elements exactly; the candidates are then ranked exactly by
// (order-preserving 32-bit key, lower position first) and the missing number of them is emitted.
// Fallback: when the boundary bin holds more than 1024 elements (flat or degenerate rows, massive
// ties) an 11+11+10 bit radix descent restricted to that bin finds the exact threshold key.
// The selected SET is deterministic; the order inside the output row is not part of the contract.
// Nothing here waits on another CTA.
#include "common.cuh"

namespace dsa {

constexpr int kSelThreads = 1024;
constexpr int kSelRowCap = 49152;  // scores staged in dynamic shared memory (192 KB)
constexpr int kSelBins = 2048;
constexpr int kSelCandCap = 1024;
constexpr int kSelTableCap = 2048;      // block_table entries staged in shared memory (128K tokens)
constexpr float kSelFloor = -3.0e38f;  // -inf / NaN scores are ranked as this value

struct SelShared {
  uint32_t hist[kSelBins];
  uint32_t cand_key[kSelCandCap];
  int cand_idx[kSelCandCap];
  int32_t table[kSelTableCap];
  uint32_t warp_sums[32];
  uint32_t red_a[32], red_b[32];
  uint32_t digit, above, ties, cnt_gt, cnt_gt2, cnt_eq, cnt_cand, kmin, kmax;
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

// Find the digit d (bins are scanned from the top) such that count(bins > d) < k <= count(bins >= d).
// Thread t owns bins nb-1-per*t ... downwards.  Results in sh.digit / sh.above / sh.ties.
__device__ __forceinline__ void find_boundary_bin(SelShared& sh, uint32_t nb, uint32_t k) {
  const int tid = threadIdx.x;
  const int per = nb / kSelThreads;  // 2 or 1
  uint32_t c_hi = sh.hist[nb - 1 - per * tid];
  uint32_t c_lo = per == 2 ? sh.hist[nb - 2 - per * tid] : 0u;
  uint32_t incl = block_inclusive_scan(c_hi + c_lo, sh.warp_sums);
  uint32_t excl = incl - (c_hi + c_lo);
  if (excl < k && k <= incl) {
    if (excl + c_hi >= k) {
      sh.digit = nb - 1 - per * tid; sh.above = excl; sh.ties = c_hi;
    } else {
      sh.digit = nb - 2 - per * tid; sh.above = excl + c_hi; sh.ties = c_lo;
    }
  }
  __syncthreads();
}

__global__ void __launch_bounds__(kSelThreads, 1)
topk_select_kernel(const float* __restrict__ scores, int64_t score_stride,
                   const int32_t* __restrict__ seq_lens, const int32_t* __restrict__ block_table,
                   int64_t bt_stride, int32_t* __restrict__ out, int64_t out_stride, int max_pages,
                   int32_t* status) {
  extern __shared__ float row_s[];
  __shared__ SelShared sh;

  const int b = blockIdx.x;
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  int len = seq_lens[b];
  len = max(0, min(len, max_pages * kPage));
  int32_t* out_row = out + (size_t)b * out_stride;
  const int32_t* table = block_table + (size_t)b * bt_stride;
  const float* row = scores + (size_t)b * score_stride;
  const int n_pages = (len + kPage - 1) / kPage;
  const bool table_staged = n_pages <= kSelTableCap;
  // the emit loops would otherwise pay a dependent global load per selected element
  auto slot_of = [&](int i) -> int32_t {
    return (table_staged ? sh.table[i >> 6] : table[i >> 6]) * kPage + (i & 63);
  };

  if (len <= kTopK) {  // every token is selected: no scores needed
    for (int i = tid; i < kTopK; i += kSelThreads)
      out_row[i] = i < len ? table[i >> 6] * kPage + (i & 63) : -1;
    return;
  }
  if (table_staged) {
    for (int i = tid; i < n_pages; i += kSelThreads) sh.table[i] = table[i];
  }

  const bool staged = len <= kSelRowCap;
  auto value_at = [&](int i) -> float { return staged ? row_s[i] : __ldg(row + i); };

  // ---- sweep A: stage the row, min / max ------------------------------------------------------
  {
    float mn = INFINITY, mx = kSelFloor;
    const bool vec = (reinterpret_cast<uintptr_t>(row) & 15u) == 0;
    const int len4 = vec ? (len & ~3) : 0;
    for (int i = tid * 4; i < len4; i += kSelThreads * 4) {  // 16-byte loads, all in flight at once
      const float4 q = __ldg(reinterpret_cast<const float4*>(row + i));
      if (staged) *reinterpret_cast<float4*>(row_s + i) = q;
      mn = fminf(fminf(mn, fmaxf(q.x, kSelFloor)), fminf(fmaxf(q.y, kSelFloor), fminf(fmaxf(q.z, kSelFloor), fmaxf(q.w, kSelFloor))));
      mx = fmaxf(fmaxf(mx, q.x), fmaxf(q.y, fmaxf(q.z, q.w)));
    }
    for (int i = len4 + tid; i < len; i += kSelThreads) {
      float v = __ldg(row + i);
      if (staged) row_s[i] = v;
      v = fmaxf(v, kSelFloor);
      mn = fminf(mn, v);
      mx = fmaxf(mx, v);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    if (lane == 0) { sh.red_a[warp] = __float_as_uint(mn); sh.red_b[warp] = __float_as_uint(mx); }
    for (int i = tid; i < kSelBins; i += kSelThreads) sh.hist[i] = 0;
    if (tid == 0) { sh.cnt_gt = 0; sh.cnt_gt2 = 0; sh.cnt_eq = 0; sh.cnt_cand = 0; }
    __syncthreads();
    if (warp == 0) {
      mn = __uint_as_float(sh.red_a[lane]);
      mx = __uint_as_float(sh.red_b[lane]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      }
      if (lane == 0) { sh.kmin = __float_as_uint(mn); sh.kmax = __float_as_uint(mx); }
    }
    __syncthreads();
  }
  const float lo = __uint_as_float(sh.kmin);
  const float span = __uint_as_float(sh.kmax) - lo;
  const float inv = span > 0.f ? (float)kSelBins / span : 0.f;
  auto bin_of = [&](float v) -> int {
    return min(kSelBins - 1, __float2int_rz((fmaxf(v, kSelFloor) - lo) * inv));
  };

  // ---- sweep B: histogram of the linear bins ---------------------------------------------------
  // When the row is staged, its shared-memory copy is overwritten by the bin numbers: the later
  // sweeps only compare bins, and the few boundary-bin elements re-read their score from L2.
  int* bin_s = reinterpret_cast<int*>(row_s);
  for (int i = tid; i < len; i += kSelThreads) {
    const int bn = bin_of(value_at(i));
    if (staged) bin_s[i] = bn;
    atomicAdd(&sh.hist[bn], 1u);
  }
  auto bin_at = [&](int i) -> int { return staged ? bin_s[i] : bin_of(__ldg(row + i)); };
  __syncthreads();
  find_boundary_bin(sh, kSelBins, kTopK);
  const int edge = (int)sh.digit;          // boundary bin
  const uint32_t above = sh.above;         // elements in higher bins: all selected
  const uint32_t in_edge = sh.ties;        // elements in the boundary bin
  const uint32_t need = kTopK - above;     // how many of them are selected (>= 1)
  const bool few = in_edge <= (uint32_t)kSelCandCap;
  __syncthreads();

  // ---- sweep C: emit everything above the boundary bin, collect the boundary bin ---------------
  // Each thread first counts its own elements above the boundary, a warp scan plus ONE shared
  // atomic per warp hands out contiguous output slots, then the elements are written: no atomic
  // (and no dependent round trip) inside the per-element loops.
  const int sweeps = (len + kSelThreads - 1) / kSelThreads;
  {
    uint32_t mine = 0;
    for (int i = tid; i < len; i += kSelThreads) mine += bin_at(i) > edge ? 1u : 0u;
    uint32_t incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t n = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += n;
    }
    uint32_t base = 0;
    if (lane == 31) base = atomicAdd(&sh.cnt_gt, incl);
    base = __shfl_sync(0xffffffffu, base, 31);
    uint32_t pos = base + incl - mine;
    for (int i = tid; i < len; i += kSelThreads) {
      const int bin = bin_at(i);
      if (bin > edge) {
        if (pos < (uint32_t)kTopK) out_row[pos] = slot_of(i);
        ++pos;
      } else if (few && bin == edge) {
        const uint32_t c = atomicAdd(&sh.cnt_cand, 1u);
        if (c < (uint32_t)kSelCandCap) {
          sh.cand_key[c] = float_to_ordered(__ldg(row + i));
          sh.cand_idx[c] = i;
        }
      }
    }
  }
  __syncthreads();

  if (few) {
    // ---- exact ranking of the candidates: higher key first, lower position first on ties -------
    const uint32_t n = min(sh.cnt_cand, (uint32_t)kSelCandCap);
    if (tid < (int)n) {
      const uint32_t ka = sh.cand_key[tid];
      const int ia = sh.cand_idx[tid];
      uint32_t rank = 0;
      if (n != need) {
        for (uint32_t j = 0; j < n; ++j) {
          const uint32_t kb = sh.cand_key[j];
          rank += (kb > ka) || (kb == ka && sh.cand_idx[j] < ia);
        }
      } else {
        rank = tid;
      }
      if (rank < need) out_row[above + rank] = slot_of(ia);
    }
    if (tid == 0 && (sh.cnt_gt != above || n != in_edge)) raise_status(status, DSA_STATUS_TOPK_COUNT);
    return;
  }

  // ---- fallback: radix descent over the ordered keys of the boundary bin ------------------------
  auto key_in_edge = [&](int i, uint32_t& key) -> bool {  // the staged copy now holds bins
    const float v = __ldg(row + i);
    key = float_to_ordered(v);
    return bin_of(v) == edge;
  };
  uint32_t prefix = 0, mask = 0, k_rem = need;
#pragma unroll 1
  for (int pass = 0; pass < 3; ++pass) {
    const int shift = pass == 0 ? 21 : (pass == 1 ? 10 : 0);
    const int bits = pass == 2 ? 10 : 11;
    const uint32_t nb = 1u << bits;
    for (int i = tid; i < kSelBins; i += kSelThreads) sh.hist[i] = 0;
    __syncthreads();
    for (int i = tid; i < len; i += kSelThreads) {
      uint32_t k;
      if (key_in_edge(i, k) && (k & mask) == prefix) atomicAdd(&sh.hist[(k >> shift) & (nb - 1)], 1u);
    }
    __syncthreads();
    find_boundary_bin(sh, nb, k_rem);
    prefix |= sh.digit << shift;
    mask |= (nb - 1) << shift;
    k_rem -= sh.above;
    __syncthreads();
  }
  const uint32_t thresh = prefix;             // key of the last selected element
  const uint32_t n_gt = need - k_rem;         // boundary-bin elements strictly above it
  const bool take_all_ties = sh.ties == k_rem;
  for (int s = 0; s < sweeps; ++s) {
    const int i = s * kSelThreads + tid;
    uint32_t k = 0;
    const bool in = i < len && key_in_edge(i, k);
    const bool gt = in && k > thresh;
    const bool eq = in && k == thresh;
    const uint32_t m = __ballot_sync(0xffffffffu, gt);
    if (m) {
      uint32_t base = 0;
      if (lane == 0) base = atomicAdd(&sh.cnt_gt2, __popc(m));
      base = __shfl_sync(0xffffffffu, base, 0);
      if (gt) {
        const uint32_t pos = above + base + __popc(m & ((1u << lane) - 1));
        if (pos < (uint32_t)kTopK) out_row[pos] = slot_of(i);
      }
    }
    if (take_all_ties && eq) {
      const uint32_t pos = above + n_gt + atomicAdd(&sh.cnt_eq, 1u);
      if (pos < (uint32_t)kTopK) out_row[pos] = slot_of(i);
    }
  }
  if (!take_all_ties) {
    // more elements equal the threshold than are needed: keep the lowest positions
    uint32_t running = 0;
    for (int s = 0; s < sweeps && running < k_rem; ++s) {
      const int i = s * kSelThreads + tid;
      uint32_t k = 0;
      const bool eq = i < len && key_in_edge(i, k) && k == thresh;
      const uint32_t incl = block_inclusive_scan(eq ? 1u : 0u, sh.warp_sums);
      const uint32_t rank = running + incl - 1;
      if (eq && rank < k_rem) out_row[above + n_gt + rank] = slot_of(i);
      if (tid == kSelThreads - 1) sh.above = incl;
      __syncthreads();
      running += sh.above;
      __syncthreads();
    }
  }
  __syncthreads();
  if (tid == 0 && (sh.cnt_gt != above || sh.cnt_gt2 != n_gt)) raise_status(status, DSA_STATUS_TOPK_COUNT);
}

cudaError_t launch_topk_select(const float* scores, int64_t score_stride, const int32_t* seq_lens,
                               const int32_t* block_table, int64_t bt_stride, int32_t* out,
                               int64_t out_stride, int batch, int max_pages, int32_t* status,
                               cudaStream_t stream) {
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(topk_select_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)(sizeof(float) * kSelRowCap));
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  size_t smem = sizeof(float) * (size_t)min(kSelRowCap, max(max_pages * kPage, 1));
  topk_select_kernel<<<batch, kSelThreads, smem, stream>>>(scores, score_stride, seq_lens,
                                                           block_table, bt_stride, out, out_stride,
                                                           max_pages, status);
  return cudaGetLastError();
}

}  // namespace dsa
