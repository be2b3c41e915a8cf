// Top-2048 selection over one fp32 score row per request, fused with the page -> global slot
// remap and the -1 padding (reference: torch.topk + remap, indexer_baseline.py:60, :82-90).
//
// One thread-block CLUSTER of 1, 2 or 4 CTAs (1024 threads each) per request: the row is cut into
// equal segments, one per CTA, so that a small batch still uses every SM; the CTAs exchange only
// their min/max, their 2048-bin histograms, their counts and the few boundary candidates through
// distributed shared memory.  A segment is staged in shared memory when it fits (<= 45056 scores),
// otherwise every sweep streams it from L2/global.
//
// Fast path (three sweeps): (A) min and max of the row; (B) a 2048-bin histogram over the LINEAR
// map of [min,max] -- scores of one request are spread over hundreds of bins, so shared-memory
// atomics rarely collide, unlike a histogram of the leading float bits where a few exponent bins
// take everything, and the staged scores are replaced in place by their bins; (C) one sweep over the
// bins: an element of a bin above the boundary bin is emitted at (elements in higher bins) + (its
// rank inside the bin, from a per-bin cursor), the few elements inside the boundary bin become
// candidates.  The linear map
// is monotone, so the bins order the elements exactly; the candidates are then ranked exactly by
// (order-preserving 32-bit key, lower position first) and the missing number of them is emitted.
// Fallback: when the boundary bin holds more than 1024 elements (flat or degenerate rows, massive
// ties) an 11+11+10 bit radix descent restricted to that bin finds the exact threshold key.
// The selected SET is deterministic; the order inside the output row is not part of the contract.
// Nothing here waits on another CTA.
//
// Two builds of the kernel: the wide one above (1024 threads, one CTA per SM) and a narrow one
// (512 threads, a cluster of one, two CTAs per SM) for batches of hundreds of rows that each fit
// half an SM's shared memory -- a row's selection is a chain of short sweeps and block-wide scans,
// so two rows in flight per SM serve chunked prefill (4096 rows of 16-20K scores) 1.36 x faster.
#include <cooperative_groups.h>

#include "common.cuh"
#include "ptx.cuh"
#include "tmap.cuh"

namespace dsa {

namespace cg = cooperative_groups;

constexpr int kSelThreads = 1024;   // wide CTA: one per SM, rows cut over a cluster
constexpr int kSelThreadsNarrow = 512;  // narrow CTA: two per SM, one whole row each (many short rows)
constexpr int kSelRowCap = 45056;  // scores staged in dynamic shared memory (176 KB + 8 KB table + 33 KB static)
constexpr int kSelBins = 2048;
constexpr int kSelTableCap = 2048;      // block_table entries staged in shared memory (128K tokens)
constexpr float kSelFloor = kScoreFloor;  // -inf / NaN scores are ranked as this value

// kCand: boundary-bin elements ranked exactly by the first CTA (at most one per thread).
template <int kCand>
struct SelShared {
  uint32_t hist[kSelBins];
  uint32_t cand_key[kCand];
  int cand_idx[kCand];
  uint32_t warp_sums[32];
  uint32_t red_a[32], red_b[32];
  uint32_t digit, above, ties, cnt_gt2, cnt_eq, cnt_cand, kmin, kmax;
  uint32_t tot[kSelBins];          // histogram summed over the cluster, then: elements in higher bins
  uint32_t low[kSelBins];          // this bin's elements in lower-ranked CTAs, then: output cursor
  uint32_t peer_min[4], peer_max[4], peer_cand[4];  // written by the peers
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
// Thread t owns the `per` = nb / kT bins nb-1-per*t ... downwards.  Results in sh.digit / sh.above /
// sh.ties.  With `to_above`, hist[bin] is replaced by the number of elements in higher bins.
template <int kT, class Sh>
__device__ __forceinline__ void find_boundary_bin(Sh& sh, uint32_t* hist, uint32_t nb,
                                                  uint32_t k, bool to_above = false) {
  const int tid = threadIdx.x;
  const int per = max(1, (int)nb / kT);   // 1, 2 or 4
  const int top = (int)nb - 1 - per * tid;
  uint32_t c[4] = {0u, 0u, 0u, 0u};
  uint32_t sum = 0;
  if (top >= 0) {
#pragma unroll
    for (int e = 0; e < 4; ++e)
      if (e < per) { c[e] = hist[top - e]; sum += c[e]; }
  }
  const uint32_t incl = block_inclusive_scan(sum, sh.warp_sums);
  uint32_t run = incl - sum;
  if (top >= 0) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (e < per) {
        if (to_above) hist[top - e] = run;
        if (run < k && k <= run + c[e]) { sh.digit = top - e; sh.above = run; sh.ties = c[e]; }
        run += c[e];
      }
    }
  }
  __syncthreads();
}

template <int kT, int kCand, int kMinCtas>
__global__ void __launch_bounds__(kT, kMinCtas)
topk_select_kernel(const float* __restrict__ scores, int64_t score_stride,
                   const int32_t* __restrict__ seq_lens, const int32_t* __restrict__ block_table,
                   int64_t bt_stride, int32_t* __restrict__ out, int64_t out_stride, int max_pages,
                   int row_cap, uint32_t* __restrict__ minmax, int32_t* status) {
  // dynamic shared memory: row_cap staged scores, then the staged block_table entries
  extern __shared__ float row_s[];
  __shared__ SelShared<kCand> sh;
  using Sh = SelShared<kCand>;
  int32_t* table_s = reinterpret_cast<int32_t*>(row_s + row_cap);
  constexpr int kSelThreads = kT;
  constexpr int kSelCandCap = kCand;
  cg::cluster_group cluster = cg::this_cluster();
  const int csize = (int)cluster.num_blocks();   // CTAs per request: 1, 2 or 4
  const int crank = (int)cluster.block_rank();

  const int b = blockIdx.x / csize;
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  int len = seq_lens[b];
  len = max(0, min(len, max_pages * kPage));
  int32_t* out_row = out + (size_t)b * out_stride;
  const int32_t* table = block_table + (size_t)b * bt_stride;
  const float* row = scores + (size_t)b * score_stride;
  const int n_pages = (len + kPage - 1) / kPage;
  const bool table_staged = n_pages <= min(max_pages, kSelTableCap);
  // the emit loops would otherwise pay a dependent global load per selected element
  auto slot_of = [&](int i) -> int32_t {
    return (table_staged ? table_s[i >> 6] : table[i >> 6]) * kPage + (i & 63);
  };

  if (len <= kTopK) {  // every token is selected: no scores needed (uniform over the cluster)
    // The output row may still be read by the kernel before us in the stream (the previous step's
    // attention, when no scorer runs in between): no global write before the dependency wait.
    ptx::launch_dependents();
    ptx::grid_dependency_wait();
    for (int i = crank * kSelThreads + tid; i < kTopK; i += csize * kSelThreads)
      out_row[i] = i < len ? table[i >> 6] * kPage + (i & 63) : -1;
    if (minmax != nullptr && crank == 0 && tid == 0) { minmax[2 * b] = 0u; minmax[2 * b + 1] = 0u; }
    return;
  }
  if (table_staged) {
    for (int i = tid; i < n_pages; i += kSelThreads) table_s[i] = table[i];
  }

  // this CTA's segment [seg_lo, seg_hi) of the row (multiples of 4 keep the 16-byte loads aligned)
  const int seg = ((len + csize - 1) / csize + 3) & ~3;
  const int seg_lo = min(len, crank * seg), seg_hi = min(len, seg_lo + seg);
  const int seg_len = seg_hi - seg_lo;
  const bool staged = seg <= row_cap;
  auto value_at = [&](int i) -> float { return staged ? row_s[i - seg_lo] : __ldg(row + i); };

  // everything above only read the caller's inputs; the scores come from the kernel before us.
  // The successor (the attention kernel: it reads nothing before its own wait) may be scheduled
  // already while we wait for the scorer.
  ptx::launch_dependents();
  ptx::grid_dependency_wait();

  // The scorer may have left the row's min / max (ordered keys, max of key and of ~key) next to the
  // scores: then sweep A is not needed and the staging happens in sweep B.  Stale or foreign values
  // would only cost speed: the bins stay monotone, out-of-range scores are clamped to the end bins.
  uint32_t given_max = 0u, given_min_inv = 0u;
  if (minmax != nullptr) {
    given_max = minmax[2 * b];
    given_min_inv = minmax[2 * b + 1];
  }
  const bool have_minmax = given_max != 0u && given_min_inv != 0u;   // uniform over the cluster
  if (have_minmax) {
    for (int i = tid; i < kSelBins; i += kSelThreads) sh.hist[i] = 0;
    if (tid == 0) {
      sh.cnt_gt2 = 0; sh.cnt_eq = 0; sh.cnt_cand = 0;
      sh.kmin = __float_as_uint(ordered_to_float(~given_min_inv));
      sh.kmax = __float_as_uint(ordered_to_float(given_max));
    }
    __syncthreads();
  } else
  // ---- sweep A: stage the segment, min / max ----------------------------------------------------
  {
    float mn = INFINITY, mx = kSelFloor;
    const bool vec = (reinterpret_cast<uintptr_t>(row) & 15u) == 0;
    const int n4 = vec ? (seg_len & ~3) : 0;
    for (int i = tid * 4; i < n4; i += kSelThreads * 4) {  // 16-byte loads, all in flight at once
      const float4 q = __ldg(reinterpret_cast<const float4*>(row + seg_lo + i));
      if (staged) *reinterpret_cast<float4*>(row_s + i) = q;
      mn = fminf(fminf(mn, fmaxf(q.x, kSelFloor)), fminf(fmaxf(q.y, kSelFloor), fminf(fmaxf(q.z, kSelFloor), fmaxf(q.w, kSelFloor))));
      mx = fmaxf(fmaxf(mx, q.x), fmaxf(q.y, fmaxf(q.z, q.w)));
    }
    for (int i = n4 + tid; i < seg_len; i += kSelThreads) {
      float v = __ldg(row + seg_lo + i);
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
    if (tid == 0) { sh.cnt_gt2 = 0; sh.cnt_eq = 0; sh.cnt_cand = 0; }
    __syncthreads();
    if (warp == 0) {
      mn = __uint_as_float(sh.red_a[lane]);
      mx = __uint_as_float(sh.red_b[lane]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      }
      if (lane < csize) {  // publish this CTA's min / max in every CTA of the cluster
        Sh* peer = cluster.map_shared_rank(&sh, lane);
        peer->peer_min[crank] = __float_as_uint(mn);
        peer->peer_max[crank] = __float_as_uint(mx);
      }
    }
    cluster.sync();
    mn = __uint_as_float(sh.peer_min[0]);
    mx = __uint_as_float(sh.peer_max[0]);
    for (int r = 1; r < csize; ++r) {
      mn = fminf(mn, __uint_as_float(sh.peer_min[r]));
      mx = fmaxf(mx, __uint_as_float(sh.peer_max[r]));
    }
    if (tid == 0) { sh.kmin = __float_as_uint(mn); sh.kmax = __float_as_uint(mx); }
    __syncthreads();
  }
  const float lo = __uint_as_float(sh.kmin);
  const float span = __uint_as_float(sh.kmax) - lo;
  const float inv = span > 0.f ? (float)kSelBins / span : 0.f;
  auto bin_of = [&](float v) -> int {
    // clamped at both ends (and NaN -> 0): with a [lo, hi] that does not come from this very row
    // the map must still be monotone and stay inside the histogram
    return min(kSelBins - 1, __float2int_rz(fmaxf((fmaxf(v, kSelFloor) - lo) * inv, 0.f)));
  };

  // ---- sweep B: histogram of the linear bins, summed over the cluster ---------------------------
  // A staged score is replaced in place by its bin: the last sweep needs nothing else (the few
  // boundary-bin elements re-read their score from L2).
  int* bin_s = reinterpret_cast<int*>(row_s);
  // four elements per thread and step: the loads, the bin arithmetic and the atomics of the four
  // are independent, which hides the shared-memory latency that a one-element loop exposes
  const bool vec_ok = (reinterpret_cast<uintptr_t>(row) & 15u) == 0;
  const int n4s = staged && (vec_ok || !have_minmax) ? (seg_len & ~3) : 0;
  for (int i = tid * 4; i < n4s; i += kSelThreads * 4) {
    const float4 q = have_minmax ? __ldg(reinterpret_cast<const float4*>(row + seg_lo + i))
                                 : *reinterpret_cast<const float4*>(row_s + i);
    const int4 bq = make_int4(bin_of(q.x), bin_of(q.y), bin_of(q.z), bin_of(q.w));
    *reinterpret_cast<int4*>(bin_s + i) = bq;
    atomicAdd(&sh.hist[bq.x], 1u);
    atomicAdd(&sh.hist[bq.y], 1u);
    atomicAdd(&sh.hist[bq.z], 1u);
    atomicAdd(&sh.hist[bq.w], 1u);
  }
  for (int i = seg_lo + n4s + tid; i < seg_hi; i += kSelThreads) {
    const int bin = bin_of(have_minmax ? __ldg(row + i) : value_at(i));
    if (staged) bin_s[i - seg_lo] = bin;
    atomicAdd(&sh.hist[bin], 1u);
  }
  cluster.sync();
  if (have_minmax && crank == 0 && tid == 0) {   // every CTA of the cluster has read them: reset
    minmax[2 * b] = 0u;
    minmax[2 * b + 1] = 0u;
  }
  for (int k = tid; k < kSelBins; k += kSelThreads) {
    uint32_t c = 0, below_me = 0;
    for (int r = 0; r < csize; ++r) {
      const uint32_t h = cluster.map_shared_rank(&sh, r)->hist[k];
      c += h;
      if (r < crank) below_me += h;
    }
    sh.tot[k] = c;
    sh.low[k] = below_me;
  }
  __syncthreads();
  find_boundary_bin<kT>(sh, sh.tot, kSelBins, kTopK, true);   // every CTA finds the same boundary
  const int edge = (int)sh.digit;          // boundary bin
  const uint32_t above = sh.above;         // elements in higher bins: all selected
  const uint32_t in_edge = sh.ties;        // elements in the boundary bin (whole row)
  const uint32_t need = kTopK - above;     // how many of them are selected (>= 1)
  const bool few = in_edge <= (uint32_t)kSelCandCap;

  // ---- sweep C: emit; collect the boundary bin --------------------------------------------------
  // An element of bin k > edge goes to tot[k] (elements in higher bins, whole row) + its rank
  // inside the bin: first the lower-ranked CTAs' share (low[k]), then this CTA's in arrival order.
  auto candidate = [&](int i) {
    const uint32_t c = atomicAdd(&sh.cnt_cand, 1u);
    if (c < (uint32_t)kSelCandCap) {   // NaN and -inf rank as kSelFloor here as in the bins
      sh.cand_key[c] = float_to_ordered(fmaxf(__ldg(row + i), kSelFloor));
      sh.cand_idx[c] = i;
    }
  };
  for (int i = tid * 4; i < n4s; i += kSelThreads * 4) {
    const int4 bq = *reinterpret_cast<const int4*>(bin_s + i);
    const int bins[4] = {bq.x, bq.y, bq.z, bq.w};
    uint32_t rank_in_bin[4];
#pragma unroll
    for (int e = 0; e < 4; ++e)   // the four cursor updates are in flight together
      rank_in_bin[e] = bins[e] > edge ? atomicAdd(&sh.low[bins[e]], 1u) : 0u;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (bins[e] > edge) {
        const uint32_t pos = sh.tot[bins[e]] + rank_in_bin[e];
        if (pos < (uint32_t)kTopK) out_row[pos] = slot_of(seg_lo + i + e);
      } else if (few && bins[e] == edge) {
        candidate(seg_lo + i + e);
      }
    }
  }
  for (int i = seg_lo + n4s + tid; i < seg_hi; i += kSelThreads) {
    const int bin = staged ? bin_s[i - seg_lo] : bin_of(__ldg(row + i));
    if (bin > edge) {
      const uint32_t pos = sh.tot[bin] + atomicAdd(&sh.low[bin], 1u);
      if (pos < (uint32_t)kTopK) out_row[pos] = slot_of(i);
    } else if (few && bin == edge) {
      candidate(i);
    }
  }
  __syncthreads();
  if (tid == 0) cluster.map_shared_rank(&sh, 0)->peer_cand[crank] = sh.cnt_cand;
  cluster.sync();

  if (few) {
    // ---- exact ranking of the candidates by the first CTA: higher key first, lower position
    //      first on ties ------------------------------------------------------------------------
    if (crank == 0) {
      uint32_t n = min(sh.peer_cand[0], (uint32_t)kSelCandCap);
      for (int r = 1; r < csize; ++r) {
        const uint32_t nr = min(sh.peer_cand[r], (uint32_t)kSelCandCap - n);
        const Sh* peer = cluster.map_shared_rank(&sh, r);
        for (uint32_t j = tid; j < nr; j += kSelThreads) {
          sh.cand_key[n + j] = peer->cand_key[j];
          sh.cand_idx[n + j] = peer->cand_idx[j];
        }
        n += nr;
      }
      __syncthreads();
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
      if (tid == 0 && n != in_edge) raise_status(status, DSA_STATUS_TOPK_COUNT);
    }
    cluster.sync();  // the peers' shared memory stays alive until the first CTA has read it
    return;
  }

  // ---- fallback (first CTA, whole row from L2/global): radix descent over the ordered keys of the
  //      boundary bin ----------------------------------------------------------------------------
  if (crank == 0) {
    auto key_in_edge = [&](int i, uint32_t& key) -> bool {
      const float v = fmaxf(__ldg(row + i), kSelFloor);   // NaN and -inf rank as kSelFloor
      key = float_to_ordered(v);
      return bin_of(v) == edge;
    };
    const int sweeps = (len + kSelThreads - 1) / kSelThreads;
    uint32_t prefix = 0, mask = 0, k_rem = need;
#pragma unroll 1
    for (int pass = 0; pass < 3; ++pass) {
      const int shift = pass == 0 ? 21 : (pass == 1 ? 10 : 0);
      const int bits = pass == 2 ? 10 : 11;
      const uint32_t nb = 1u << bits;
      for (int i = tid; i < kSelBins; i += kSelThreads) sh.tot[i] = 0;
      __syncthreads();
      for (int i = tid; i < len; i += kSelThreads) {
        uint32_t k;
        if (key_in_edge(i, k) && (k & mask) == prefix) atomicAdd(&sh.tot[(k >> shift) & (nb - 1)], 1u);
      }
      __syncthreads();
      find_boundary_bin<kT>(sh, sh.tot, nb, k_rem);
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
        const uint32_t inc2 = block_inclusive_scan(eq ? 1u : 0u, sh.warp_sums);
        const uint32_t rank = running + inc2 - 1;
        if (eq && rank < k_rem) out_row[above + n_gt + rank] = slot_of(i);
        if (tid == kSelThreads - 1) sh.above = inc2;
        __syncthreads();
        running += sh.above;
        __syncthreads();
      }
    }
    __syncthreads();
    if (tid == 0 && sh.cnt_gt2 != n_gt) raise_status(status, DSA_STATUS_TOPK_COUNT);
  }
  cluster.sync();
}

// CTAs per request: as many as fit in one wave (a CTA of 1024 threads owns an SM), and more than
// that when a CTA's share of the longest possible row would not fit the staging buffer: a staged
// segment is read from L2 once, a streamed one in every sweep, which outweighs the extra waves
// (64 rows of 131072 scores: 57 us with 2 CTAs per row, 38 us with 4; 256 rows of 32K-128K: 169 us
// with one, 128 us with 4).
static int select_cluster_size(int batch, int max_len) {
  const int sms = sm_count();
  int c = batch * 4 <= sms ? 4 : (batch * 2 <= sms ? 2 : 1);
  while (c < 4 && (max_len + c - 1) / c > kSelRowCap) c *= 2;
  return c;
}

namespace {

template <int kT, int kCand, int kMinCtas>
cudaError_t launch_select_variant(size_t dyn_cap, int csize, int batch, int row_cap, int table_cap,
                                  const float* scores, int64_t score_stride, const int32_t* seq_lens,
                                  const int32_t* block_table, int64_t bt_stride, int32_t* out,
                                  int64_t out_stride, int max_pages, uint32_t* minmax,
                                  int32_t* status, cudaStream_t stream) {
  static std::atomic<uint64_t> smem_opted{0};
  auto kernel = topk_select_kernel<kT, kCand, kMinCtas>;
  cudaError_t e = opt_in_dynamic_smem(reinterpret_cast<const void*>(kernel), dyn_cap, smem_opted);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(batch * csize));
  cfg.blockDim = dim3(kT);
  cfg.dynamicSmemBytes = sizeof(float) * (size_t)row_cap + sizeof(int32_t) * (size_t)table_cap;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = csize;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = pdl_enabled();
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return cudaLaunchKernelEx(&cfg, kernel, scores, score_stride, seq_lens, block_table, bt_stride,
                            out, out_stride, max_pages, row_cap, minmax, status);
}

}  // namespace

cudaError_t launch_topk_select(const float* scores, int64_t score_stride, const int32_t* seq_lens,
                               const int32_t* block_table, int64_t bt_stride, int32_t* out,
                               int64_t out_stride, int batch, int max_pages, uint32_t* minmax,
                               int32_t* status, cudaStream_t stream) {
  const int csize = select_cluster_size(batch, max_pages * kPage);
  const int seg_max = (((max_pages * kPage + csize - 1) / csize) + 3) & ~3;
  const int row_cap = min(kSelRowCap, max(seg_max, 4));
  const int table_cap = min(max(max_pages, 1), kSelTableCap);
  const size_t wide_cap = sizeof(float) * kSelRowCap + sizeof(int32_t) * kSelTableCap;
  // Many rows that each fit half an SM's shared memory (chunked prefill: thousands of rows of a few
  // ten thousand scores): two narrow CTAs per SM.  A row's selection is a chain of short sweeps
  // and block-wide scans, latency-bound, so two rows in flight per SM nearly double the rate.
  constexpr size_t kNarrowDynCap = 113 * 1024 - sizeof(SelShared<kSelThreadsNarrow>) - 256;
  const size_t dyn = sizeof(float) * (size_t)row_cap + sizeof(int32_t) * (size_t)table_cap;
  if (csize == 1 && seg_max <= row_cap && dyn <= kNarrowDynCap && batch >= 2 * sm_count())
    return launch_select_variant<kSelThreadsNarrow, kSelThreadsNarrow, 2>(
        kNarrowDynCap, csize, batch, row_cap, table_cap, scores, score_stride, seq_lens,
        block_table, bt_stride, out, out_stride, max_pages, minmax, status, stream);
  return launch_select_variant<kSelThreads, 1024, 1>(
      wide_cap, csize, batch, row_cap, table_cap, scores, score_stride, seq_lens, block_table,
      bt_stride, out, out_stride, max_pages, minmax, status, stream);
}

}  // namespace dsa
