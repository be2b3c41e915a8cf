// Top-2048 selection that starts from a finished histogram (reference: torch.topk + page remap +
// -1 padding, indexer_baseline.py:60, :82-90).
//
// The scorer (indexer_score_tc_kernel<true>) has already counted every score of a request into
// 4096 bins over the top 12 bits of its order-preserving key.  What is left is a short chain:
//   (1) boundary bin: one read of the 16 KB histogram and one block scan (every CTA of the request's
//       cluster does it for itself, while its slice of the score row is on its way into shared memory);
//   (2) one counting sweep over the staged slice (elements above the boundary bin, elements inside
//       it) and one block scan: every selected element then has its place in the output row without
//       any atomic -- the row's totals are known from the histogram, so the first CTA of a pair
//       fills the row from the front and the second from the back (a cluster of four exchanges the
//       CTAs' totals through distributed shared memory);
//   (3) the writing sweep; elements of the boundary bin go (key, position) into the first CTA's
//       candidate list;
//   (4) the first CTA picks the missing elements among the candidates exactly, by (key, lower
//       position first), eight bits of the 52-bit composite per pass (normally one or two passes).
// A boundary bin with more than 2048 elements (flat rows, mass ties) falls back to a radix descent
// over the row.  One cluster of 1, 2 or 4 CTAs of 1024 threads per request; nothing waits on
// another CTA outside cluster barriers.
#include <cooperative_groups.h>

#include "common.cuh"
#include "ptx.cuh"
#include "tmap.cuh"

namespace dsa {

namespace cg = cooperative_groups;

constexpr int kShThreads = 1024;
constexpr int kShRowCap = 45056;        // scores staged in dynamic shared memory (176 KB)
constexpr int kShCandCap = 2048;
constexpr int kShTableCap = 2048;       // block_table entries staged in shared memory (128K tokens)
constexpr int kShBinShift = 20;         // bin = top 12 bits of the ordered key

struct ShShared {
  uint32_t cand_key[kShCandCap];
  uint32_t cand_idx[kShCandCap];
  int32_t table[kShTableCap];
  uint32_t sub[256];
  uint32_t warp_sums[32];
  uint32_t last[32];                    // candidates of the boundary digit, when they are few
  uint32_t edge, above, in_edge, digit, dabove, dcount, emit_cnt, last_n;
  uint32_t peer_sel[4], peer_cnd[4];    // written by the peers
};

__device__ __forceinline__ uint32_t sh_key(float v) { return float_to_ordered(fmaxf(v, kScoreFloor)); }

// Exclusive prefix sum over the CTA in thread order (two block barriers, and a third unless the
// caller itself passes a block or cluster barrier before warp_sums is written again).
template <bool kTrailingBarrier = true>
__device__ __forceinline__ uint32_t sh_block_excl_scan(uint32_t v, uint32_t* warp_sums, uint32_t* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += n;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    uint32_t w = warp_sums[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t n = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += n;
    }
    warp_sums[lane] = w;
  }
  __syncthreads();
  const uint32_t before = warp > 0 ? warp_sums[warp - 1] : 0u;
  if (total != nullptr) *total = warp_sums[31];
  if (kTrailingBarrier) __syncthreads();  // warp_sums may be reused by the caller
  return before + incl - v;
}

// Digit d of sh.sub[0..255], scanned from the top, with count(> d) < want <= count(>= d); done by
// the first warp (eight digits per lane).  Results in sh.digit / dabove / dcount.
__device__ __forceinline__ void sh_pick_digit(ShShared& sh, uint32_t want) {
  const int lane = threadIdx.x & 31;
  if (threadIdx.x < 32) {
    uint32_t c[8], mine = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) { c[k] = sh.sub[255 - 8 * lane - k]; mine += c[k]; }
    uint32_t incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t n = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += n;
    }
    uint32_t run = incl - mine;
    if (run < want && want <= incl) {
      bool found = false;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        if (!found && run + c[k] >= want) {
          sh.digit = 255 - 8 * lane - k; sh.dabove = run; sh.dcount = c[k];
          found = true;
        }
        run += c[k];
      }
    }
  }
  __syncthreads();
}

__global__ void __launch_bounds__(kShThreads, 1)
topk_select_hist_kernel(const float* __restrict__ scores, int64_t score_stride,
                        const int32_t* __restrict__ seq_lens, const int32_t* __restrict__ block_table,
                        int64_t bt_stride, int32_t* __restrict__ out, int64_t out_stride,
                        int max_pages, uint32_t* __restrict__ ghist, const __grid_constant__ RowSend xs, int32_t* status) {
  extern __shared__ float row_s[];
  __shared__ ShShared sh;
  cg::cluster_group cluster = cg::this_cluster();
  const int csize = (int)cluster.num_blocks();   // CTAs per request: 1, 2 or 4
  const int crank = (int)cluster.block_rank();

  const int b = blockIdx.x / csize;
  const int tid = threadIdx.x;
  int len = seq_lens[b];
  len = max(0, min(len, max_pages * kPage));
  int32_t* out_row = out + (size_t)b * out_stride;
  const int32_t* table = block_table + (size_t)b * bt_stride;
  const float* row = scores + (size_t)b * score_stride;
  const int n_pages = (len + kPage - 1) / kPage;
  const bool table_staged = n_pages <= kShTableCap;
  auto slot_of = [&](int i) -> int32_t {
    return (table_staged ? sh.table[i >> 6] : __ldg(table + (i >> 6))) * kPage + (i & 63);
  };
  // inputs of the caller only: safe before the dependency wait
  if (table_staged) {
    for (int i = tid; i < n_pages; i += kShThreads) sh.table[i] = table[i];
  }
  if (tid == 0) {
    sh.in_edge = 0xFFFFFFFFu; sh.edge = 0; sh.above = 0; sh.emit_cnt = 0; sh.last_n = 0;
    sh.dcount = 0xFFFFFFFFu;
  }
  if (tid < 256) sh.sub[tid] = 0;   // first CTA: digit histogram of the candidates, filled as they arrive
  // The successor (the attention kernel) reads nothing before its own wait; nothing is written
  // here before ours: the output row may still be read by the kernel before us in the stream.
  ptx::launch_dependents();
  ptx::grid_dependency_wait();

  // Head-sharded layers: the first CTA sends the finished row to the peers' staging buffers, while
  // other requests are still being selected (the take side is index_rows_exchange_kernel).
  auto send_row = [&]() {
    if (xs.world > 1) {
      __syncthreads();
      send_row_pairs(xs, out_row, xs.row_offset + b);
    }
  };
  if (len <= kTopK) {  // every token is selected: no scores, no histogram (uniform over the cluster)
    __syncthreads();
    for (int i = crank * kShThreads + tid; i < kTopK; i += csize * kShThreads)
      out_row[i] = i < len ? slot_of(i) : -1;
    if (xs.world > 1) {
      if (csize > 1) cluster.sync();   // the other CTAs' part of the row
      if (crank == 0) send_row();
    }
    return;
  }

  // this CTA's segment [seg_lo, seg_hi) of the row (multiples of 4 keep the 16-byte loads aligned)
  const int seg = ((len + csize - 1) / csize + 3) & ~3;
  const int seg_lo = min(len, crank * seg), seg_hi = min(len, seg_lo + seg);
  const int seg_len = seg_hi - seg_lo;
  const bool staged = seg <= kShRowCap;
  const bool vec = (reinterpret_cast<uintptr_t>(row) & 15u) == 0;

  // ---- (1) histogram -> boundary bin, while the slice travels into shared memory ----------------
  // thread t owns bins 4095-4t .. 4092-4t (one 16-byte load), so thread order is rank order
  uint4* g4 = reinterpret_cast<uint4*>(ghist + (size_t)b * kHistBins);
  const uint4 h = __ldcg(g4 + (kHistBins / 4 - 1 - tid));
  // a staged slice is kept as order-preserving KEYS: the sweeps below then only compare integers
  uint32_t* key_s = reinterpret_cast<uint32_t*>(row_s);
  const int n4s = staged && vec ? (seg_len & ~3) : 0;   // elements handled four at a time
  if (staged) {
    for (int i = tid * 4; i < n4s; i += kShThreads * 4) {
      const float4 q = __ldcg(reinterpret_cast<const float4*>(row + seg_lo + i));
      *reinterpret_cast<uint4*>(key_s + i) = make_uint4(sh_key(q.x), sh_key(q.y), sh_key(q.z), sh_key(q.w));
    }
    for (int i = n4s + tid; i < seg_len; i += kShThreads) key_s[i] = sh_key(__ldcg(row + seg_lo + i));
  }
  {
    const uint32_t mine = h.x + h.y + h.z + h.w;
    const uint32_t excl = sh_block_excl_scan<false>(mine, sh.warp_sums, nullptr);   // barrier below
    if (excl < (uint32_t)kTopK && (uint32_t)kTopK <= excl + mine) {
      const uint32_t c[4] = {h.w, h.z, h.y, h.x};   // highest bin first
      uint32_t run = excl;
      bool found = false;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (!found && run + c[k] >= (uint32_t)kTopK) {
          sh.edge = (uint32_t)(kHistBins - 1 - 4 * tid - k); sh.above = run; sh.in_edge = c[k];
          found = true;
        }
        run += c[k];
      }
    }
  }
  __syncthreads();   // boundary known; staged slice complete
  const uint32_t edge = sh.edge, above = sh.above, in_edge = sh.in_edge;
  if (in_edge == 0xFFFFFFFFu) {   // the histogram does not hold this row (workspace not zeroed?)
    if (tid == 0 && crank == 0) raise_status(status, DSA_STATUS_TOPK_COUNT);
    if (crank == 0) send_row();   // flagged; the peers still get a row, so that none of them waits
    return;                       // uniform over the cluster: every CTA read the same histogram
  }
  // A cluster of one or two meets only once more (after the writing pass).  Its first CTA's digit
  // histogram must be zero before a peer adds to it: arrive here, wait before the writing pass --
  // by then every CTA has long arrived, so the wait costs nothing.
  const bool exchange = csize > 2;
  if (!exchange) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  const uint32_t need = (uint32_t)kTopK - above;   // elements wanted from the boundary bin (>= 1)
  const bool few = in_edge <= (uint32_t)kShCandCap;
  auto key_at = [&](int i) -> uint32_t { return staged ? key_s[i - seg_lo] : sh_key(__ldcg(row + i)); };
  // key > hi_edge: above the boundary bin; key - lo_edge < 2^20 (unsigned): inside it
  const uint32_t lo_edge = edge << kShBinShift, hi_edge = lo_edge | 0xFFFFFu;

  // ---- (2) classification ---------------------------------------------------------------------------
  // A thread owns four consecutive elements per step of 4096 (at most 11 steps of a staged slice)
  // plus at most one element of the ragged end: one pass turns them into two bit masks (bit 4 s + e
  // for element e of step s, bit 63 for the ragged one), kept in registers for the writing pass.
  // A streamed slice (too long to stage) is swept from L2 twice instead.
  const bool fast = staged && seg_len <= 44 * kShThreads + 3 * kShThreads && (seg_len - n4s) <= kShThreads;
  uint64_t sel_mask = 0, cnd_mask = 0;
  uint32_t n_sel = 0, n_cnd = 0;
  if (fast) {
    int step = 0;
    for (int i = tid * 4; i < n4s; i += kShThreads * 4, ++step) {
      const uint4 k = *reinterpret_cast<const uint4*>(key_s + i);
      const uint32_t ks[4] = {k.x, k.y, k.z, k.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        sel_mask |= (uint64_t)(ks[e] > hi_edge) << (4 * step + e);
        cnd_mask |= (uint64_t)(ks[e] - lo_edge < 0x100000u) << (4 * step + e);
      }
    }
    if (n4s + tid < seg_len) {
      const uint32_t k = key_s[n4s + tid];
      sel_mask |= (uint64_t)(k > hi_edge) << 63;
      cnd_mask |= (uint64_t)(k - lo_edge < 0x100000u) << 63;
    }
    n_sel = (uint32_t)__popcll(sel_mask);
    n_cnd = (uint32_t)__popcll(cnd_mask);
  } else {
    for (int i = seg_lo + tid; i < seg_hi; i += kShThreads) {
      const uint32_t k = key_at(i);
      n_sel += k > hi_edge;
      n_cnd += k - lo_edge < 0x100000u;
    }
  }
  uint32_t totals = 0;
  const uint32_t excl = sh_block_excl_scan<false>(n_sel | (n_cnd << 16), sh.warp_sums, &totals);   // cluster barrier below
  // (a CTA holds at most 45056 staged elements, a streamed slice counts below 65536 per field only
  //  when it is shorter than that: longer streamed slices are rejected by the launcher)
  //
  // Places in the output row and in the candidate list.  Both totals of the ROW are known from
  // the histogram (`above`, `in_edge`), so a cluster of two needs no exchange: the first CTA fills
  // both lists from the front, the second from the back.  A cluster of four exchanges the CTAs'
  // totals through distributed shared memory.  In both cases the totals go to the first CTA, which
  // checks them against the histogram once the cluster has met.
  if (exchange) {
    if (tid < csize) {   // publish this CTA's totals in every CTA of the cluster
      ShShared* peer = cluster.map_shared_rank(&sh, tid);
      peer->peer_sel[crank] = totals & 0xFFFFu;
      peer->peer_cnd[crank] = totals >> 16;
    }
    cluster.sync();
  } else {
    if (tid == 0) {
      ShShared* peer = cluster.map_shared_rank(&sh, 0);
      peer->peer_sel[crank] = totals & 0xFFFFu;
      peer->peer_cnd[crank] = totals >> 16;
    }
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  }
  // sel_at / cnd_at: this thread's first place; `dir` +1 from the front, -1 (as unsigned) from the back
  uint32_t sel_at = excl & 0xFFFFu, cnd_at = excl >> 16;
  uint32_t dir = 1u;
  if (exchange) {
    for (int r = 0; r < crank; ++r) { sel_at += sh.peer_sel[r]; cnd_at += sh.peer_cnd[r]; }
  } else if (crank == 1) {
    sel_at = above - 1u - sel_at;      // wraps past zero only with inconsistent counts: the bound
    cnd_at = in_edge - 1u - cnd_at;    // checks below then skip the write
    dir = 0xFFFFFFFFu;
  }

  // ---- (3) writing pass: selected elements to their places, boundary bin to the candidate list ---
  ShShared* first = cluster.map_shared_rank(&sh, 0);
  if (fast) {
    // element of mask bit `bit`, as a position in the row
    auto position = [&](int bit) -> int {
      return bit == 63 ? seg_lo + n4s + tid : seg_lo + tid * 4 + (bit >> 2) * (kShThreads * 4) + (bit & 3);
    };
    while (sel_mask) {
      const int bit = __ffsll((long long)sel_mask) - 1;
      sel_mask &= sel_mask - 1;
      if (sel_at < above) out_row[sel_at] = slot_of(position(bit));
      sel_at += dir;
    }
    while (few && cnd_mask) {
      const int bit = __ffsll((long long)cnd_mask) - 1;
      cnd_mask &= cnd_mask - 1;
      const int i = position(bit);
      if (cnd_at < in_edge) {
        const uint32_t k = key_s[i - seg_lo];
        first->cand_key[cnd_at] = k;
        first->cand_idx[cnd_at] = (uint32_t)i;
        atomicAdd(&first->sub[(k >> 12) & 255u], 1u);   // first pass of (4): key bits 12..19
      }
      cnd_at += dir;
    }
  } else {
    for (int i = seg_lo + tid; i < seg_hi; i += kShThreads) {
      const uint32_t k = key_at(i);
      if (k > hi_edge) {
        if (sel_at < above) out_row[sel_at] = slot_of(i);
        sel_at += dir;
      } else if (k - lo_edge < 0x100000u) {
        if (few && cnd_at < in_edge) {
          first->cand_key[cnd_at] = k;
          first->cand_idx[cnd_at] = (uint32_t)i;
          atomicAdd(&first->sub[(k >> 12) & 255u], 1u);
        }
        cnd_at += dir;
      }
    }
  }
  cluster.sync();   // candidates and totals are in the first CTA's shared memory; the peers are done
  if (crank != 0) return;
  if (tid < kHistBins / 4) g4[tid] = make_uint4(0u, 0u, 0u, 0u);   // every CTA of the cluster has read it
  uint32_t nc = 0, sel_all = 0;
  for (int r = 0; r < csize; ++r) { nc += sh.peer_cnd[r]; sel_all += sh.peer_sel[r]; }
  if (sel_all != above || nc != in_edge) {
    // the histogram is not this row's (junk in the workspace): the places above were not the
    // elements' own, and candidate entries may be missing -- flag the call and leave the row
    if (tid == 0) raise_status(status, DSA_STATUS_TOPK_COUNT);
    send_row();
    return;
  }

  // ---- (4) the first CTA chooses `need` elements of the boundary bin -----------------------------
  auto emit = [&](int i) {
    const uint32_t p = above + atomicAdd(&sh.emit_cnt, 1u);
    if (p < (uint32_t)kTopK) out_row[p] = slot_of(i);
  };
  if (few) {
    nc = min(nc, (uint32_t)kShCandCap);
    if (need >= nc) {
      for (uint32_t j = tid; j < nc; j += kShThreads) emit((int)sh.cand_idx[j]);
    } else {
      // composite = low 20 key bits, then ~position (the lower position wins a tie)
      auto composite = [&](uint32_t j) -> uint64_t {
        return ((uint64_t)(sh.cand_key[j] & 0xFFFFFu) << 32) | (uint64_t)(~sh.cand_idx[j]);
      };
      uint64_t pfx = 0, msk = 0;
      uint32_t want = need;
#pragma unroll 1
      for (int pass = 0; pass < 7; ++pass) {
        const int shift = pass < 6 ? 44 - 8 * pass : 0;
        if (pass > 0) {   // (the first pass's histogram was filled while the candidates arrived)
          if (tid < 256) sh.sub[tid] = 0;
          if (tid == 0) sh.dcount = 0xFFFFFFFFu;
          __syncthreads();
          for (uint32_t j = tid; j < nc; j += kShThreads) {
            const uint64_t cj = composite(j);
            if ((cj & msk) == pfx) atomicAdd(&sh.sub[(uint32_t)(cj >> shift) & 255u], 1u);
          }
          __syncthreads();
        }
        sh_pick_digit(sh, want);
        const uint32_t d = sh.digit, da = sh.dabove, dc = sh.dcount;
        if (dc == 0xFFFFFFFFu) {   // cannot happen with consistent counts
          if (tid == 0) raise_status(status, DSA_STATUS_TOPK_COUNT);
          break;
        }
        const bool take_all = dc == want - da;
        // A boundary digit with a handful of candidates (the usual case after one pass: a few
        // hundred candidates over 256 digits) is settled at once: they are collected, and each
        // ranks itself among them.
        const bool settle = !take_all && dc <= 32u;
        for (uint32_t j = tid; j < nc; j += kShThreads) {
          const uint64_t cj = composite(j);
          if ((cj & msk) != pfx) continue;
          const uint32_t dg = (uint32_t)(cj >> shift) & 255u;
          if (dg > d || (take_all && dg == d)) emit((int)sh.cand_idx[j]);
          else if (settle && dg == d) sh.last[atomicAdd(&sh.last_n, 1u) & 31u] = j;
        }
        if (take_all) break;
        if (settle) {
          __syncthreads();
          if (tid < dc) {
            const uint64_t cj = composite(sh.last[tid]);
            uint32_t rank = 0;
            for (uint32_t k = 0; k < dc; ++k) rank += composite(sh.last[k]) > cj;
            if (rank < want - da) emit((int)sh.cand_idx[sh.last[tid]]);
          }
          break;
        }
        want -= da;
        pfx |= (uint64_t)d << shift;
        msk |= 255ull << shift;
        __syncthreads();   // everyone has read the digit before it is reset
      }
    }
  } else {
    // radix descent over the whole row (L2) for the exact threshold key inside the boundary bin,
    // then the ties in position order
    uint32_t pfx = edge << kShBinShift, msk = 0xFFFu << kShBinShift, want = need;
#pragma unroll 1
    for (int pass = 0; pass < 3; ++pass) {
      const int shift = pass == 0 ? 12 : (pass == 1 ? 4 : 0);
      const uint32_t dmask = pass == 2 ? 15u : 255u;
      if (tid < 256) sh.sub[tid] = 0;
      if (tid == 0) sh.dcount = 0xFFFFFFFFu;
      __syncthreads();
      for (int i = tid; i < len; i += kShThreads) {
        const uint32_t k = sh_key(__ldcg(row + i));
        if ((k & msk) == pfx) atomicAdd(&sh.sub[(k >> shift) & dmask], 1u);
      }
      __syncthreads();
      sh_pick_digit(sh, want);
      if (sh.dcount == 0xFFFFFFFFu) {
        if (tid == 0) raise_status(status, DSA_STATUS_TOPK_COUNT);
        break;
      }
      want -= sh.dabove;
      pfx |= sh.digit << shift;
      msk |= dmask << shift;
      __syncthreads();
    }
    const uint32_t thresh = pfx;   // key of the last selected element; `want` copies of it are taken
    for (int i = tid; i < len; i += kShThreads) {
      const uint32_t k = sh_key(__ldcg(row + i));
      if ((k >> kShBinShift) == edge && k > thresh) emit(i);
    }
    uint32_t running = 0;
    for (int base = 0; base < len && running < want; base += kShThreads * 4) {
      const int i = base + tid * 4;
      uint32_t eq = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (i + e < len && sh_key(__ldcg(row + i + e)) == thresh) eq |= 1u << e;
      uint32_t block_total = 0;
      uint32_t rank = running + sh_block_excl_scan((uint32_t)__popc(eq), sh.warp_sums, &block_total);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if ((eq >> e) & 1u) {
          if (rank < want) emit(i + e);
          ++rank;
        }
      }
      running += block_total;
    }
  }
  __syncthreads();
  if (tid == 0 && sh.emit_cnt != need) raise_status(status, DSA_STATUS_TOPK_COUNT);
  send_row();
}

// CTAs per request: as many as fit in one wave, more when a CTA's share of the longest possible
// row would not fit the staging buffer (a staged slice is read from L2 once).
static int sh_cluster_size(int batch, int max_len) {
  const int sms = sm_count();
  int c = batch * 4 <= sms ? 4 : (batch * 2 <= sms ? 2 : 1);
  while (c < 4 && (max_len + c - 1) / c > kShRowCap) c *= 2;
  return c;
}

// Rows whose slice per CTA could not be counted in 16 bits when streamed are left to the
// histogram-free selection kernel.
bool topk_select_hist_supports(int batch, int max_pages) {
  const int c = sh_cluster_size(batch, max_pages * kPage);
  const int64_t seg = ((int64_t)max_pages * kPage + c - 1) / c;
  return batch <= kHistMaxBatch && (seg <= kShRowCap || seg < 65536);
}

cudaError_t launch_topk_select_hist(const float* scores, int64_t score_stride, const int32_t* seq_lens,
                                    const int32_t* block_table, int64_t bt_stride, int32_t* out,
                                    int64_t out_stride, int batch, int max_pages, uint32_t* ghist,
                                    const RowSend* send, int32_t* status, cudaStream_t stream) {
  static std::atomic<uint64_t> smem_opted{0};
  {
    cudaError_t e = opt_in_dynamic_smem(reinterpret_cast<const void*>(topk_select_hist_kernel),
                                        sizeof(float) * kShRowCap, smem_opted);
    if (e != cudaSuccess) return e;
  }
  const int csize = sh_cluster_size(batch, max_pages * kPage);
  const int seg_max = (((max_pages * kPage + csize - 1) / csize) + 3) & ~3;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(batch * csize));
  cfg.blockDim = dim3(kShThreads);
  cfg.dynamicSmemBytes = sizeof(float) * (size_t)min(kShRowCap, max(seg_max, 4));
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
  RowSend xs = {};
  if (send != nullptr) xs = *send;
  return cudaLaunchKernelEx(&cfg, topk_select_hist_kernel, scores, score_stride, seq_lens,
                            block_table, bt_stride, out, out_stride, max_pages, ghist, xs, status);
}

}  // namespace dsa
