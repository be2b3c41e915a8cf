// FP8 indexer, scorer and top-2048 selection in ONE kernel (decode shapes).
//
//   score[b,t] = scale[t] * sum_h w[b,h] * relu( q[b,h,:] . k[t,:] )         (indexer_baseline.py:75-80)
//   topk[b,:]  = slots of the 2048 largest scores of request b, -1 padded     (indexer_baseline.py:60, :82-90)
//
// The scorer alone streams the key cache at the HBM rate; a selection kernel launched after it is
// a chain of latencies that starts only when the stream has ended.  Here the selection rides on
// the stream instead:
//
//   * work is cut into CHUNKS of 8 tiles (1024 tokens) of one request, numbered request by
//     request, and handed out through one global counter: all CTAs work on the same few requests
//     at any time, so requests are completed one after the other while the stream goes on, and a
//     slow SM simply takes fewer chunks;
//   * the epilogue warps, which hold every score in a register anyway, count it into a 4096-bin
//     histogram over the top 12 bits of its order-preserving key (shared memory, added to the
//     request's histogram in global memory at the end of the chunk: a few hundred reductions);
//   * the CTA that completes the LAST chunk of a request (an arrival counter -- nobody waits)
//     selects for that request while the others keep streaming: boundary bin from the histogram,
//     one sweep over the score row (L2) that emits every element above the boundary bin and
//     collects the few hundred inside it, then an exact radix selection among those by
//     (key, lower position first).  Rows whose boundary bin holds more than 2048 elements (flat
//     rows, mass ties) take a radix descent over the row instead;
//   * requests of at most 2048 tokens are emitted whole by whichever CTA draws their chunk.
//
// Pipeline inside a CTA as in the stand-alone scorer: warp 0 = TMA producer (chunk draw, page
// lookup one chunk ahead, 2-D TMA box + scale copy per page into a 4-deep ring), warp 1 = tcgen05
// issuer (M=128 tokens x N=64 heads x K=32, four TMEM accumulators), warps 2-5 = epilogue.  The
// roles communicate through the ring only: every stage carries a small descriptor (tile, chunk
// boundaries, end marker).  Two CTAs per SM.  Every wait is bounded, including the epilogue warps'
// own group barrier.
#include "common.cuh"
#include "ptx.cuh"
#include "tmap.cuh"

namespace dsa {

constexpr int kFuStages = 4;
constexpr int kFuAcc = 4;
constexpr int kFuTile = 128;
constexpr int kFuThreads = 192;
constexpr int kFuEpi = 128;                 // epilogue threads (warps 2..5)
constexpr int kFuChunkTiles = 8;
constexpr int kFuTmemCols = 256;            // 4 accumulators x 64 fp32 columns
constexpr int kFuTileDataBytes = 2 * kPageDataBytes;
constexpr int kFuBinShift = 20;             // bin = top 12 bits of the ordered key
constexpr int kFuCandCap = 2048;
constexpr uint32_t kFuIdesc = ptx::idesc(ptx::kFmtE4M3, ptx::kFmtE4M3, false, false, 128, 64);

enum { kFuTileStage = 0, kFuShortRow = 1, kFuEnd = 2 };

struct FuMeta {
  int kind;     // kFuTileStage / kFuShortRow / kFuEnd
  int b;        // request
  int tile;     // tile index inside the request
  int first;    // first tile of a chunk: new q, new weights
  int count;    // tiles in this chunk (valid on the first tile)
  int len;      // clamped length of the request
  int chunks;   // chunks of the request
  int pad;
};

struct FuShared {
  // data[stage] and q[slot] sit in the 1024-byte aligned dynamic region before this struct
  alignas(16) uint32_t hist[kFusedBins];   // per chunk; during a selection: candidate keys | positions
  alignas(16) uint32_t sub[256];
  float scale[kFuStages][kFuTile];
  FuMeta meta[kFuStages];
  int cprefix[kFusedMaxBatch + 1];         // chunks before request b
  int len[kFusedMaxBatch];                 // clamped lengths
  int partial[kFuThreads];
  uint32_t wsum[4];
  uint32_t edge, above, in_edge, emit_cnt, cand_cnt, is_last, digit, dabove, dcount;
  uint64_t full[kFuStages], empty[kFuStages];
  uint64_t qfull[2], qempty[2];
  uint64_t accfull[kFuAcc], accempty[kFuAcc];
  uint64_t group;                          // barrier of the four epilogue warps
  uint32_t tmem_base;
  volatile int abort_flag;
};

constexpr size_t kFuDynBytes = 1024 + (size_t)kFuStages * kFuTileDataBytes + 2 * kPageDataBytes +
                               sizeof(FuShared);

__device__ __forceinline__ int fu_chunks_of(int len) {
  if (len <= kTopK) return 1;   // emitted whole (an empty request too: 2048 x -1)
  const int tiles = (len + kFuTile - 1) / kFuTile;
  return (tiles + kFuChunkTiles - 1) / kFuChunkTiles;
}

// Largest b with prefix[b] <= w (prefix is non-decreasing, prefix[batch] > w).
__device__ __forceinline__ int fu_locate(const int* prefix, int batch, int w) {
  int lo = 0, hi = batch;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (prefix[mid] <= w) lo = mid; else hi = mid;
  }
  return lo;
}

__device__ __forceinline__ uint32_t fu_key(float v) { return float_to_ordered(fmaxf(v, kScoreFloor)); }

__global__ void __launch_bounds__(kFuThreads, 2)
indexer_topk_fused_kernel(const __grid_constant__ CUtensorMap tmap_k,
                          const __grid_constant__ CUtensorMap tmap_q,
                          const uint8_t* __restrict__ k_cache, const float* __restrict__ weights,
                          const int32_t* __restrict__ seq_lens,
                          const int32_t* __restrict__ block_table, int64_t bt_stride,
                          float* scores, int64_t score_stride, int32_t* __restrict__ out,
                          int64_t out_stride, int batch, int num_pages, int max_pages,
                          uint32_t* ctl, uint32_t* ghist, int32_t* status) {
  extern __shared__ unsigned char dyn_raw[];
  const uint32_t raw_addr = smem_u32(dyn_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  unsigned char* base = dyn_raw + pad;
  const uint32_t data_addr = raw_addr + pad;                          // kFuStages x 16 KB
  const uint32_t q_addr = data_addr + kFuStages * kFuTileDataBytes;    // 2 x 8 KB
  FuShared& sh = *reinterpret_cast<FuShared*>(base + kFuStages * kFuTileDataBytes + 2 * kPageDataBytes);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  // set-up that reads nothing from global memory: it may overlap the tail of the kernel before us
  if (warp == 0) {
    if (lane == 0) {
      for (int i = 0; i < kFuStages; ++i) {
        ptx::mbar_init(smem_u32(&sh.full[i]), 1);
        ptx::mbar_init(smem_u32(&sh.empty[i]), 1 + 4);  // MMA issuer + 4 epilogue warps
      }
      for (int i = 0; i < 2; ++i) {
        ptx::mbar_init(smem_u32(&sh.qfull[i]), 1);
        ptx::mbar_init(smem_u32(&sh.qempty[i]), 1);
      }
      for (int i = 0; i < kFuAcc; ++i) {
        ptx::mbar_init(smem_u32(&sh.accfull[i]), 1);
        ptx::mbar_init(smem_u32(&sh.accempty[i]), 4);
      }
      ptx::mbar_init(smem_u32(&sh.group), 4);
      ptx::fence_barrier_init();
      ptx::prefetch_tensormap(&tmap_k);
      ptx::prefetch_tensormap(&tmap_q);
      sh.abort_flag = 0;
    }
    __syncwarp();
    ptx::tmem_alloc(smem_u32(&sh.tmem_base), kFuTmemCols);
    ptx::tmem_relinquish();
  }
  for (int i = tid; i < kFusedBins; i += kFuThreads) sh.hist[i] = 0;
  ptx::grid_dependency_wait();  // the inputs, and the rows we write, may belong to the kernel before us
  ptx::launch_dependents();     // the next kernel may run its own set-up; it waits for our completion

  // ---- chunks per request -> exclusive prefix (all threads) -----------------------------------
  {
    const int chunk = (batch + kFuThreads - 1) / kFuThreads;
    const int lo = min(batch, tid * chunk), hi = min(batch, lo + chunk);
    int sum = 0;
    for (int b = lo; b < hi; ++b) {
      const int len = max(0, min(seq_lens[b], max_pages * kPage));
      sh.len[b] = len;
      sum += fu_chunks_of(len);
    }
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    if (lane == 31) sh.partial[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      const int nw = kFuThreads / 32;
      int wsum = lane < nw ? sh.partial[lane] : 0, wincl = wsum;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, wincl, o);
        if (lane >= o) wincl += up;
      }
      if (lane < nw) sh.partial[lane] = wincl - wsum;   // chunks before this warp's requests
      if (lane == nw - 1) sh.cprefix[batch] = wincl;
    }
    __syncthreads();
    int run = sh.partial[warp] + incl - sum;
    for (int b = lo; b < hi; ++b) {
      sh.cprefix[b] = run;
      run += fu_chunks_of(sh.len[b]);
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();

  const int total_chunks = sh.cprefix[batch];
  const uint32_t tmem_base = sh.tmem_base;

#define FU_WAIT(bar, parity)                                   \
  if (!ptx::mbar_wait(smem_u32(&(bar)), (parity))) {           \
    sh.abort_flag = 1;                                         \
    raise_status(status, DSA_STATUS_WAIT_TIMEOUT);             \
  }

  if (warp == 0) {
    // ======================= producer =======================
    int stage = 0, phase = 0, qslot = 0, qphase = 0;
    auto draw = [&]() -> int {
      int c = 0;
      if (lane == 0) c = (int)atomicAdd(&ctl[kFusedCtlNext], 1u);
      return __shfl_sync(0xffffffffu, c, 0);
    };
    // A chunk as the producer sees it; lane i holds the raw page ids of its tile i.
    int c_b = 0, c_j0 = 0, c_count = -1, c_len = 0, c_chunks = 0, c_p0 = 0, c_p1 = -1;
    auto decode = [&](int c, int& b, int& j0, int& count, int& len, int& chunks, int& p0, int& p1) {
      b = 0; j0 = 0; len = 0; chunks = 0; p0 = 0; p1 = -1;
      if (c >= total_chunks) { count = -1; return; }
      b = fu_locate(sh.cprefix, batch, c);
      len = sh.len[b];
      chunks = sh.cprefix[b + 1] - sh.cprefix[b];
      if (len <= kTopK) { count = 0; return; }
      const int tiles = (len + kFuTile - 1) / kFuTile;
      j0 = (c - sh.cprefix[b]) * kFuChunkTiles;
      count = min(kFuChunkTiles, tiles - j0);
      if (lane < count) {
        const int ji = j0 + lane;
        const int n_pages = (len + kPage - 1) / kPage;
        const int32_t* row = block_table + (size_t)b * bt_stride + 2 * ji;
        p0 = row[0];
        // a request's second page of a tile exists iff 2 ji + 1 < n_pages (<= max_pages)
        p1 = (2 * ji + 1 < n_pages) ? row[1] : -1;
      }
    };
    decode(draw(), c_b, c_j0, c_count, c_len, c_chunks, c_p0, c_p1);
    int next_id = draw();
    for (;;) {
      // one lane reads the flag for the whole warp: the loop contains warp-wide shuffles
      if (__shfl_sync(0xffffffffu, (int)sh.abort_flag, 0)) break;
      if (c_count < 0) {   // no chunk left: tell the other roles
        if (lane == 0) {
          FU_WAIT(sh.empty[stage], phase ^ 1);
          sh.meta[stage].kind = kFuEnd;
          ptx::mbar_arrive(smem_u32(&sh.full[stage]));
        }
        break;
      }
      // the chunk after this one: its page ids travel while this chunk's copies are issued
      int n_b, n_j0, n_count, n_len, n_chunks, n_p0, n_p1;
      decode(next_id, n_b, n_j0, n_count, n_len, n_chunks, n_p0, n_p1);
      next_id = draw();
      if (c_count == 0) {
        if (lane == 0) {
          FU_WAIT(sh.empty[stage], phase ^ 1);
          FuMeta& m = sh.meta[stage];
          m.kind = kFuShortRow; m.b = c_b; m.len = c_len;
          ptx::mbar_arrive(smem_u32(&sh.full[stage]));
        }
        if (++stage == kFuStages) { stage = 0; phase ^= 1; }
      } else {
        for (int i = 0; i < c_count; ++i) {
          int a0 = __shfl_sync(0xffffffffu, c_p0, i);
          int a1 = __shfl_sync(0xffffffffu, c_p1, i);
          const bool second = 2 * (c_j0 + i) + 1 < (c_len + kPage - 1) / kPage;
          if (lane == 0 && !sh.abort_flag) {
            if (a0 < 0 || a0 >= num_pages) { raise_status(status, DSA_STATUS_BAD_PAGE); a0 = 0; }
            if (second && (a1 < 0 || a1 >= num_pages)) { raise_status(status, DSA_STATUS_BAD_PAGE); a1 = 0; }
            if (i == 0) {
              FU_WAIT(sh.qempty[qslot], qphase ^ 1);
              ptx::mbar_expect_tx(smem_u32(&sh.qfull[qslot]), kPageDataBytes);
              ptx::tma_load_2d(q_addr + qslot * kPageDataBytes, &tmap_q, 0, c_b * kIdxHeads,
                               smem_u32(&sh.qfull[qslot]));
              qslot ^= 1;
              if (qslot == 0) qphase ^= 1;
            }
            FU_WAIT(sh.empty[stage], phase ^ 1);
            FuMeta& m = sh.meta[stage];
            m.kind = kFuTileStage; m.b = c_b; m.tile = c_j0 + i; m.first = i == 0; m.count = c_count;
            m.len = c_len; m.chunks = c_chunks;
            const uint32_t bar = smem_u32(&sh.full[stage]);
            const uint32_t dst = data_addr + stage * kFuTileDataBytes;
            const uint32_t sdst = smem_u32(&sh.scale[stage][0]);
            ptx::mbar_expect_tx(bar, (second ? 2 : 1) * kPageBytes);
            ptx::tma_load_2d(dst, &tmap_k, 0, a0 * 66, bar);
            ptx::bulk_load_1d(sdst, k_cache + (size_t)a0 * kPageBytes + kPageDataBytes, 256, bar);
            if (second) {
              ptx::tma_load_2d(dst + kPageDataBytes, &tmap_k, 0, a1 * 66, bar);
              ptx::bulk_load_1d(sdst + 256, k_cache + (size_t)a1 * kPageBytes + kPageDataBytes, 256, bar);
            }
          }
          if (++stage == kFuStages) { stage = 0; phase ^= 1; }
          __syncwarp();
        }
      }
      c_b = n_b; c_j0 = n_j0; c_count = n_count; c_len = n_len; c_chunks = n_chunks;
      c_p0 = n_p0; c_p1 = n_p1;
    }
  } else if (warp == 1) {
    // ======================= MMA issuer =======================
    if (lane == 0) {
      int stage = 0, phase = 0, qslot = 0, qphase = 0, acc = 0, aphase = 0;
      bool have_q = false;
      uint32_t qbase = q_addr;
      // descriptor bits that never change: LBO = 16 B, SBO = 1024 B, version 1, 128-byte swizzle
      const uint64_t desc_hi = ptx::smem_desc_sw128(0, 16, 1024);
      for (;;) {
        FU_WAIT(sh.full[stage], phase);
        if (sh.abort_flag) break;
        const int kind = sh.meta[stage].kind, first = sh.meta[stage].first;
        if (kind == kFuEnd) break;
        if (kind == kFuShortRow) {
          ptx::mbar_arrive(smem_u32(&sh.empty[stage]));
        } else {
          if (first) {
            if (have_q) ptx::tc_commit(smem_u32(&sh.qempty[qslot ^ 1]));  // previous q: free once read
            FU_WAIT(sh.qfull[qslot], qphase);
            qbase = q_addr + qslot * kPageDataBytes;
            qslot ^= 1;
            if (qslot == 0) qphase ^= 1;
            have_q = true;
          }
          FU_WAIT(sh.accempty[acc], aphase ^ 1);
          if (sh.abort_flag) break;
          ptx::tc_fence_after();
          const uint64_t adesc = desc_hi | (uint64_t)((data_addr + stage * kFuTileDataBytes) >> 4);
          const uint64_t bdesc = desc_hi | (uint64_t)(qbase >> 4);
          const uint32_t d = tmem_base + acc * kIdxHeads;
#pragma unroll
          for (int k = 0; k < 4; ++k)  // K = 32 fp8 = 32 bytes per instruction -> +2 in 16 B units
            ptx::mma_f8(d, adesc + 2 * k, bdesc + 2 * k, kFuIdesc, k > 0);
          ptx::tc_commit(smem_u32(&sh.empty[stage]));
          ptx::tc_commit(smem_u32(&sh.accfull[acc]));
          if (++acc == kFuAcc) { acc = 0; aphase ^= 1; }
        }
        if (++stage == kFuStages) { stage = 0; phase ^= 1; }
      }
    }
    __syncwarp();
  } else {
    // ======================= epilogue + selection =======================
    const int ew = warp - 2;                 // warp inside the group
    const int et = ew * 32 + lane;           // thread inside the group
    const int quarter = warp & 3;            // TMEM lane quarter this warp may read
    const int rowi = quarter * 32 + lane;    // token row of the tile handled by this thread
    const uint32_t lt_mask = (1u << lane) - 1u;
    int stage = 0, phase = 0, acc = 0, aphase = 0;
    uint32_t gphase = 0;
    bool alive = true;

    // barrier of the 128 epilogue threads, bounded like every other wait
    auto group_sync = [&]() -> bool {
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(smem_u32(&sh.group));
      const bool ok = ptx::mbar_wait(smem_u32(&sh.group), gphase);
      gphase ^= 1u;
      if (!ok) {
        sh.abort_flag = 1;
        raise_status(status, DSA_STATUS_WAIT_TIMEOUT);
      }
      return ok;
    };
    // exclusive prefix of v over the group in thread order; two group barriers
    auto group_scan = [&](uint32_t v, uint32_t& excl) -> bool {
      uint32_t incl = v;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
      }
      if (lane == 31) sh.wsum[ew] = incl;
      if (!group_sync()) return false;
      uint32_t before = 0;
      for (int k = 0; k < ew; ++k) before += sh.wsum[k];
      excl = before + incl - v;
      return group_sync();   // wsum may be rewritten after this
    };
    // Digit selection over sh.sub[0..255], scanned from the top: the digit d with
    // count(digits > d) < want <= count(digits >= d).  Results in sh.digit / dabove / dcount.
    auto pick_digit = [&](uint32_t want) -> bool {
      const uint32_t c_hi = sh.sub[255 - 2 * et], c_lo = sh.sub[254 - 2 * et];
      uint32_t excl;
      if (!group_scan(c_hi + c_lo, excl)) return false;
      if (excl < want && want <= excl + c_hi + c_lo) {
        if (excl + c_hi >= want) {
          sh.digit = 255 - 2 * et; sh.dabove = excl; sh.dcount = c_hi;
        } else {
          sh.digit = 254 - 2 * et; sh.dabove = excl + c_hi; sh.dcount = c_lo;
        }
      }
      return group_sync();
    };

    // ---- selection for request b, run by the CTA that completed its last chunk ----------------
    auto select_row = [&](int b, int len) -> bool {
      const float* row = scores + (size_t)b * score_stride;
      const int32_t* table = block_table + (size_t)b * bt_stride;
      int32_t* out_row = out + (size_t)b * out_stride;
      auto slot_of = [&](int i) -> int32_t { return __ldg(table + (i >> 6)) * kPage + (i & 63); };
      auto emit = [&](int i) {
        const uint32_t p = atomicAdd(&sh.emit_cnt, 1u);
        if (p < (uint32_t)kTopK) out_row[p] = slot_of(i);
      };
      // (1) boundary bin.  Thread et owns the 32 bins [hi-31, hi], hi = 4095 - 32 et, so thread
      // order is rank order; the histogram is put back to zero for the next call.
      uint32_t c[32];
      {
        uint4* g4 = reinterpret_cast<uint4*>(ghist + (size_t)b * kFusedBins) + (kFusedBins / 4 - 8 - 8 * et);
#pragma unroll
        for (int v = 0; v < 8; ++v) {
          const uint4 q = __ldcg(g4 + v);
          c[4 * v] = q.x; c[4 * v + 1] = q.y; c[4 * v + 2] = q.z; c[4 * v + 3] = q.w;
        }
#pragma unroll
        for (int v = 0; v < 8; ++v) __stcg(g4 + v, make_uint4(0u, 0u, 0u, 0u));
      }
      uint32_t mine = 0;
#pragma unroll
      for (int k = 0; k < 32; ++k) mine += c[k];
      if (et == 0) {
        sh.in_edge = 0xFFFFFFFFu; sh.edge = 0; sh.above = 0; sh.emit_cnt = 0; sh.cand_cnt = 0;
      }
      uint32_t excl;
      if (!group_scan(mine, excl)) return false;
      if (excl < (uint32_t)kTopK && (uint32_t)kTopK <= excl + mine) {
        uint32_t run = excl;
        bool found = false;
#pragma unroll
        for (int k = 31; k >= 0; --k) {
          if (!found && run + c[k] >= (uint32_t)kTopK) {
            sh.edge = (uint32_t)(kFusedBins - 32 - 32 * et + k); sh.above = run; sh.in_edge = c[k];
            found = true;
          }
          run += c[k];
        }
      }
      if (!group_sync()) return false;
      const uint32_t edge = sh.edge, above = sh.above, in_edge = sh.in_edge;
      if (in_edge == 0xFFFFFFFFu) {   // the histogram does not hold this row (workspace not zeroed?)
        if (et == 0) raise_status(status, DSA_STATUS_TOPK_COUNT);
        return group_sync();
      }
      const uint32_t need = (uint32_t)kTopK - above;   // elements wanted from the boundary bin (>= 1)
      const bool few = in_edge <= (uint32_t)kFuCandCap;
      uint32_t* ck = sh.hist;                 // candidate keys
      uint32_t* ci = sh.hist + kFuCandCap;    // candidate positions

      // (2) one sweep over the row: emit what lies above the boundary bin, collect the bin itself.
      // Eight 16-byte loads per thread are in flight at a time (the sweep is bound by L2 latency).
      for (int base0 = 0; base0 < len; base0 += kFuEpi * 4 * 8) {
        float4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int i = base0 + (u * kFuEpi + et) * 4;
          v[u] = i < len ? __ldcg(reinterpret_cast<const float4*>(row + i))
                         : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int i = base0 + (u * kFuEpi + et) * 4;
          if (base0 + u * kFuEpi * 4 >= len) break;   // uniform over the group
          const float vals[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
          uint32_t key[4], sel[4], cnd[4], n_sel = 0, n_cnd = 0;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            key[e] = fu_key(vals[e]);
            const uint32_t bin = key[e] >> kFuBinShift;
            const bool in = i + e < len;
            sel[e] = __ballot_sync(0xffffffffu, in && bin > edge);
            cnd[e] = __ballot_sync(0xffffffffu, in && few && bin == edge);
            n_sel += __popc(sel[e]);
            n_cnd += __popc(cnd[e]);
          }
          if (n_sel) {
            uint32_t at = 0;
            if (lane == 0) at = atomicAdd(&sh.emit_cnt, n_sel);
            at = __shfl_sync(0xffffffffu, at, 0);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              if ((sel[e] >> lane) & 1u) {
                const uint32_t p = at + __popc(sel[e] & lt_mask);
                if (p < (uint32_t)kTopK) out_row[p] = slot_of(i + e);
              }
              at += __popc(sel[e]);
            }
          }
          if (n_cnd) {
            uint32_t at = 0;
            if (lane == 0) at = atomicAdd(&sh.cand_cnt, n_cnd);
            at = __shfl_sync(0xffffffffu, at, 0);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              if ((cnd[e] >> lane) & 1u) {
                const uint32_t p = at + __popc(cnd[e] & lt_mask);
                if (p < (uint32_t)kFuCandCap) { ck[p] = key[e]; ci[p] = (uint32_t)(i + e); }
              }
              at += __popc(cnd[e]);
            }
          }
        }
      }
      if (!group_sync()) return false;

      if (few) {
        // (3) exact choice of `need` among the nc candidates by the 52-bit composite
        // (low 20 key bits, then ~position: the lower position wins a tie), eight bits per pass.
        const uint32_t nc = min(sh.cand_cnt, (uint32_t)kFuCandCap);
        if (et == 0 && (nc != in_edge || sh.emit_cnt != above)) raise_status(status, DSA_STATUS_TOPK_COUNT);
        if (need >= nc) {
          for (uint32_t j = et; j < nc; j += kFuEpi) emit((int)ci[j]);
        } else {
          auto composite = [&](uint32_t j) -> uint64_t {
            return ((uint64_t)(ck[j] & 0xFFFFFu) << 32) | (uint64_t)(~ci[j]);
          };
          uint64_t pfx = 0, msk = 0;
          uint32_t want = need;
#pragma unroll 1
          for (int pass = 0; pass < 7; ++pass) {
            const int shift = pass < 6 ? 44 - 8 * pass : 0;
            sh.sub[et] = 0; sh.sub[et + kFuEpi] = 0;
            if (et == 0) sh.dcount = 0xFFFFFFFFu;
            if (!group_sync()) return false;
            for (uint32_t j = et; j < nc; j += kFuEpi) {
              const uint64_t cj = composite(j);
              if ((cj & msk) == pfx) atomicAdd(&sh.sub[(uint32_t)(cj >> shift) & 255u], 1u);
            }
            if (!group_sync()) return false;
            if (!pick_digit(want)) return false;
            const uint32_t d = sh.digit, da = sh.dabove, dc = sh.dcount;
            if (dc == 0xFFFFFFFFu) {   // cannot happen with consistent counts
              if (et == 0) raise_status(status, DSA_STATUS_TOPK_COUNT);
              break;
            }
            const bool take_all = dc == want - da;
            for (uint32_t j = et; j < nc; j += kFuEpi) {
              const uint64_t cj = composite(j);
              if ((cj & msk) != pfx) continue;
              const uint32_t dg = (uint32_t)(cj >> shift) & 255u;
              if (dg > d || (take_all && dg == d)) emit((int)ci[j]);
            }
            if (take_all) break;
            want -= da;
            pfx |= (uint64_t)d << shift;
            msk |= 255ull << shift;
            if (!group_sync()) return false;   // everyone has read the digit before it is reset
          }
        }
      } else {
        // (3') the boundary bin is too full (flat row, mass ties): radix descent over the row for
        // the exact threshold key inside the bin, then the ties in position order.
        uint32_t pfx = edge << kFuBinShift, msk = 0xFFFu << kFuBinShift, want = need;
        if (et == 0 && sh.emit_cnt != above) raise_status(status, DSA_STATUS_TOPK_COUNT);
#pragma unroll 1
        for (int pass = 0; pass < 3; ++pass) {
          const int shift = pass == 0 ? 12 : (pass == 1 ? 4 : 0);
          const uint32_t dmask = pass == 2 ? 15u : 255u;
          sh.sub[et] = 0; sh.sub[et + kFuEpi] = 0;
          if (et == 0) sh.dcount = 0xFFFFFFFFu;
          if (!group_sync()) return false;
          for (int i = et; i < len; i += kFuEpi) {
            const uint32_t k = fu_key(__ldcg(row + i));
            if ((k & msk) == pfx) atomicAdd(&sh.sub[(k >> shift) & dmask], 1u);
          }
          if (!group_sync()) return false;
          if (!pick_digit(want)) return false;
          if (sh.dcount == 0xFFFFFFFFu) {
            if (et == 0) raise_status(status, DSA_STATUS_TOPK_COUNT);
            break;
          }
          want -= sh.dabove;
          pfx |= sh.digit << shift;
          msk |= dmask << shift;
          if (!group_sync()) return false;   // everyone has read the digit before it is reset
        }
        const uint32_t thresh = pfx;   // key of the last selected element; `want` copies of it are taken
        for (int i = et; i < len; i += kFuEpi) {
          const uint32_t k = fu_key(__ldcg(row + i));
          if ((k >> kFuBinShift) == edge && k > thresh) emit(i);
        }
        uint32_t running = 0;
        for (int base0 = 0; base0 < len && running < want; base0 += kFuEpi * 4) {
          const int i = base0 + et * 4;
          uint32_t eq = 0;
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (i + e < len && fu_key(__ldcg(row + i + e)) == thresh) eq |= 1u << e;
          uint32_t excl2;
          if (!group_scan((uint32_t)__popc(eq), excl2)) return false;
          uint32_t rank = running + excl2;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            if ((eq >> e) & 1u) {
              if (rank < want) emit(i + e);
              ++rank;
            }
          }
          if (et == kFuEpi - 1) sh.dabove = excl2 + (uint32_t)__popc(eq);   // ties in this block
          if (!group_sync()) return false;
          running += sh.dabove;
          if (!group_sync()) return false;
        }
      }
      if (!group_sync()) return false;
      if (et == 0 && sh.emit_cnt != (uint32_t)kTopK) raise_status(status, DSA_STATUS_TOPK_COUNT);
      // the histogram doubles as the candidate store: zero for the next chunk
#pragma unroll
      for (int v = 0; v < kFusedBins / 4 / kFuEpi; ++v)
        reinterpret_cast<uint4*>(sh.hist)[v * kFuEpi + et] = make_uint4(0u, 0u, 0u, 0u);
      return group_sync();
    };

    // ---- chunk loop -----------------------------------------------------------------------------
    while (alive) {
      FU_WAIT(sh.full[stage], phase);
      if (sh.abort_flag) break;
      const FuMeta m = sh.meta[stage];
      if (m.kind == kFuEnd) break;
      if (m.kind == kFuShortRow) {
        // every cached token is selected: no scores needed
        const int32_t* table = block_table + (size_t)m.b * bt_stride;
        int32_t* out_row = out + (size_t)m.b * out_stride;
        for (int i = et; i < kTopK; i += kFuEpi)
          out_row[i] = i < m.len ? __ldg(table + (i >> 6)) * kPage + (i & 63) : -1;
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(smem_u32(&sh.empty[stage]));
        if (++stage == kFuStages) { stage = 0; phase ^= 1; }
        continue;
      }
      // a chunk of m.count tiles of request m.b, starting at tile m.tile
      float wreg[kIdxHeads];
      {
        const float4* wp = reinterpret_cast<const float4*>(weights + (size_t)m.b * kIdxHeads);
#pragma unroll
        for (int i = 0; i < kIdxHeads / 4; ++i) {
          const float4 v = __ldg(wp + i);
          wreg[4 * i] = v.x; wreg[4 * i + 1] = v.y; wreg[4 * i + 2] = v.z; wreg[4 * i + 3] = v.w;
        }
      }
      float* srow = scores + (size_t)m.b * score_stride;
      for (int i = 0; i < m.count && alive; ++i) {
        if (i > 0) {
          FU_WAIT(sh.full[stage], phase);
        }
        const float sc = sh.scale[stage][rowi];
        FU_WAIT(sh.accfull[acc], aphase);
        if (sh.abort_flag) { alive = false; break; }
        ptx::tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * kIdxHeads;
        float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          uint32_t r[16];
          ptx::tmem_ld16(taddr + cc * 16, r);
          ptx::tmem_wait_ld();
#pragma unroll
          for (int h = 0; h < 16; ++h)
            part[h & 3] = fmaf(wreg[cc * 16 + h], fmaxf(__uint_as_float(r[h]), 0.f), part[h & 3]);
        }
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          ptx::mbar_arrive(smem_u32(&sh.accempty[acc]));
          ptx::mbar_arrive(smem_u32(&sh.empty[stage]));
        }
        const int t = (m.tile + i) * kFuTile + rowi;
        const float val = ((part[0] + part[1]) + (part[2] + part[3])) * sc;
        if (t < m.len) {
          srow[t] = val;
          atomicAdd(&sh.hist[fu_key(val) >> kFuBinShift], 1u);
        }
        if (++stage == kFuStages) { stage = 0; phase ^= 1; }
        if (++acc == kFuAcc) { acc = 0; aphase ^= 1; }
      }
      if (!alive) break;
#ifdef FU_NO_CHUNKEND
      continue;
#endif
      // ---- end of the chunk: publish the histogram, count the arrival -------------------------
      if (!group_sync()) break;   // every count of this chunk is in sh.hist
      {
        uint32_t* g = ghist + (size_t)m.b * kFusedBins;
        uint4* h4 = reinterpret_cast<uint4*>(sh.hist);
#pragma unroll
        for (int v = 0; v < kFusedBins / 4 / kFuEpi; ++v) {
          const int q = v * kFuEpi + et;
          const uint4 cnt = h4[q];
          if (cnt.x | cnt.y | cnt.z | cnt.w) {
            if (cnt.x) atomicAdd(g + 4 * q, cnt.x);
            if (cnt.y) atomicAdd(g + 4 * q + 1, cnt.y);
            if (cnt.z) atomicAdd(g + 4 * q + 2, cnt.z);
            if (cnt.w) atomicAdd(g + 4 * q + 3, cnt.w);
            h4[q] = make_uint4(0u, 0u, 0u, 0u);
          }
        }
      }
      __threadfence();            // this thread's scores and counts are visible device-wide ...
      if (!group_sync()) break;   // ... for every thread of the group
      if (et == 0) {
        const uint32_t old = atomicAdd(&ctl[kFusedCtlDone + m.b], 1u);
        const uint32_t last = old + 1u == (uint32_t)m.chunks;
        if (last) ctl[kFusedCtlDone + m.b] = 0u;   // every arrival is in: ready for the next call
        __threadfence();
        sh.is_last = last;
      }
      if (!group_sync()) break;
#ifndef FU_NO_SELECT
      if (sh.is_last) {
        if (!select_row(m.b, m.len)) break;
      }
#endif
    }
  }
#undef FU_WAIT

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    if (sh.abort_flag) {
      // let bulk copies that were already issued land before the CTA's shared memory is released
      for (int i = 0; i < 64; ++i) __nanosleep(20000);
    }
    ptx::tmem_dealloc(tmem_base, kFuTmemCols);
    if (lane == 0) {
      // the last CTA to leave puts the chunk counter back to zero for the next call
      __threadfence();
      const uint32_t old = atomicAdd(&ctl[kFusedCtlExited], 1u);
      if (old + 1u == gridDim.x) {
        ctl[kFusedCtlNext] = 0u;
        ctl[kFusedCtlExited] = 0u;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------ host
cudaError_t launch_indexer_topk_fused(const void* q_fp8, const void* k_cache, const float* weights,
                                      const int32_t* seq_lens, const int32_t* block_table,
                                      int64_t bt_stride, float* scores, int64_t score_stride,
                                      int32_t* out, int64_t out_stride, int batch, int num_pages,
                                      int max_pages, uint32_t* ctl, uint32_t* ghist, int32_t* status,
                                      cudaStream_t stream) {
  if (batch > kFusedMaxBatch) return cudaErrorInvalidValue;
  static std::atomic<uint64_t> smem_opted{0};
  cudaError_t e = opt_in_dynamic_smem(reinterpret_cast<const void*>(indexer_topk_fused_kernel),
                                      kFuDynBytes, smem_opted);
  if (e != cudaSuccess) return e;
  CUtensorMap tmap_k, tmap_q;
  if (!make_tmap_2d_sw128(&tmap_k, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, k_cache, 128,
                          (uint64_t)num_pages * 66, 128, 64) ||
      !make_tmap_2d_sw128(&tmap_q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, q_fp8, 128,
                          (uint64_t)batch * kIdxHeads, 128, 64))
    return cudaErrorInvalidValue;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * sm_count()));
  cfg.blockDim = dim3(kFuThreads);
  cfg.dynamicSmemBytes = kFuDynBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled();
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, indexer_topk_fused_kernel, tmap_k, tmap_q,
                            static_cast<const uint8_t*>(k_cache), weights, seq_lens, block_table,
                            bt_stride, scores, score_stride, out, out_stride, batch, num_pages,
                            max_pages, ctl, ghist, status);
}

}  // namespace dsa
