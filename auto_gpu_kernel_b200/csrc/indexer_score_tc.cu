// FP8 indexer scorer on the 5th-generation tensor cores (tcgen05 kind::f8f6f4, TMEM accumulators).
//
//   score[b,t] = scale[t] * sum_h w[b,h] * relu( q[b,h,:] . k[t,:] )
// (reference arithmetic: indexer_baseline.py:75-80; kernels this replaces: score_kernel of
//  indexer_fused.py:80-158 and the Gluon _g_score_kernel of archive/fable/dsa_topk_indexer_*.py).
//
// Decode is bound by the HBM stream of the paged key cache (132 bytes per cached token), so the
// kernel is a persistent, warp-specialised pipeline that keeps many pages in flight per SM:
//
//   warp 0  producer : walks its share of (request, 128-token tile) work items, looks the two pages
//                      of a tile up in block_table (32 tiles per coalesced lookup) and issues, per
//                      page, one 2-D TMA box (64 rows x 128 B, 128-byte swizzle) for the keys and one
//                      256-byte bulk copy for the fp32 scales, into a 4-deep shared-memory ring;
//   warp 1  MMA      : per tile 4 x tcgen05.mma M=128 (tokens) x N=64 (heads) x K=32, A = key tile,
//                      B = the request's q (both K-major in shared memory), D in one of 4 TMEM
//                      accumulator slots; tcgen05.commit releases the ring slot and publishes D;
//   warps 2-5 epilogue: tcgen05.ld of the token's 64 head sums, relu, dot with w, times the token
//                      scale, one coalesced fp32 store per token.
//
// Two such CTAs run per SM (each uses half of the shared memory, registers and TMEM): the three
// roles are strictly serial instruction streams, and at 64 accumulator columns per tile their issue
// latency, not the tensor pipe, bounds one pipeline, so two independent pipelines per SM are needed
// to keep the HBM stream saturated.
// Work is split evenly in tiles (not requests) across CTAs using an in-kernel prefix sum of the
// device-resident seq_lens, so ragged batches balance without a host synchronisation.
// Every mbarrier wait is time-bounded; on expiry the CTA records DSA_STATUS_WAIT_TIMEOUT, lets
// copies in flight land, frees its TMEM and returns.
#include "common.cuh"
#include "ptx.cuh"
#include "tmap.cuh"

namespace dsa {

constexpr int kTcStages = 4;
constexpr int kTcAcc = 4;
constexpr int kTcTile = 128;
constexpr int kTcThreads = 192;
constexpr int kTcMaxBatch = 2048;
constexpr int kTcTmemCols = 256;            // 4 accumulators x 64 fp32 columns
constexpr int kTileDataBytes = 2 * kPageDataBytes;  // 16384
constexpr uint32_t kIdescF8 = ptx::idesc(ptx::kFmtE4M3, ptx::kFmtE4M3, false, false, 128, 64);

struct TcShared {
  // data[stage] and q[slot] sit in the 1024-byte aligned dynamic region before this struct
  alignas(16) uint32_t hist[kHistBins];   // kHist: counts of the current request's scores per key bin
  float scale[kTcStages][kTcTile];
  int prefix[kTcMaxBatch + 1];
  int partial[kTcThreads];
  uint64_t full[kTcStages], empty[kTcStages];
  uint64_t qfull[2], qempty[2];
  uint64_t accfull[kTcAcc], accempty[kTcAcc];
  uint64_t group;                          // kHist: barrier of the four epilogue warps
  uint32_t tmem_base;
  volatile int abort_flag;
};

constexpr size_t kTcDynBytes = 1024 + (size_t)kTcStages * kTileDataBytes + 2 * kPageDataBytes +
                               sizeof(TcShared);

__device__ __forceinline__ int tiles_of(int len, int max_pages, int skip_short) {
  len = max(0, min(len, max_pages * kPage));
  if (skip_short && len <= kTopK) return 0;
  return (len + kTcTile - 1) / kTcTile;
}

// Largest b with prefix[b] <= w (prefix is non-decreasing, prefix[batch] > w).
__device__ __forceinline__ int locate(const int* prefix, int batch, int w) {
  int lo = 0, hi = batch;
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (prefix[mid] <= w) lo = mid; else hi = mid;
  }
  return lo;
}

// kHist: the epilogue also counts every score into a 4096-bin histogram over the top 12 bits of its
// order-preserving key (shared memory, added to the request's histogram in `ghist` when the CTA
// moves on to another request): the selection kernel then starts from the finished histogram.
template <bool kHist>
__global__ void __launch_bounds__(kTcThreads, 2)
indexer_score_tc_kernel(const __grid_constant__ CUtensorMap tmap_k,
                        const __grid_constant__ CUtensorMap tmap_q,
                        const uint8_t* __restrict__ k_cache, const float* __restrict__ weights,
                        const int32_t* __restrict__ seq_lens,
                        const int32_t* __restrict__ block_table, int64_t bt_stride,
                        float* __restrict__ scores, int64_t score_stride, int batch, int num_pages,
                        int max_pages, int skip_short, uint32_t* __restrict__ minmax,
                        uint32_t* __restrict__ ghist, int32_t* status) {
  extern __shared__ unsigned char dyn_raw[];
  const uint32_t raw_addr = smem_u32(dyn_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  unsigned char* base = dyn_raw + pad;
  const uint32_t data_addr = raw_addr + pad;                          // kTcStages x 16 KB
  const uint32_t q_addr = data_addr + kTcStages * kTileDataBytes;      // 2 x 8 KB
  TcShared& sh = *reinterpret_cast<TcShared*>(base + kTcStages * kTileDataBytes + 2 * kPageDataBytes);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  // set-up that reads nothing from global memory, so that it can overlap the tail of the kernel
  // before us in the stream (programmatic dependent launch)
  if (warp == 0) {
    if (lane == 0) {
      for (int i = 0; i < kTcStages; ++i) {
        ptx::mbar_init(smem_u32(&sh.full[i]), 1);
        ptx::mbar_init(smem_u32(&sh.empty[i]), 1 + 4);  // MMA commit + 4 epilogue warps
      }
      for (int i = 0; i < 2; ++i) {
        ptx::mbar_init(smem_u32(&sh.qfull[i]), 1);
        ptx::mbar_init(smem_u32(&sh.qempty[i]), 1);
      }
      for (int i = 0; i < kTcAcc; ++i) {
        ptx::mbar_init(smem_u32(&sh.accfull[i]), 1);
        ptx::mbar_init(smem_u32(&sh.accempty[i]), 4);
      }
      ptx::mbar_init(smem_u32(&sh.group), 4);
      ptx::fence_barrier_init();
      ptx::prefetch_tensormap(&tmap_k);
      ptx::prefetch_tensormap(&tmap_q);
    }
    __syncwarp();
    ptx::tmem_alloc(smem_u32(&sh.tmem_base), kTcTmemCols);
    ptx::tmem_relinquish();
  }
  if (kHist) {
    for (int i = tid; i < kHistBins; i += kTcThreads) sh.hist[i] = 0;
  }
  // ---- tiles per request -> exclusive prefix (all threads) ------------------------------------
  {
    const int chunk = (batch + kTcThreads - 1) / kTcThreads;
    const int lo = min(batch, tid * chunk), hi = min(batch, lo + chunk);
    int sum = 0;
    for (int b = lo; b < hi; ++b) sum += tiles_of(seq_lens[b], max_pages, skip_short);
    // exclusive scan of the per-thread sums: inside each warp by shuffles, then over the warps
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    if (lane == 31) sh.partial[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      const int nw = kTcThreads / 32;
      int wsum = lane < nw ? sh.partial[lane] : 0, wincl = wsum;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, wincl, o);
        if (lane >= o) wincl += up;
      }
      if (lane < nw) sh.partial[lane] = wincl - wsum;   // tiles before this warp
      if (lane == nw - 1) sh.prefix[batch] = wincl;
      if (lane == 0) sh.abort_flag = 0;
    }
    __syncthreads();
    int run = sh.partial[warp] + incl - sum;
    for (int b = lo; b < hi; ++b) {
      sh.prefix[b] = run;
      run += tiles_of(seq_lens[b], max_pages, skip_short);
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();

  const int total = sh.prefix[batch];
  const int per = (total + gridDim.x - 1) / gridDim.x;
  const int w0 = min(total, (int)blockIdx.x * per), w1 = min(total, w0 + per);
  const uint32_t tmem_base = sh.tmem_base;

  // Page ids of 32 consecutive tiles starting at w, one tile per lane (producer warp).  Both
  // entries of a tile are requested at once (the row has max_pages entries, so the second read is
  // in bounds); whether the second page belongs to the request is decided afterwards, so the
  // lookup costs one round trip, not two.
  auto lookup = [&](int w, int& bi, int& p0, int& p1, int& has2) {
    const int wi = min(w + lane, w1 - 1);
    bi = locate(sh.prefix, batch, wi);
    const int ji = wi - sh.prefix[bi];
    const int len = max(0, min(seq_lens[bi], max_pages * kPage));
    const int n_pages = (len + kPage - 1) / kPage;
    const int32_t* row = block_table + (size_t)bi * bt_stride + 2 * ji;
    p0 = row[0];
    p1 = (2 * ji + 1 < max_pages) ? row[1] : -1;
    has2 = 2 * ji + 1 < n_pages;          // the tile has a second page
  };
  int first_b = 0, first_p0 = 0, first_p1 = -1, first_has2 = 0;
  if (warp == 0 && w0 < w1) lookup(w0, first_b, first_p0, first_p1, first_has2);

  // Everything above read only seq_lens and block_table, before the dependency wait (like the
  // selection does): the kernels this library chains never write the caller's inputs, and a foreign
  // kernel before us starts us early only if it triggers its dependents itself -- it must then not
  // write those two afterwards.  q, weights and the cache are read after the wait.
  ptx::grid_dependency_wait();
  // Only now may the selection kernel be scheduled (as SMs free up; it waits for our scores): it
  // reads seq_lens and block_table before its own wait, which is safe once OUR predecessor is done.
  ptx::launch_dependents();

#define DSA_WAIT(bar, parity)                                  \
  if (!ptx::mbar_wait(smem_u32(&(bar)), (parity))) {           \
    sh.abort_flag = 1;                                         \
    raise_status(status, DSA_STATUS_WAIT_TIMEOUT);             \
  }

  if (w0 < w1) {
    if (warp == 0) {
      // ======================= producer =======================
      int stage = 0, phase = 0, qslot = 0, qphase = 0, cur_b = -1;
      int next_b = first_b, next_p0 = first_p0, next_p1 = first_p1, next_has2 = first_has2;
      for (int w = w0; w < w1 && !sh.abort_flag; w += 32) {
        const int bi = next_b;
        int p0 = next_p0, p1 = next_p1;
        const bool has_second = next_has2 != 0;
        // the ids of the 32 tiles after these travel while these are issued
        if (w + 32 < w1) lookup(w + 32, next_b, next_p0, next_p1, next_has2);
        if (p0 < 0 || p0 >= num_pages) { raise_status(status, DSA_STATUS_BAD_PAGE); p0 = 0; }
        if (!has_second) {
          p1 = -1;
        } else if (p1 < 0 || p1 >= num_pages) {
          raise_status(status, DSA_STATUS_BAD_PAGE);
          p1 = 0;
        }
        const int n = min(32, w1 - w);
        for (int i = 0; i < n; ++i) {
          const int tb = __shfl_sync(0xffffffffu, bi, i);
          const int a0 = __shfl_sync(0xffffffffu, p0, i);
          const int a1 = __shfl_sync(0xffffffffu, p1, i);
          if (lane == 0 && !sh.abort_flag) {
            if (tb != cur_b) {
              DSA_WAIT(sh.qempty[qslot], qphase ^ 1);
              ptx::mbar_expect_tx(smem_u32(&sh.qfull[qslot]), kPageDataBytes);
              ptx::tma_load_2d(q_addr + qslot * kPageDataBytes, &tmap_q, 0, tb * kIdxHeads,
                               smem_u32(&sh.qfull[qslot]));
              cur_b = tb;
              qslot ^= 1;
              if (qslot == 0) qphase ^= 1;
            }
            DSA_WAIT(sh.empty[stage], phase ^ 1);
            const uint32_t bar = smem_u32(&sh.full[stage]);
            const uint32_t dst = data_addr + stage * kTileDataBytes;
            const uint32_t sdst = smem_u32(&sh.scale[stage][0]);
            ptx::mbar_expect_tx(bar, (a1 >= 0 ? 2 : 1) * kPageBytes);
            ptx::tma_load_2d(dst, &tmap_k, 0, a0 * 66, bar);
            ptx::bulk_load_1d(sdst, k_cache + (size_t)a0 * kPageBytes + kPageDataBytes, 256, bar);
            if (a1 >= 0) {
              ptx::tma_load_2d(dst + kPageDataBytes, &tmap_k, 0, a1 * 66, bar);
              ptx::bulk_load_1d(sdst + 256, k_cache + (size_t)a1 * kPageBytes + kPageDataBytes, 256,
                                bar);
            }
            if (++stage == kTcStages) { stage = 0; phase ^= 1; }
          }
          __syncwarp();
        }
      }
    } else if (warp == 1) {
      // ======================= MMA issuer =======================
      if (lane == 0) {
        int stage = 0, phase = 0, qslot = 0, qphase = 0, acc = 0, aphase = 0;
        int b = locate(sh.prefix, batch, w0), next_change = w0;
        uint32_t qbase = q_addr;
        // descriptor bits that never change: LBO = 16 B, SBO = 1024 B, version 1, 128-byte swizzle
        const uint64_t desc_hi = ptx::smem_desc_sw128(0, 16, 1024);
        for (int w = w0; w < w1; ++w) {
          if (w >= next_change) {  // first tile of a request
            if (w > w0) ptx::tc_commit(smem_u32(&sh.qempty[qslot ^ 1]));  // previous q: free when read
            while (sh.prefix[b + 1] <= w) ++b;
            next_change = sh.prefix[b + 1];
            DSA_WAIT(sh.qfull[qslot], qphase);
            qbase = q_addr + qslot * kPageDataBytes;
            qslot ^= 1;
            if (qslot == 0) qphase ^= 1;
          }
          DSA_WAIT(sh.accempty[acc], aphase ^ 1);
          DSA_WAIT(sh.full[stage], phase);
          if (sh.abort_flag) break;
          ptx::tc_fence_after();
          const uint64_t adesc = desc_hi | (uint64_t)((data_addr + stage * kTileDataBytes) >> 4);
          const uint64_t bdesc = desc_hi | (uint64_t)(qbase >> 4);
          const uint32_t d = tmem_base + acc * kIdxHeads;
#pragma unroll
          for (int k = 0; k < 4; ++k)  // K = 32 fp8 = 32 bytes per instruction -> +2 in 16 B units
            ptx::mma_f8(d, adesc + 2 * k, bdesc + 2 * k, kIdescF8, k > 0);
          ptx::tc_commit(smem_u32(&sh.empty[stage]));
          ptx::tc_commit(smem_u32(&sh.accfull[acc]));
          if (++stage == kTcStages) { stage = 0; phase ^= 1; }
          if (++acc == kTcAcc) { acc = 0; aphase ^= 1; }
        }
      }
      __syncwarp();
    } else {
      // ======================= epilogue =======================
      const int quarter = warp & 3;
      const int rowi = quarter * 32 + lane;
      int stage = 0, phase = 0, acc = 0, aphase = 0;
      int b = locate(sh.prefix, batch, w0), next_change = w0, first_tile = 0, len = 0;
      float wreg[kIdxHeads];
      // running max of the ordered score keys of the current request, and of their complements
      // (= its min): handed to the selection so that it can bin the row without a sweep of its own
      uint32_t key_max = 0u, key_min_inv = 0u;
      auto flush_minmax = [&](int req) {
        if (minmax != nullptr && lane == 0 && key_max != 0u) {
          atomicMax(&minmax[2 * req], key_max);
          atomicMax(&minmax[2 * req + 1], key_min_inv);
        }
        key_max = 0u;
        key_min_inv = 0u;
      };
      // kHist: all four warps have counted the request's scores -> add the counts to its histogram
      // in global memory and clear them (bounded group barrier before and after)
      uint32_t gphase = 0;
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
      // (`last`: the CTA's final flush -- the counters need not be cleared, nobody counts again)
      auto flush_hist = [&](int req, bool last) -> bool {
        if (!group_sync()) return false;
        const int et = (warp - 2) * 32 + lane;
        uint32_t* g = ghist + (size_t)req * kHistBins;
        uint4* h4 = reinterpret_cast<uint4*>(sh.hist);
#pragma unroll
        for (int v = 0; v < kHistBins / 4 / 128; ++v) {
          const int q = v * 128 + et;
          const uint4 cnt = h4[q];
          if (cnt.x | cnt.y | cnt.z | cnt.w) {
            if (cnt.x) atomicAdd(g + 4 * q, cnt.x);
            if (cnt.y) atomicAdd(g + 4 * q + 1, cnt.y);
            if (cnt.z) atomicAdd(g + 4 * q + 2, cnt.z);
            if (cnt.w) atomicAdd(g + 4 * q + 3, cnt.w);
            if (!last) h4[q] = make_uint4(0u, 0u, 0u, 0u);
          }
        }
        return last || group_sync();
      };
      bool alive = true;
      for (int w = w0; w < w1; ++w) {
        if (w >= next_change) {
          if (w > w0) {
            if (kHist) { if (!flush_hist(b, false)) { alive = false; break; } }
            else flush_minmax(b);
          }
          while (sh.prefix[b + 1] <= w) ++b;
          next_change = sh.prefix[b + 1];
          first_tile = sh.prefix[b];
          const float4* wp = reinterpret_cast<const float4*>(weights + (size_t)b * kIdxHeads);
#pragma unroll
          for (int i = 0; i < kIdxHeads / 4; ++i) {
            float4 v = __ldg(wp + i);
            wreg[4 * i] = v.x; wreg[4 * i + 1] = v.y; wreg[4 * i + 2] = v.z; wreg[4 * i + 3] = v.w;
          }
          len = max(0, min(seq_lens[b], max_pages * kPage));
        }
        DSA_WAIT(sh.full[stage], phase);
        const float sc = sh.scale[stage][rowi];
        DSA_WAIT(sh.accfull[acc], aphase);
        if (sh.abort_flag) break;
        ptx::tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * kIdxHeads;
        // four 16-column chunks keep the live register set small enough for two CTAs per SM;
        // four independent partial sums keep the FMA chains short
        float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t r[16];
          ptx::tmem_ld16(taddr + c * 16, r);
          ptx::tmem_wait_ld();
#pragma unroll
          for (int h = 0; h < 16; ++h)
            part[h & 3] = fmaf(wreg[c * 16 + h], fmaxf(__uint_as_float(r[h]), 0.f), part[h & 3]);
        }
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          ptx::mbar_arrive(smem_u32(&sh.accempty[acc]));
          ptx::mbar_arrive(smem_u32(&sh.empty[stage]));
        }
        const int t = (w - first_tile) * kTcTile + rowi;
        const float val = ((part[0] + part[1]) + (part[2] + part[3])) * sc;
        if (t < len) scores[(size_t)b * score_stride + t] = val;
        if (kHist) {
          if (t < len) atomicAdd(&sh.hist[float_to_ordered(fmaxf(val, kScoreFloor)) >> 20], 1u);
        } else if (minmax != nullptr) {
          const uint32_t key = t < len ? float_to_ordered(fmaxf(val, kScoreFloor)) : 0u;
          key_max = max(key_max, __reduce_max_sync(0xffffffffu, key));
          key_min_inv = max(key_min_inv, __reduce_max_sync(0xffffffffu, t < len ? ~key : 0u));
        }
        if (++stage == kTcStages) { stage = 0; phase ^= 1; }
        if (++acc == kTcAcc) { acc = 0; aphase ^= 1; }
      }
      if (kHist) { if (alive) flush_hist(b, true); }
      else flush_minmax(b);
    }
  }
#undef DSA_WAIT

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    if (sh.abort_flag) {
      // let bulk copies that were already issued land before the CTA's shared memory is released
      for (int i = 0; i < 64; ++i) __nanosleep(20000);
    }
    ptx::tmem_dealloc(tmem_base, kTcTmemCols);
  }
}

// ------------------------------------------------------------------------------------------ host
static bool make_rows128_map(CUtensorMap* map, const void* base, uint64_t rows) {
  // rows x 128 bytes, box = 64 rows x 128 bytes, 128-byte swizzle
  return make_tmap_2d_sw128(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, base, 128, rows, 128, 64);
}

cudaError_t launch_indexer_score_tc(const void* q_fp8, const void* k_cache, const float* weights,
                                    const int32_t* seq_lens, const int32_t* block_table,
                                    int64_t bt_stride, float* scores, int64_t score_stride,
                                    int batch, int num_pages, int max_pages, int skip_short,
                                    uint32_t* minmax, uint32_t* ghist, int32_t* status,
                                    cudaStream_t stream) {
  static std::atomic<uint64_t> smem_opted_a{0}, smem_opted_b{0};
  {
    cudaError_t e = opt_in_dynamic_smem(reinterpret_cast<const void*>(indexer_score_tc_kernel<false>),
                                        kTcDynBytes, smem_opted_a);
    if (e == cudaSuccess)
      e = opt_in_dynamic_smem(reinterpret_cast<const void*>(indexer_score_tc_kernel<true>),
                              kTcDynBytes, smem_opted_b);
    if (e != cudaSuccess) return e;
  }
  if (ghist != nullptr && batch > kHistMaxBatch) return cudaErrorInvalidValue;
  CUtensorMap tmap_k;
  if (!make_rows128_map(&tmap_k, k_cache, (uint64_t)num_pages * 66)) return cudaErrorInvalidValue;
  for (int b0 = 0; b0 < batch; b0 += kTcMaxBatch) {
    const int nb = min(kTcMaxBatch, batch - b0);
    CUtensorMap tmap_q;
    const uint8_t* qp = static_cast<const uint8_t*>(q_fp8) + (size_t)b0 * kIdxHeads * kIdxDim;
    if (!make_rows128_map(&tmap_q, qp, (uint64_t)nb * kIdxHeads)) return cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * sm_count()));
    cfg.blockDim = dim3(kTcThreads);
    cfg.dynamicSmemBytes = kTcDynBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled();
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(
        &cfg, ghist != nullptr ? indexer_score_tc_kernel<true> : indexer_score_tc_kernel<false>, tmap_k,
        tmap_q, static_cast<const uint8_t*>(k_cache), weights + (size_t)b0 * kIdxHeads, seq_lens + b0,
        block_table + (size_t)b0 * bt_stride, bt_stride, scores + (size_t)b0 * score_stride,
        score_stride, nb, num_pages, max_pages, skip_short,
        minmax != nullptr ? minmax + 2 * (size_t)b0 : nullptr, ghist, status);
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

}  // namespace dsa
