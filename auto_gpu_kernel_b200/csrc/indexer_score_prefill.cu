// FP8 indexer scorer for chunked prefill: many query rows over ONE request's pages.
//
//   score[i,t] = scale[t] * sum_h w[i,h] * relu( q[i,h,:] . k[t,:] ),   t < seq_lens[i]
// (reference arithmetic: indexer_baseline.py:75-80, called with one block_table row shared by all
//  query rows -- row stride 0).
//
// With thousands of rows over a few MB of keys the work is bound by the FP8 tensor pipe, not by
// HBM, so the product is shaped to run tcgen05.mma at its full rate: tokens are M = 128, and the
// N dimension packs FOUR query rows x 64 heads = 256 columns (an N = 64 instruction costs the
// same ~46 cycles as N = 92; from N = 96 up the N/2 cycles are all useful, and fewer, larger
// instructions keep the single issuing thread off the critical path).  Eight consecutive rows
// form a group: the group's q (64 KB) stays in shared memory while the key tiles of the request
// stream through a 4-deep TMA ring (from L2: the keys are read once from HBM), and every key tile
// is multiplied with both halves of the group into the two 256-column TMEM accumulators.
//
//   warp 0       producer : q of the next group (2 TMA boxes of 256 x 128 B), key tiles + scales
//   warp 1       MMA      : per tile 2 x (4 x tcgen05.mma M=128 N=256 K=32)
//   warps 2-17   epilogue : warp group j (4 warps, one per TMEM lane quarter) reduces row j of
//                each accumulator: tcgen05.ld of the row's 64 head sums, relu, dot with the row's
//                w, times the token scale, coalesced fp32 store.  An accumulator is handed back to
//                the tensor pipe as soon as its values are in registers.  The epilogue costs two
//                instructions per accumulator column -- about as many issue cycles as the products
//                take on the tensor pipe -- and a tcgen05.ld has a latency of a few hundred
//                cycles, hence four warps per scheduler.
//
// Work is split evenly in (group, tile) items over one persistent CTA per SM by an in-kernel
// prefix sum over the device-resident seq_lens.  Every mbarrier wait is time-bounded.
#include "common.cuh"
#include "ptx.cuh"
#include "tmap.cuh"

namespace dsa {

namespace {

constexpr int kPfStages = 4;
constexpr int kPfTile = 128;
constexpr int kPfRows = 8;                       // query rows per group
constexpr int kPfSlots = 2;                      // TMEM accumulators per key tile
constexpr int kPfSlotRows = kPfRows / kPfSlots;  // 4 query rows per accumulator
constexpr int kPfSlotCols = kPfSlotRows * kIdxHeads;   // 256 fp32 columns
constexpr int kPfEpiGroups = 4;                  // epilogue warp groups (4 warps each)
constexpr int kPfThreads = 64 + kPfEpiGroups * 128;    // 576
constexpr int kPfMaxGroups = 2048;               // rows per launch <= 16384
constexpr int kPfTmemCols = kPfSlots * kPfSlotCols;           // 512
constexpr int kPfTileBytes = 2 * kPageDataBytes;             // 16384
constexpr int kPfQHalfBytes = kPfSlotRows * kIdxHeads * kIdxDim;  // 32768: one TMA box
constexpr int kPfQSlotBytes = kPfSlotRows * kIdxHeads * kIdxDim;  // q rows of one accumulator
constexpr int kPfQBytes = 2 * kPfQHalfBytes;                  // 65536
constexpr uint32_t kIdescPf = ptx::idesc(ptx::kFmtE4M3, ptx::kFmtE4M3, false, false, 128, kPfSlotCols);

struct PfShared {
  float scale[kPfStages][kPfTile];
  float w[kPfEpiGroups][kPfSlots][kIdxHeads];   // per epilogue group: the weights of its rows
  int prefix[kPfMaxGroups + 1];
  int partial[kPfThreads];
  uint64_t full[kPfStages], empty[kPfStages];
  uint64_t qfull[2], qempty[2];
  uint64_t accfull[kPfSlots], accempty[kPfSlots];
  uint32_t tmem_base;
  volatile int abort_flag;
};

constexpr size_t kPfDynBytes = 1024 + (size_t)kPfStages * kPfTileBytes + 2 * kPfQBytes +
                               sizeof(PfShared);

constexpr int kPfMaxCols = 3;   // of every 4 columns, how many use max() for the relu (measured best)

__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ float2 unpack2(uint64_t v) {
  float2 r;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(r.x), "=f"(r.y) : "l"(v));
  return r;
}
// d = a * b + c on two packed fp32 lanes (round to nearest even, like fmaf on each lane)
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
// relu of accumulator column `col` (mod 4): max(x, 0), or x + |x| = 2 relu(x) for the columns
// whose weight is stored halved.
template <int col>
__device__ __forceinline__ float relu_col(uint32_t bits) {
  const float x = __uint_as_float(bits);
  if (col < kPfMaxCols) return fmaxf(x, 0.f);
  return x + fabsf(x);
}

__device__ __forceinline__ int clamp_len(int len, int max_pages) {
  return max(0, min(len, max_pages * kPage));
}

// Tiles a group needs: enough for its longest row; none if every row is emitted whole by the
// selection (skip_short and length <= top-k).
__device__ __forceinline__ int group_tiles(const int32_t* seq_lens, int g, int rows, int max_pages,
                                           int skip_short) {
  int longest = 0;
  for (int r = g * kPfRows; r < min(rows, (g + 1) * kPfRows); ++r) {
    const int len = clamp_len(seq_lens[r], max_pages);
    if (skip_short && len <= kTopK) continue;
    longest = max(longest, len);
  }
  return (longest + kPfTile - 1) / kPfTile;
}

__device__ __forceinline__ int locate_group(const int* prefix, int groups, int w) {
  int lo = 0, hi = groups;
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (prefix[mid] <= w) lo = mid; else hi = mid;
  }
  return lo;
}

__global__ void __launch_bounds__(kPfThreads, 1)
indexer_score_prefill_kernel(const __grid_constant__ CUtensorMap tmap_k,
                             const __grid_constant__ CUtensorMap tmap_q,
                             const uint8_t* __restrict__ k_cache, const float* __restrict__ weights,
                             const int32_t* __restrict__ seq_lens,
                             const int32_t* __restrict__ block_row, float* __restrict__ scores,
                             int64_t score_stride, int rows, int num_pages, int max_pages,
                             int skip_short, int32_t* status) {
  extern __shared__ unsigned char dyn_raw[];
  const uint32_t raw_addr = smem_u32(dyn_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  unsigned char* base = dyn_raw + pad;
  const uint32_t data_addr = raw_addr + pad;                       // kPfStages x 16 KB
  const uint32_t q_addr = data_addr + kPfStages * kPfTileBytes;     // 2 x 64 KB
  PfShared& sh = *reinterpret_cast<PfShared*>(base + kPfStages * kPfTileBytes + 2 * kPfQBytes);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int groups = (rows + kPfRows - 1) / kPfRows;
  ptx::launch_dependents();

  // ---- tiles per group -> exclusive prefix ------------------------------------------------------
  {
    const int chunk = (groups + kPfThreads - 1) / kPfThreads;
    const int lo = min(groups, tid * chunk), hi = min(groups, lo + chunk);
    int sum = 0;
    for (int g = lo; g < hi; ++g) sum += group_tiles(seq_lens, g, rows, max_pages, skip_short);
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
      const int nw = kPfThreads / 32;
      int wsum = lane < nw ? sh.partial[lane] : 0, wincl = wsum;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, wincl, o);
        if (lane >= o) wincl += up;
      }
      if (lane < nw) sh.partial[lane] = wincl - wsum;   // tiles before this warp
      if (lane == nw - 1) sh.prefix[groups] = wincl;
      if (lane == 0) sh.abort_flag = 0;
    }
    __syncthreads();
    int run = sh.partial[warp] + incl - sum;
    for (int g = lo; g < hi; ++g) {
      sh.prefix[g] = run;
      run += group_tiles(seq_lens, g, rows, max_pages, skip_short);
    }
  }
  if (warp == 0) {
    if (lane == 0) {
      for (int i = 0; i < kPfStages; ++i) {
        ptx::mbar_init(smem_u32(&sh.full[i]), 1);
        ptx::mbar_init(smem_u32(&sh.empty[i]), 1 + 4 * kPfEpiGroups);   // MMA commit + epilogue warps
      }
      for (int i = 0; i < 2; ++i) {
        ptx::mbar_init(smem_u32(&sh.qfull[i]), 1);
        ptx::mbar_init(smem_u32(&sh.qempty[i]), 1);
      }
      for (int i = 0; i < kPfSlots; ++i) {
        ptx::mbar_init(smem_u32(&sh.accfull[i]), 1);
        ptx::mbar_init(smem_u32(&sh.accempty[i]), 4 * kPfEpiGroups);
      }
      ptx::fence_barrier_init();
      ptx::prefetch_tensormap(&tmap_k);
      ptx::prefetch_tensormap(&tmap_q);
    }
    __syncwarp();
    ptx::tmem_alloc(smem_u32(&sh.tmem_base), kPfTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();

  const int total = sh.prefix[groups];
  const int per = (total + gridDim.x - 1) / gridDim.x;
  const int w0 = min(total, (int)blockIdx.x * per), w1 = min(total, w0 + per);
  const uint32_t tmem_base = sh.tmem_base;

#define DSA_WAIT(bar, parity)                                  \
  if (!ptx::mbar_wait(smem_u32(&(bar)), (parity))) {           \
    sh.abort_flag = 1;                                         \
    raise_status(status, DSA_STATUS_WAIT_TIMEOUT);             \
  }

  if (w0 < w1) {
    if (warp == 0) {
      // ======================= producer =======================
      // The page ids of 32 items are looked up at once (one global-load latency per 32 tiles),
      // then lane 0 issues the copies item by item.
      int stage = 0, phase = 0, qslot = 0, qphase = 0, cur_g = -1;
      for (int w = w0; w < w1 && !sh.abort_flag; w += 32) {
        const int wi = min(w + lane, w1 - 1);
        const int gi = locate_group(sh.prefix, groups, wi);
        const int ji = wi - sh.prefix[gi];
        int longest = 0;
        for (int r = gi * kPfRows; r < min(rows, (gi + 1) * kPfRows); ++r)
          longest = max(longest, clamp_len(seq_lens[r], max_pages));
        const int n_pages = (longest + kPage - 1) / kPage;   // later entries of block_row are not ids
        int p0 = block_row[2 * ji];
        const bool has_second = 2 * ji + 1 < n_pages;
        int p1 = has_second ? block_row[2 * ji + 1] : -1;
        if (p0 < 0 || p0 >= num_pages) { raise_status(status, DSA_STATUS_BAD_PAGE); p0 = 0; }
        if (has_second && (p1 < 0 || p1 >= num_pages)) { raise_status(status, DSA_STATUS_BAD_PAGE); p1 = 0; }
        const int n = min(32, w1 - w);
        for (int i = 0; i < n; ++i) {
          const int tg = __shfl_sync(0xffffffffu, gi, i);
          const int a0 = __shfl_sync(0xffffffffu, p0, i);
          const int a1 = __shfl_sync(0xffffffffu, p1, i);
          if (lane == 0 && !sh.abort_flag) {
            if (tg != cur_g) {
              DSA_WAIT(sh.qempty[qslot], qphase ^ 1);
              const uint32_t bar = smem_u32(&sh.qfull[qslot]);
              ptx::mbar_expect_tx(bar, kPfQBytes);
              const uint32_t dst = q_addr + qslot * kPfQBytes;
              ptx::tma_load_2d(dst, &tmap_q, 0, tg * kPfRows * kIdxHeads, bar);
              ptx::tma_load_2d(dst + kPfQHalfBytes, &tmap_q, 0, (tg * kPfRows + kPfSlotRows) * kIdxHeads,
                               bar);
              cur_g = tg;
              qslot ^= 1;
              if (qslot == 0) qphase ^= 1;
            }
            DSA_WAIT(sh.empty[stage], phase ^ 1);
            const uint32_t bar = smem_u32(&sh.full[stage]);
            const uint32_t dst = data_addr + stage * kPfTileBytes;
            const uint32_t sdst = smem_u32(&sh.scale[stage][0]);
            ptx::mbar_expect_tx(bar, (a1 >= 0 ? 2 : 1) * kPageBytes);
            ptx::tma_load_2d(dst, &tmap_k, 0, a0 * 66, bar);
            ptx::bulk_load_1d(sdst, k_cache + (size_t)a0 * kPageBytes + kPageDataBytes, 256, bar);
            if (a1 >= 0) {
              ptx::tma_load_2d(dst + kPageDataBytes, &tmap_k, 0, a1 * 66, bar);
              ptx::bulk_load_1d(sdst + 256, k_cache + (size_t)a1 * kPageBytes + kPageDataBytes, 256,
                                bar);
            }
            if (++stage == kPfStages) { stage = 0; phase ^= 1; }
          }
          __syncwarp();
        }
      }
    } else if (warp == 1) {
      // ======================= MMA issuer =======================
      if (lane == 0) {
        int stage = 0, phase = 0, qslot = 0, qphase = 0, aphase = 0;
        int g = locate_group(sh.prefix, groups, w0), next_change = w0;
        uint32_t qbase = q_addr;
        const uint64_t desc_hi = ptx::smem_desc_sw128(0, 16, 1024);
        for (int w = w0; w < w1; ++w) {
          if (w >= next_change) {
            if (w > w0) ptx::tc_commit(smem_u32(&sh.qempty[qslot ^ 1]));  // previous q: free when read
            while (sh.prefix[g + 1] <= w) ++g;
            next_change = sh.prefix[g + 1];
            DSA_WAIT(sh.qfull[qslot], qphase);
            qbase = q_addr + qslot * kPfQBytes;
            qslot ^= 1;
            if (qslot == 0) qphase ^= 1;
          }
          DSA_WAIT(sh.full[stage], phase);
          if (sh.abort_flag) break;
          const uint64_t adesc = desc_hi | (uint64_t)((data_addr + stage * kPfTileBytes) >> 4);
#pragma unroll
          for (int slot = 0; slot < kPfSlots; ++slot) {
            DSA_WAIT(sh.accempty[slot], aphase ^ 1);
            ptx::tc_fence_after();
            const uint64_t bdesc = desc_hi | (uint64_t)((qbase + slot * kPfQSlotBytes) >> 4);
            const uint32_t d = tmem_base + slot * kPfSlotCols;
#pragma unroll
            for (int k = 0; k < 4; ++k)
              ptx::mma_f8(d, adesc + 2 * k, bdesc + 2 * k, kIdescPf, k > 0);
            ptx::tc_commit(smem_u32(&sh.accfull[slot]));
          }
          ptx::tc_commit(smem_u32(&sh.empty[stage]));
          aphase ^= 1;
          if (++stage == kPfStages) { stage = 0; phase ^= 1; }
        }
      }
      __syncwarp();
    } else {
      // ======================= epilogue =======================
      // warp group j (four warps, one per TMEM lane quarter) owns row j of each accumulator:
      // rows j and 4 + j of the group.  Four warps per scheduler hide the tcgen05.ld latency.
      const int grp = (warp - 2) >> 2;
      const int quarter = warp & 3;              // TMEM lane quarter this warp may read
      const int rowi = quarter * 32 + lane;      // token within the tile
      const int etid = ((warp - 2) & 3) * 32 + lane;   // 0..127 within the warp group
      int stage = 0, phase = 0, aphase = 0;
      int g = locate_group(sh.prefix, groups, w0), next_change = w0, first_tile = 0;
      int len[kPfSlots] = {0, 0};
      for (int w = w0; w < w1; ++w) {
        if (w >= next_change) {
          while (sh.prefix[g + 1] <= w) ++g;
          next_change = sh.prefix[g + 1];
          first_tile = sh.prefix[g];
          ptx::named_bar_sync(1 + grp, 128);    // everyone is done with the previous weights
          {
            const int k = etid / kIdxHeads, h = etid % kIdxHeads;   // 128 threads: 2 rows x 64 heads
            const int r = g * kPfRows + k * kPfSlotRows + grp;
            const float wv = r < rows ? weights[(size_t)r * kIdxHeads + h] : 0.f;
            sh.w[grp][k][h] = (h & 3) >= kPfMaxCols ? 0.5f * wv : wv;
          }
#pragma unroll
          for (int k = 0; k < kPfSlots; ++k) {
            const int r = g * kPfRows + k * kPfSlotRows + grp;
            len[k] = r < rows ? clamp_len(seq_lens[r], max_pages) : 0;
          }
          ptx::named_bar_sync(1 + grp, 128);
        }
        DSA_WAIT(sh.full[stage], phase);
        const float sc = sh.scale[stage][rowi];
        const int t = (w - first_tile) * kPfTile + rowi;
#pragma unroll
        for (int k = 0; k < kPfSlots; ++k) {
          DSA_WAIT(sh.accfull[k], aphase);
          if (sh.abort_flag) break;
          ptx::tc_fence_after();
          const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + k * kPfSlotCols +
                                 grp * kIdxHeads;
          uint32_t v0[32], v1[32];
          ptx::tmem_ld32(taddr, v0);             // both halves of the row in flight together
          ptx::tmem_ld32(taddr + 32, v1);
          ptx::tmem_wait_ld();
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(smem_u32(&sh.accempty[k]));   // values are in registers
          // relu + weighted sum, two columns per packed FMA.  max() runs on the half-rate ALU
          // pipe, so the columns h % 4 >= kPfMaxCols take relu(x) = (x + |x|) / 2 on the FMA pipe
          // instead (their weights are stored halved): both pipes stay below the tensor pipe's time.
          uint64_t acc01 = 0ull, acc23 = 0ull;
          const ulonglong2* wp = reinterpret_cast<const ulonglong2*>(&sh.w[grp][k][0]);
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            const ulonglong2 wv = wp[c];
            const uint32_t* v = c < 8 ? &v0[4 * c] : &v1[4 * (c - 8)];
            acc01 = fma2(wv.x, pack2(relu_col<0>(v[0]), relu_col<1>(v[1])), acc01);
            acc23 = fma2(wv.y, pack2(relu_col<2>(v[2]), relu_col<3>(v[3])), acc23);
          }
          const float2 s01 = unpack2(acc01), s23 = unpack2(acc23);
          const float total = (s01.x + s01.y) + (s23.x + s23.y);
          const int r = g * kPfRows + k * kPfSlotRows + grp;
          if (t < len[k])
            scores[(size_t)r * score_stride + t] = total * sc;
        }
        if (sh.abort_flag) break;
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(smem_u32(&sh.empty[stage]));
        aphase ^= 1;
        if (++stage == kPfStages) { stage = 0; phase ^= 1; }
      }
    }
  }
#undef DSA_WAIT

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    if (sh.abort_flag) {
      for (int i = 0; i < 64; ++i) __nanosleep(20000);   // let issued bulk copies land
    }
    ptx::tmem_dealloc(tmem_base, kPfTmemCols);
  }
}

}  // namespace

// Rows of one launch share `block_row` (the request's page list).  Returns cudaErrorInvalidValue
// when the tensor maps cannot be encoded.
cudaError_t launch_indexer_score_prefill(const void* q_fp8, const void* k_cache,
                                         const float* weights, const int32_t* seq_lens,
                                         const int32_t* block_row, float* scores,
                                         int64_t score_stride, int rows, int num_pages,
                                         int max_pages, int skip_short, int32_t* status,
                                         cudaStream_t stream) {
  static std::atomic<uint64_t> smem_opted{0};
  {
    cudaError_t e = opt_in_dynamic_smem(reinterpret_cast<const void*>(indexer_score_prefill_kernel),
                                        kPfDynBytes, smem_opted);
    if (e != cudaSuccess) return e;
  }
  CUtensorMap tmap_k;
  if (!make_tmap_2d_sw128(&tmap_k, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, k_cache, 128,
                          (uint64_t)num_pages * 66, 128, 64))
    return cudaErrorInvalidValue;
  const int per_launch = kPfMaxGroups * kPfRows;
  for (int r0 = 0; r0 < rows; r0 += per_launch) {
    const int nr = min(per_launch, rows - r0);
    CUtensorMap tmap_q;
    const uint8_t* qp = static_cast<const uint8_t*>(q_fp8) + (size_t)r0 * kIdxHeads * kIdxDim;
    if (!make_tmap_2d_sw128(&tmap_q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, qp, 128,
                            (uint64_t)nr * kIdxHeads, 128, 256))
      return cudaErrorInvalidValue;
    indexer_score_prefill_kernel<<<sm_count(), kPfThreads, kPfDynBytes, stream>>>(
        tmap_k, tmap_q, static_cast<const uint8_t*>(k_cache), weights + (size_t)r0 * kIdxHeads,
        seq_lens + r0, block_row, scores + (size_t)r0 * score_stride, score_stride, nr, num_pages,
        max_pages, skip_short, status);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

}  // namespace dsa
