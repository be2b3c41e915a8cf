// Sparse MLA attention over the selected rows on the 5th-generation tensor cores.
//
//   logit[h,k] = (q_nope[h].ckv[idx[k]] + q_pe[h].kpe[idx[k]]) * sm_scale      idx == -1 -> masked
//   lse[h]     = log2( sum_k e^{logit[h,k]} )          out[h] = softmax_k(logit[h,:]) @ ckv[idx[:]]
// (reference arithmetic: sparse_baseline.py:18-45; kernels this replaces: sparse_fused.py:23-285 and
//  the Gluon _dsa_decode_gluon of archive/fable/dsa_sparse_attention_*.py:77-433).
//
// Decode is bound by the HBM gather of 2048 random rows (1024 B ckv + 128 B kpe) per token, so the
// design goal is bytes in flight; the 16 heads share every gathered row.
//
// Heads (16) are far below the tcgen05 M minimum, so the products are issued transposed: the
// gathered rows are the M dimension and the heads are N = 16.
//   S^T[64 rows,16]   = K[64,576] . Q^T            A = gathered tile, K-major; B = q, K-major
//   O^T[512,16]      += V^T[512,64] . P^T          A = the SAME shared-memory tile read MN-major
//                                                  (V is the 512-wide ckv part of the row);
//                                                  B = P^T[16,64] bf16 written by the softmax warps
// Shared-memory tile layout (one stage = 64 rows): nine [64 rows x 128 B] blocks (eight ckv column
// blocks, one kpe block), each in the canonical 128-byte-swizzle layout, so one gather feeds both
// products.
//
// Work split: the (token, 64-row tile) sequence is cut into equal contiguous ranges, one per CTA
// (one CTA per SM), so SMs are balanced even when tokens x splits does not divide the SM count.  A
// CTA's range covers parts ("segments") of at most a few tokens; a token covered by several CTAs is
// merged by whichever of them finishes last (atomic arrival counter, nobody waits).
//
// Warp roles (320 threads): warps 0-3 softmax + epilogue (TMEM lane quarter = warp), warp 4 MMA
// issuer, warps 5-8 gather producers, warp 9 L2 prefetcher (it walks the index rows three tiles
// ahead of the gather and issues one bulk L2 prefetch per selected row, so HBM latency is taken
// by requests that need no shared-memory stage and the gather itself is served from L2).  A producer warp instruction copies one 128-byte column
// block of four rows (8 lanes x 16 B per row, cp.async with zero-fill for masked rows) straight to
// its swizzled place; a thread keeps its four row indices in registers, so the 36 copies of a
// tile are address arithmetic with immediates only.  (The TMA tile::gather4 mode was measured
// here at ~70 cycles per 512-byte instruction, a quarter of what this path sustains.)  Two stages.
// A tcgen05.mma costs max(45.6, N/2) cycles whatever M is, so at N = 16 the tensor pipe time is
// instruction count x 46 cycles: descriptors are stepped with one 32-bit add per instruction to
// keep the issuing thread under that, and S^T uses four partial accumulators round-robin.
// The running max is only refreshed (and O rescaled in TMEM) when a logit exceeds it by more than
// 2^8, so the common tile costs one exp2 per logit and no cross-thread reduction; row sums stay
// per-thread until the end of the segment.  All waits are time-bounded; group decisions are taken
// by one thread and broadcast, so a timeout makes every role leave together.
#include "common.cuh"
#include "ptx.cuh"
#include "tmap.cuh"
#include "attn_plan.cuh"

namespace dsa {

constexpr int kAtBlockBytes = kAtTile * 128;       // 8192
constexpr int kAtStageBytes = 9 * kAtBlockBytes;   // 73728
constexpr int kAtQBlockBytes = kHeads * 128;       // 2048
constexpr int kAtQBytes = 9 * kAtQBlockBytes;      // 18432
constexpr int kAtPBytes = kHeads * 128;            // 2048
constexpr int kAtThreads = 320;
constexpr int kAtPrefetchAhead = 3;                // tiles the L2 prefetcher runs ahead of the gather
constexpr int kAtTmemCols = 256;
constexpr int kAtSCol = 64;                        // O^T at 0..63; S^T buffer b at 64+64b (4 partials x 16)
constexpr float kAtLog2e = 1.4426950408889634f;
constexpr float kAtRescaleGap = 8.f;
constexpr uint32_t kIdescQK = ptx::idesc(ptx::kFmtBF16, ptx::kFmtBF16, false, false, 64, 16);
constexpr uint32_t kIdescPV = ptx::idesc(ptx::kFmtBF16, ptx::kFmtBF16, true, false, 128, 16);

struct AtShared {
  int idx[2][kAtTile];
  int live_w[2][4];      // per producer warp: the tile has at least one valid row
  int need[4];
  float red[4][kHeads];
  float merge_f[32][kHeads];  // per-segment rescale factors of the token being merged
  float merge_inv[kHeads];
  int go[2];
  uint64_t kv_full[2], kv_empty[2], q_full[2], q_empty[2];
  uint64_t s_full[2], s_empty[2], p_full[2], p_empty[2], o_free;
  uint32_t tmem_base;
  volatile int abort_flag;
  volatile int tiles_gathered;  // progress of producer warp 0, paces the L2 prefetcher
  int is_last;
};

constexpr size_t kAtDynBytes = 1024 + 2 * kAtStageBytes + 2 * kAtQBytes + 2 * kAtPBytes + sizeof(AtShared);

// The softmax group (128 threads) waits on mbarriers through its first thread, which broadcasts
// the outcome through shared memory: a timeout then makes all of them leave the loop together.
// `bar2` (0 = none) is waited first; it only adds an acquire on a barrier that is already complete.
__device__ __forceinline__ bool group_wait(AtShared& sh, int& toggle, bool leader, uint32_t bar2,
                                           uint32_t bar, uint32_t parity, int32_t* status) {
  if (leader) {
    bool ok = !sh.abort_flag;
    if (ok && bar2) ok = ptx::mbar_wait(bar2, parity);
    if (ok) ok = ptx::mbar_wait(bar, parity);
    if (!ok && !sh.abort_flag) {
      sh.abort_flag = 1;
      raise_status(status, DSA_STATUS_WAIT_TIMEOUT);
    }
    sh.go[toggle] = ok ? 1 : 0;
  }
  ptx::named_bar_sync(1, 128);
  const bool go = sh.go[toggle] != 0;
  toggle ^= 1;
  return go;
}

// Merge the per-segment partial results of one token (run by the 128 softmax threads of the CTA
// that arrived last).  Threads 0..15 turn the segments' (m, l) into rescale factors; then every
// thread owns four consecutive output columns and walks the 16 heads, so each warp reads 512
// contiguous bytes per (segment, head) and the loads of different heads are independent.
__device__ void at_merge_segments(AtShared& sh, const AtPartials& w, int t, int n_seg, int segs_max,
                                  __nv_bfloat16* out, float* lse, int tid) {
  if (tid < kHeads) {
    const int h = tid;
    float mx = -INFINITY;
    for (int s = 0; s < n_seg; ++s) mx = fmaxf(mx, w.m[((size_t)t * segs_max + s) * kHeads + h]);
    float lsum = 0.f;
    for (int s = 0; s < n_seg; ++s) {
      const size_t o = ((size_t)t * segs_max + s) * kHeads + h;
      const float ms = w.m[o];
      const float fs = (ms == -INFINITY) ? 0.f : exp2f(ms - mx);
      sh.merge_f[s][h] = fs;
      lsum += w.l[o] * fs;
    }
    sh.merge_inv[h] = lsum > 0.f ? 1.f / lsum : 0.f;
    lse[(size_t)t * kHeads + h] = lsum > 0.f ? mx + log2f(lsum) : -INFINITY;
  }
  ptx::named_bar_sync(1, 128);
  const int c0 = tid * 4;
  float4 a[kHeads];
#pragma unroll
  for (int h = 0; h < kHeads; ++h) a[h] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s = 0; s < n_seg; ++s) {
    const float* base = w.acc + ((size_t)t * segs_max + s) * kHeads * kCkv + c0;
    float4 v[kHeads];
#pragma unroll
    for (int h = 0; h < kHeads; ++h) v[h] = *reinterpret_cast<const float4*>(base + h * kCkv);  // 16 loads in flight
#pragma unroll
    for (int h = 0; h < kHeads; ++h) {
      const float fs = sh.merge_f[s][h];
      a[h].x += v[h].x * fs; a[h].y += v[h].y * fs; a[h].z += v[h].z * fs; a[h].w += v[h].w * fs;
    }
  }
#pragma unroll
  for (int h = 0; h < kHeads; ++h) {
    const float inv = sh.merge_inv[h];
    __nv_bfloat162 lo = __floats2bfloat162_rn(a[h].x * inv, a[h].y * inv);
    __nv_bfloat162 hi = __floats2bfloat162_rn(a[h].z * inv, a[h].w * inv);
    uint2 packed = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    *reinterpret_cast<uint2*>(out + ((size_t)t * kHeads + h) * kCkv + c0) = packed;
  }
  ptx::named_bar_sync(1, 128);  // merge_f / merge_inv may be rewritten by a later merge
}

__global__ void __launch_bounds__(kAtThreads, 1)
sparse_attn_tc_kernel(const __nv_bfloat16* __restrict__ q_nope, const __nv_bfloat16* __restrict__ q_pe,
                      const __nv_bfloat16* __restrict__ ckv, const __nv_bfloat16* __restrict__ kpe,
                      const int32_t* __restrict__ indices, int64_t index_stride, float scale_log2,
                      __nv_bfloat16* __restrict__ out, float* __restrict__ lse, int tokens, int topk,
                      int64_t num_slots, AtPlan plan, void* ws_raw, int32_t* status) {
  extern __shared__ unsigned char dyn_raw[];
  const uint32_t raw_addr = smem_u32(dyn_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  const uint32_t kv_addr = raw_addr + pad;                 // 2 stages
  const uint32_t q_addr = kv_addr + 2 * kAtStageBytes;     // 2 q buffers
  const uint32_t p_addr = q_addr + 2 * kAtQBytes;          // 2 P^T buffers
  unsigned char* p_ptr = dyn_raw + pad + 2 * kAtStageBytes + 2 * kAtQBytes;
  AtShared& sh = *reinterpret_cast<AtShared*>(p_ptr + 2 * kAtPBytes);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tpt = plan.tiles_per_token;
  const long total = (long)tokens * tpt;
  const long w0 = (long)blockIdx.x * plan.per_cta;
  const long w1 = w0 + plan.per_cta < total ? w0 + plan.per_cta : total;

  if (warp == 4) {
    if (lane == 0) {
      for (int i = 0; i < 2; ++i) {
        ptx::mbar_init(smem_u32(&sh.kv_full[i]), 128 + 4);  // cp.async arrivals + 4 warp leaders
        ptx::mbar_init(smem_u32(&sh.kv_empty[i]), 4 + 1);   // softmax warps + MMA
        ptx::mbar_init(smem_u32(&sh.q_full[i]), 128);
        ptx::mbar_init(smem_u32(&sh.q_empty[i]), 1);
        ptx::mbar_init(smem_u32(&sh.s_full[i]), 1);
        ptx::mbar_init(smem_u32(&sh.s_empty[i]), 4);
        ptx::mbar_init(smem_u32(&sh.p_full[i]), 4);
        ptx::mbar_init(smem_u32(&sh.p_empty[i]), 1);
      }
      ptx::mbar_init(smem_u32(&sh.o_free), 4);
      sh.abort_flag = 0;
      sh.tiles_gathered = 0;
      ptx::fence_barrier_init();
    }
    __syncwarp();
    ptx::tmem_alloc(smem_u32(&sh.tmem_base), kAtTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = sh.tmem_base;

  if (w0 < w1) {
    if (warp < 4) {
      // =========================== softmax + epilogue ===========================
      // Tile i of this CTA uses KV stage i&1 and S^T buffer i&1 (phase (i>>1)&1 of their barriers);
      // P^T buffers are numbered by live tiles only.
      const bool leader = tid == 0;
      const bool has_row = lane < 16;
      const int row = warp * 16 + (lane & 15);
      const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
      int toggle = 0, i_tile = 0, pl = 0, seg_live = 0;
      long cur_t = -1;
      float m_run[kHeads], l_part[kHeads];
      AtPartials part = at_carve(ws_raw, tokens, plan.segs_max);
      long t = w0 / tpt;
      int j = (int)(w0 - t * tpt) - 1;
      for (long w = w0; w < w1; ++w, ++i_tile) {
        if (++j == tpt) { j = 0; ++t; }
        if (t != cur_t) {
#pragma unroll
          for (int h = 0; h < kHeads; ++h) { m_run[h] = -INFINITY; l_part[h] = 0.f; }
          seg_live = 0;
          cur_t = t;
        }
        const int sbuf = i_tile & 1, sphase = (i_tile >> 1) & 1;
        if (!group_wait(sh, toggle, leader, smem_u32(&sh.kv_full[sbuf]), smem_u32(&sh.s_full[sbuf]),
                        sphase, status)) break;
        const bool live = (sh.live_w[sbuf][0] | sh.live_w[sbuf][1] | sh.live_w[sbuf][2] | sh.live_w[sbuf][3]) != 0;
        const bool valid = has_row && sh.idx[sbuf][row] >= 0;
        float x[kHeads];
        if (live) {
          ptx::tc_fence_after();
          uint32_t sr[16], sp1[16], sp2[16], sp3[16];
          const uint32_t s_addr = tmem_base + lane_base + kAtSCol + sbuf * 64;
          ptx::tmem_ld16(s_addr, sr);
          ptx::tmem_ld16(s_addr + 16, sp1);
          ptx::tmem_ld16(s_addr + 32, sp2);
          ptx::tmem_ld16(s_addr + 48, sp3);
          ptx::tmem_wait_ld();
          ptx::tc_fence_before();
#pragma unroll
          for (int h = 0; h < kHeads; ++h) {
            const float s4 = (__uint_as_float(sr[h]) + __uint_as_float(sp1[h])) +
                             (__uint_as_float(sp2[h]) + __uint_as_float(sp3[h]));
            x[h] = valid ? s4 * scale_log2 : -INFINITY;
          }
        }
        __syncwarp();
        if (lane == 0) {  // S^T buffer and the stage's index row have been read by this warp
          ptx::mbar_arrive(smem_u32(&sh.s_empty[sbuf]));
          ptx::mbar_arrive(smem_u32(&sh.kv_empty[sbuf]));
        }
        if (live) {
          bool need = false;
#pragma unroll
          for (int h = 0; h < kHeads; ++h) need |= x[h] > m_run[h] + kAtRescaleGap;
          const bool warp_need = __any_sync(0xffffffffu, need);
          if (lane == 0) sh.need[warp] = warp_need;
          ptx::named_bar_sync(1, 128);
          if (sh.need[0] | sh.need[1] | sh.need[2] | sh.need[3]) {
            // refresh the running max of every head, rescale what was accumulated so far
#pragma unroll
            for (int h = 0; h < kHeads; ++h) {
              float v = x[h];
#pragma unroll
              for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
              if (lane == 0) sh.red[warp][h] = v;
            }
            ptx::named_bar_sync(1, 128);
            float corr[kHeads];
#pragma unroll
            for (int h = 0; h < kHeads; ++h) {
              float mx = fmaxf(fmaxf(sh.red[0][h], sh.red[1][h]), fmaxf(sh.red[2][h], sh.red[3][h]));
              float m_new = fmaxf(m_run[h], mx);
              corr[h] = m_new == -INFINITY ? 1.f : exp2f(m_run[h] - m_new);
              m_run[h] = m_new;
              l_part[h] *= corr[h];
            }
            if (seg_live > 0) {
              // PV of the previous live tile is complete when its P^T buffer has been released;
              // every earlier phase of that barrier is known complete (see the P^T write below).
              if (!group_wait(sh, toggle, leader, 0, smem_u32(&sh.p_empty[(pl - 1) & 1]),
                              ((pl - 1) >> 1) & 1, status)) break;
              ptx::tc_fence_after();
#pragma unroll
              for (int c = 0; c < 4; ++c) {
                uint32_t o[16];
                ptx::tmem_ld16(tmem_base + lane_base + c * 16, o);
                ptx::tmem_wait_ld();
#pragma unroll
                for (int h = 0; h < kHeads; ++h) o[h] = __float_as_uint(__uint_as_float(o[h]) * corr[h]);
                ptx::tmem_st16(tmem_base + lane_base + c * 16, o);
              }
              ptx::tmem_wait_st();
              ptx::tc_fence_before();
            }
          }
          // P^T buffer pl&1 was last read by the PV of live tile pl-2.  The MMA thread issued that PV
          // before this tile's QK, and tcgen05.commit covers everything issued before it, so the
          // s_full arrival observed above implies that PV is complete: the buffer is free.
          if (has_row) {
            unsigned char* pb = p_ptr + (pl & 1) * kAtPBytes;
#pragma unroll
            for (int h = 0; h < kHeads; ++h) {
              const float m_use = m_run[h] == -INFINITY ? 0.f : m_run[h];
              const float p = exp2f(x[h] - m_use);
              l_part[h] += p;
              *reinterpret_cast<__nv_bfloat16*>(pb + h * 128 + ((((row >> 3) ^ (h & 7)) & 7) << 4) +
                                                (row & 7) * 2) = __float2bfloat16_rn(p);
            }
          }
          ptx::fence_proxy_async_smem();
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(smem_u32(&sh.p_full[pl & 1]));
          ++pl;
          ++seg_live;
        }
        if (j == tpt - 1 || w == w1 - 1) {
          // ------------------ end of this CTA's segment of token t ------------------
          if (seg_live > 0) {
            if (!group_wait(sh, toggle, leader, 0, smem_u32(&sh.p_empty[(pl - 1) & 1]),
                            ((pl - 1) >> 1) & 1, status)) break;
            ptx::tc_fence_after();
          }
#pragma unroll
          for (int h = 0; h < kHeads; ++h) {
            float v = has_row ? l_part[h] : 0.f;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) sh.red[warp][h] = v;
          }
          ptx::named_bar_sync(1, 128);
          float l_tot[kHeads];
#pragma unroll
          for (int h = 0; h < kHeads; ++h)
            l_tot[h] = (sh.red[0][h] + sh.red[1][h]) + (sh.red[2][h] + sh.red[3][h]);
          const long first_tile = t * tpt, last_tile = first_tile + tpt - 1;
          const int cta_first = (int)(first_tile / plan.per_cta), cta_last = (int)(last_tile / plan.per_cta);
          const int n_seg = cta_last - cta_first + 1, seg = (int)blockIdx.x - cta_first;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t o[16];
            if (seg_live > 0) {
              ptx::tmem_ld16(tmem_base + lane_base + c * 16, o);
              ptx::tmem_wait_ld();
            } else {
#pragma unroll
              for (int h = 0; h < kHeads; ++h) o[h] = 0u;
            }
            const int dim = c * 128 + warp * 32 + lane;
            if (n_seg == 1) {
#pragma unroll
              for (int h = 0; h < kHeads; ++h) {
                const float inv = l_tot[h] > 0.f ? 1.f / l_tot[h] : 0.f;
                out[((size_t)t * kHeads + h) * kCkv + dim] = __float2bfloat16_rn(__uint_as_float(o[h]) * inv);
              }
            } else {
#pragma unroll
              for (int h = 0; h < kHeads; ++h)
                part.acc[(((size_t)t * plan.segs_max + seg) * kHeads + h) * kCkv + dim] = __uint_as_float(o[h]);
            }
          }
          if (tid < kHeads) {
            // m_run / l_tot are identical in every thread; pick head `tid` without dynamic indexing
            float mh = 0.f, lh = 0.f;
#pragma unroll
            for (int h = 0; h < kHeads; ++h) if (h == tid) { mh = m_run[h]; lh = l_tot[h]; }
            if (n_seg == 1) {
              lse[(size_t)t * kHeads + tid] = lh > 0.f ? mh + log2f(lh) : -INFINITY;
            } else {
              part.m[((size_t)t * plan.segs_max + seg) * kHeads + tid] = lh > 0.f ? mh : -INFINITY;
              part.l[((size_t)t * plan.segs_max + seg) * kHeads + tid] = lh;
            }
          }
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(smem_u32(&sh.o_free));
          if (n_seg > 1) {
            __threadfence();
            ptx::named_bar_sync(1, 128);
            if (leader) {
              const int old = atomicAdd(&part.counters[t], 1);
              sh.is_last = old == n_seg - 1;
              if (sh.is_last) part.counters[t] = 0;
            }
            ptx::named_bar_sync(1, 128);
            if (sh.is_last) {
              __threadfence();
              at_merge_segments(sh, part, (int)t, n_seg, plan.segs_max, out, lse, tid);
            }
          }
        }
      }
    } else if (warp == 4) {
      // =========================== MMA issuer ===========================
      // Event loop of one thread: a PV product is issued as soon as the softmax warps have
      // published its P^T (that frees the tile's stage for the next gather at the earliest
      // moment); otherwise the QK product of the next tile is issued once its gather has landed.
      // Up to two PV products can be pending (tile i+1 scored before tile i is weighted).
      if (lane == 0) {
        const int n_tiles = (int)(w1 - w0);
        int qk_i = 0, np = 0, seg_no = 0, qb = 0, qphase = 0;
        long cur_t = -1, t = w0 / tpt;
        int j = (int)(w0 - t * tpt);  // (t, j) of tile qk_i
        bool seg_first = true, ok = true;
        uint32_t q_lo = 0;
        int pend_n = 0, pend_stage[2] = {0, 0};
        bool pend_first[2] = {false, false};
        // constant descriptor halves: K-major (LBO 16, SBO 1024) and MN-major (LBO 8192, SBO 1024)
        const uint64_t dk = ptx::smem_desc_sw128(0, 16, 1024), dmn = ptx::smem_desc_sw128(0, kAtBlockBytes, 1024);
        const uint32_t k_hi = (uint32_t)(dk >> 32), k_lo0 = (uint32_t)dk;
        const uint32_t mn_hi = (uint32_t)(dmn >> 32), mn_lo0 = (uint32_t)dmn;
        auto fail = [&]() {
          if (!sh.abort_flag) { sh.abort_flag = 1; raise_status(status, DSA_STATUS_WAIT_TIMEOUT); }
          ok = false;
        };
        auto wait = [&](uint64_t& bar, uint32_t parity) {
          if (ok && !(!sh.abort_flag && ptx::mbar_wait(smem_u32(&bar), parity))) fail();
        };
        auto issue_pv = [&]() {  // head of the pending queue; its P^T is known to be published
          const int pbuf = np & 1, st = pend_stage[0];
          ptx::tc_fence_after();
          const uint32_t a_lo = mn_lo0 + ((kv_addr + st * kAtStageBytes) >> 4);
          const uint32_t b_lo = k_lo0 + ((p_addr + pbuf * kAtPBytes) >> 4);
          const bool first = pend_first[0];
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              ptx::mma_bf16_split(tmem_base + c * 16, a_lo + ((2 * c * kAtBlockBytes + ks * 2048) >> 4),
                                  mn_hi, b_lo + ((ks * 32) >> 4), k_hi, kIdescPV,
                                  (first && ks == 0) ? 0u : 1u);
            }
          }
          ptx::tc_commit(smem_u32(&sh.kv_empty[st]));
          ptx::tc_commit(smem_u32(&sh.p_empty[pbuf]));
          ++np;
          pend_stage[0] = pend_stage[1];
          pend_first[0] = pend_first[1];
          --pend_n;
        };
        uint64_t idle_since = 0;
        while (ok && (qk_i < n_tiles || pend_n > 0)) {
          bool progressed = false;
          if (pend_n > 0 && ptx::mbar_try_wait(smem_u32(&sh.p_full[np & 1]), (np >> 1) & 1)) {
            issue_pv();
            progressed = true;
          } else if (qk_i < n_tiles) {
            const int stage = qk_i & 1, phase = (qk_i >> 1) & 1;
            if (t != cur_t) {
              // segment switch: everything of the previous segment must be issued and read first
              if (cur_t >= 0) {
                while (ok && pend_n > 0) {
                  wait(sh.p_full[np & 1], (np >> 1) & 1);
                  if (ok) issue_pv();
                }
                ptx::tc_commit(smem_u32(&sh.q_empty[qb ^ 1]));
                wait(sh.o_free, seg_no & 1);  // epilogue of the previous segment has read O^T
                ++seg_no;
              }
              wait(sh.q_full[qb], qphase);
              if (!ok) break;
              q_lo = k_lo0 + ((q_addr + qb * kAtQBytes) >> 4);
              qb ^= 1;
              if (qb == 0) qphase ^= 1;
              cur_t = t;
              seg_first = true;
              progressed = true;
            } else if (pend_n < 2 && ptx::mbar_try_wait(smem_u32(&sh.kv_full[stage]), phase) &&
                       ptx::mbar_try_wait(smem_u32(&sh.s_empty[stage]), phase ^ 1)) {
              ptx::fence_proxy_async_smem();  // cp.async-written tile / q -> visible to the MMA's reads
              const bool live = (sh.live_w[stage][0] | sh.live_w[stage][1] | sh.live_w[stage][2] |
                                 sh.live_w[stage][3]) != 0;
              if (live) {
                ptx::tc_fence_after();
                const uint32_t a_lo = k_lo0 + ((kv_addr + stage * kAtStageBytes) >> 4);
                const uint32_t d0 = tmem_base + kAtSCol + stage * 64;
#pragma unroll
                for (int kb = 0; kb < 9; ++kb) {
#pragma unroll
                  for (int k = 0; k < 4; ++k) {
                    ptx::mma_bf16_split(d0 + 16 * k, a_lo + ((kb * kAtBlockBytes + k * 32) >> 4), k_hi,
                                        q_lo + ((kb * kAtQBlockBytes + k * 32) >> 4), k_hi, kIdescQK,
                                        kb != 0 ? 1u : 0u);
                  }
                  // a PV whose P^T shows up meanwhile goes first: it frees a stage for the gather
                  if ((kb == 2 || kb == 5) && pend_n > 0 &&
                      ptx::mbar_try_wait(smem_u32(&sh.p_full[np & 1]), (np >> 1) & 1)) {
                    issue_pv();
                    ptx::tc_fence_after();
                  }
                }
                ptx::tc_commit(smem_u32(&sh.s_full[stage]));
                pend_stage[pend_n] = stage;
                pend_first[pend_n] = seg_first;
                ++pend_n;
                seg_first = false;
              } else {
                ptx::mbar_arrive(smem_u32(&sh.s_full[stage]));
                ptx::mbar_arrive(smem_u32(&sh.kv_empty[stage]));
              }
              ++qk_i;
              if (++j == tpt) { j = 0; ++t; }
              progressed = true;
            }
          }
          if (progressed) {
            idle_since = 0;
          } else {
            const uint64_t now = ptx::global_timer_ns();
            if (idle_since == 0) idle_since = now;
            else if (now - idle_since > 250000000ull || sh.abort_flag) fail();
          }
        }
      }
      __syncwarp();
    } else if (warp == 9) {
      // =========================== L2 prefetcher ===========================
      long t = w0 / tpt;
      int j = (int)(w0 - t * tpt);
      const int n_tiles = (int)(w1 - w0);
      for (int i = 0; i < n_tiles && !sh.abort_flag; ++i) {
        // stay at most kAtPrefetchAhead tiles ahead of the gather (bounded sleep-poll: this is only
        // pacing, nothing depends on it)
        for (int spin = 0; spin < 20000 && i >= sh.tiles_gathered + kAtPrefetchAhead && !sh.abort_flag; ++spin)
          __nanosleep(100);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int k = j * kAtTile + half * 32 + lane;
          const int slot = k < topk ? __ldg(indices + (size_t)t * index_stride + k) : -1;
          if (slot >= 0 && slot < num_slots) {
            ptx::bulk_prefetch_l2(ckv + (size_t)slot * kCkv, kCkv * 2);
            ptx::bulk_prefetch_l2(kpe + (size_t)slot * kKpe, kKpe * 2);
          }
        }
        if (++j == tpt) { j = 0; ++t; }
      }
    } else {
      // =========================== gather producers (4 warps) ===========================
      const int pw = warp - 5;                       // producer warp 0..3
      const int sub = lane >> 3, ch = lane & 7;      // row inside a 4-row group, 16-byte chunk of a block
      int i_tile = 0, qb = 0, qphase = 0;
      long cur_t = -1;
      bool ok = true;
      auto load_indices = [&](long tt, int jj, int& a, int& b) {
        const int k0 = jj * kAtTile + lane, k1 = k0 + 32;
        a = k0 < topk ? __ldg(indices + (size_t)tt * index_stride + k0) : -1;
        b = k1 < topk ? __ldg(indices + (size_t)tt * index_stride + k1) : -1;
      };
      long t = w0 / tpt;
      int j = (int)(w0 - t * tpt);
      int nv0, nv1;
      load_indices(t, j, nv0, nv1);
      for (long w = w0; w < w1; ++w, ++i_tile) {
        const int stage = i_tile & 1, phase = (i_tile >> 1) & 1;
        if (t != cur_t) {
          if (lane == 0) {
            ok = !sh.abort_flag && ptx::mbar_wait(smem_u32(&sh.q_empty[qb]), qphase ^ 1);
            if (!ok && !sh.abort_flag) { sh.abort_flag = 1; raise_status(status, DSA_STATUS_WAIT_TIMEOUT); }
          }
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) break;
          const uint32_t qdst = q_addr + qb * kAtQBytes;
          const int ptid = pw * 32 + lane;
#pragma unroll
          for (int it = 0; it < 9; ++it) {
            const int c = it * 128 + ptid, h = c / 72, jj = c - h * 72;
            const __nv_bfloat16* src = jj < 64 ? q_nope + ((size_t)(t * kHeads + h) * kCkv + jj * 8)
                                               : q_pe + ((size_t)(t * kHeads + h) * kKpe + (jj - 64) * 8);
            ptx::cp_async16(qdst + (jj >> 3) * kAtQBlockBytes + h * 128 + (((jj & 7) ^ (h & 7)) << 4), src, 16);
          }
          ptx::cp_async_arrive_noinc(smem_u32(&sh.q_full[qb]));
          cur_t = t;
          qb ^= 1;
          if (qb == 0) qphase ^= 1;
        }
        // the tile's 64 indices, two per lane (positions lane and lane+32); every warp reads all of
        // them so that each knows on its own whether the tile has any valid row.  They were
        // requested one tile ahead, so their latency is hidden behind the previous tile's copies.
        int v0 = nv0, v1 = nv1;
        long t_next = t;
        int j_next = j + 1;
        if (j_next == tpt) { j_next = 0; ++t_next; }
        if (w + 1 < w1) load_indices(t_next, j_next, nv0, nv1);
        if (v0 >= num_slots || v1 >= num_slots) {
          raise_status(status, DSA_STATUS_BAD_SLOT);
          if (v0 >= num_slots) v0 = -1;
          if (v1 >= num_slots) v1 = -1;
        }
        if (v0 < 0) v0 = -1;
        if (v1 < 0) v1 = -1;
        const bool live = __any_sync(0xffffffffu, v0 >= 0 || v1 >= 0);
        // rows of this thread: group g = pw + 4*gi, row = 4*g + sub
        int slot[4];
#pragma unroll
        for (int gi = 0; gi < 4; ++gi) {
          const int r = 4 * (pw + 4 * gi) + sub;
          const int a = __shfl_sync(0xffffffffu, v0, r & 31), b = __shfl_sync(0xffffffffu, v1, r & 31);
          slot[gi] = r < 32 ? a : b;
        }
        if (lane == 0) {
          ok = !sh.abort_flag && ptx::mbar_wait(smem_u32(&sh.kv_empty[stage]), phase ^ 1);
          if (!ok && !sh.abort_flag) { sh.abort_flag = 1; raise_status(status, DSA_STATUS_WAIT_TIMEOUT); }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        if (live) {
          const uint32_t dst0 = kv_addr + stage * kAtStageBytes;
#pragma unroll
          for (int gi = 0; gi < 4; ++gi) {
            const int r = 4 * (pw + 4 * gi) + sub;
            const int sl = slot[gi];
            const uint32_t nbytes = sl >= 0 ? 16u : 0u;
            const __nv_bfloat16* src_c = ckv + ((size_t)(sl >= 0 ? sl : 0) * kCkv + ch * 8);
            const __nv_bfloat16* src_p = kpe + ((size_t)(sl >= 0 ? sl : 0) * kKpe + ch * 8);
            const uint32_t dst = dst0 + r * 128 + ((ch ^ (r & 7)) << 4);
#pragma unroll
            for (int kb = 0; kb < 8; ++kb) ptx::cp_async16(dst + kb * kAtBlockBytes, src_c + kb * 64, nbytes);
            ptx::cp_async16(dst + 8 * kAtBlockBytes, src_p, nbytes);
          }
        }
        if (ch == 0) {
#pragma unroll
          for (int gi = 0; gi < 4; ++gi) sh.idx[stage][4 * (pw + 4 * gi) + sub] = slot[gi];
        }
        if (lane == 0) sh.live_w[stage][pw] = live ? 1 : 0;
        ptx::cp_async_arrive_noinc(smem_u32(&sh.kv_full[stage]));
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(smem_u32(&sh.kv_full[stage]));
        if (pw == 0 && lane == 0) sh.tiles_gathered = i_tile + 1;
        t = t_next;
        j = j_next;
      }
      ptx::cp_async_wait_all();
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    if (sh.abort_flag) {
      for (int i = 0; i < 64; ++i) __nanosleep(20000);
    }
    ptx::tmem_dealloc(tmem_base, kAtTmemCols);
  }
}

size_t at_tc_workspace_bytes_auto(int tokens, int topk) {
  return at_tc_workspace_bytes(tokens, topk, sm_count());
}

cudaError_t launch_sparse_attn_tc(const void* q_nope, const void* q_pe, const void* ckv,
                                  const void* kpe, const int32_t* indices, int64_t index_stride,
                                  float sm_scale, void* out, float* lse, int tokens, int topk,
                                  int64_t num_slots, void* ws, int32_t* status, cudaStream_t stream) {
  static std::atomic<uint64_t> smem_opted{0};
  {
    cudaError_t e = opt_in_dynamic_smem(reinterpret_cast<const void*>(sparse_attn_tc_kernel), kAtDynBytes,
                                        smem_opted);
    if (e != cudaSuccess) return e;
  }
  AtPlan plan = at_make_plan(tokens, topk, sm_count());
  sparse_attn_tc_kernel<<<plan.grid, kAtThreads, kAtDynBytes, stream>>>(
      static_cast<const __nv_bfloat16*>(q_nope), static_cast<const __nv_bfloat16*>(q_pe),
      static_cast<const __nv_bfloat16*>(ckv), static_cast<const __nv_bfloat16*>(kpe), indices,
      index_stride, sm_scale * kAtLog2e, static_cast<__nv_bfloat16*>(out), lse, tokens, topk,
      num_slots, plan, ws, status);
  return cudaGetLastError();
}

}  // namespace dsa
