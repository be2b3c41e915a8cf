// Sparse MLA attention over the selected rows, decode shape (16 heads per token).
//
//   logit[h,k] = (q_nope[h].ckv[idx[k]] + q_pe[h].kpe[idx[k]]) * sm_scale      idx == -1 -> masked
//   lse[h]     = log2( sum_k e^{logit[h,k]} )          out[h] = softmax_k(logit[h,:]) @ ckv[idx[:]]
// (reference arithmetic: sparse_baseline.py:18-45; kernels this replaces: sparse_fused.py:23-285 and
//  the Gluon _dsa_decode_gluon of archive/fable/dsa_sparse_attention_*.py:77-433).
//
// Why warp-level MMA here: with 16 heads the tcgen05 formulation has N = 16, and a tcgen05.mma costs
// max(45.6, N/2) cycles whatever M is -- 52 instructions per 64-row tile, 3.0-4.7 k cycles, more than
// the HBM time of the tile.  mma.sync m16n8k16 was measured on this part at 2.0 cycles per
// instruction per SM (about 1020 MAC/clk); M = 16 is exactly the head count, so a tile is 544
// instructions = 1.1 k cycles, and the kernel is bound by the gather as it should be.
//
// Structure (one CTA of 8 warps per SM, no warp specialisation, no mbarrier, nothing that spins):
//   * three 64-row stages in shared memory, filled by cp.async 16-byte copies issued by all warps
//     two tiles ahead; a tile is nine [64 rows x 128 B] blocks (8 ckv column blocks + kpe) with the
//     16-byte chunks of a row XOR-swizzled by (row & 7), so both ldmatrix patterns below are
//     conflict-free; masked rows (-1) are zero-filled.  Measured alternatives for the gather, all
//     slower at the headline shape (64 tokens): cp.async.bulk per row into linear padded rows
//     (92.7 us against 50.5 us at the time: ~70 cycles per bulk request), an L2 bulk-prefetch stream a
//     few tiles ahead (56-69 us against 42-44 us), two or three of the nine blocks by TMA
//     tile::gather4 next to the cp.async copies (36.1-37.4 us against 35.1 us; 4096-token prefill
//     1.81-1.85 ms against 1.54 ms);
//   * S[16 heads, 64 rows] = Q.K^T: warp w owns rows 8w..8w+7; q lives in registers as the 36
//     A fragments of the token (loaded once per token), K fragments come from ldmatrix.x4;
//   * online softmax in base 2 with a lazily refreshed running max (refreshed, and O rescaled in
//     registers, only when a logit exceeds it by more than 2^8); P^T goes through 2 KB of shared
//     memory so that every warp sees all 64 rows;
//   * O[16 heads, 512] += P.V: warp w owns output columns 64w..64w+63 = column block w of the same
//     tile, read with ldmatrix.x4.trans; accumulators stay in registers;
//   * work split, chosen on the host: (a) a CLUSTER of 1/2/4/8 CTAs per token when that fills at
//     least 85 % of the SMs: each CTA takes an equal share of the token's tiles and the partial
//     results are merged through distributed shared memory (every warp's 64 output columns go to
//     the CTA that owns that column block; no global partials, fences or atomics); (b) otherwise the
//     (token, tile) sequence is cut into equal contiguous ranges, one per CTA, and tokens covered by
//     several CTAs leave partials in the workspace that the last-arriving CTA merges.
#include <cooperative_groups.h>

#include <cstdlib>

#include "attn_plan.cuh"
#include "common.cuh"
#include "ptx.cuh"
#include "tmap.cuh"

namespace dsa {

namespace cg = cooperative_groups;

constexpr int kMmStages = 3;
constexpr int kMmBlockBytes = kAtTile * 128;        // 8192
constexpr int kMmStageBytes = 9 * kMmBlockBytes;    // 73728
constexpr int kMmThreads = 256;
constexpr int kMmPBytes = kHeads * 128;             // P^T [16 heads][64 rows] bf16
constexpr float kMmLog2e = 1.4426950408889634f;
constexpr float kMmRescaleGap = 8.f;

struct MmShared {
  int idx[kMmStages][kAtTile];
  int live[kMmStages];
  float red[8][kHeads];
  int is_last;
};

constexpr size_t kMmDynBytes = 128 + kMmStages * kMmStageBytes + kMmPBytes + sizeof(MmShared);

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
// D[16x8] += A[16x16] . B[16x8], bf16 inputs, fp32 accumulate.
__device__ __forceinline__ void hmma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf162(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait_group() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Merge of a token's partials by the CTA that arrives last, in the accumulator layout of the
// kernel: every thread reads, for each segment in ascending order, the 32 values it would itself
// have written (its own segment included, so that the summation order -- and with it the result,
// bit for bit -- does not depend on which CTA happens to arrive last).  Two segments per round
// with all loads of a round in flight: the merge is latency-bound, one L2 round trip per round.
__device__ __forceinline__ void mm_merge_segments(const AtPartials& part, long t, int n_seg,
                                                  int segs_max, float (&o)[8][4],
                                                  __nv_bfloat16* out, float* lse, int w, int g, int t4) {
  const int col = 64 * w + 2 * t4;
  float mx0 = -INFINITY, mx1 = -INFINITY, ls0 = 0.f, ls1 = 0.f;
#pragma unroll
  for (int nn = 0; nn < 8; ++nn) o[nn][0] = o[nn][1] = o[nn][2] = o[nn][3] = 0.f;
  for (int s0 = 0; s0 < n_seg; s0 += 2) {
    float2 v[2][16];
    float ms[2][2], lsg[2][2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int s = s0 + u < n_seg ? s0 + u : s0;
      const size_t slot = (size_t)t * segs_max + s;
      const float* pa = part.acc + (slot * kHeads + g) * kCkv + col;
#pragma unroll
      for (int nn = 0; nn < 8; ++nn) {
        v[u][nn] = *reinterpret_cast<const float2*>(pa + 8 * nn);
        v[u][8 + nn] = *reinterpret_cast<const float2*>(pa + 8 * kCkv + 8 * nn);
      }
      ms[u][0] = part.m[slot * kHeads + g];
      ms[u][1] = part.m[slot * kHeads + g + 8];
      lsg[u][0] = part.l[slot * kHeads + g];
      lsg[u][1] = part.l[slot * kHeads + g + 8];
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (s0 + u >= n_seg) continue;
      const float n0 = fmaxf(mx0, ms[u][0]), n1 = fmaxf(mx1, ms[u][1]);
      const float c0 = mx0 == -INFINITY ? 0.f : exp2f(mx0 - n0), c1 = mx1 == -INFINITY ? 0.f : exp2f(mx1 - n1);
      const float f0 = ms[u][0] == -INFINITY ? 0.f : exp2f(ms[u][0] - n0);
      const float f1 = ms[u][1] == -INFINITY ? 0.f : exp2f(ms[u][1] - n1);
#pragma unroll
      for (int nn = 0; nn < 8; ++nn) {
        o[nn][0] = o[nn][0] * c0 + v[u][nn].x * f0;
        o[nn][1] = o[nn][1] * c0 + v[u][nn].y * f0;
        o[nn][2] = o[nn][2] * c1 + v[u][8 + nn].x * f1;
        o[nn][3] = o[nn][3] * c1 + v[u][8 + nn].y * f1;
      }
      ls0 = ls0 * c0 + lsg[u][0] * f0;
      ls1 = ls1 * c1 + lsg[u][1] * f1;
      mx0 = n0;
      mx1 = n1;
    }
  }
  const float i0 = ls0 > 0.f ? 1.f / ls0 : 0.f, i1 = ls1 > 0.f ? 1.f / ls1 : 0.f;
  __nv_bfloat16* oa = out + ((size_t)t * kHeads + g) * kCkv + col;
  __nv_bfloat16* ob = oa + 8 * kCkv;
#pragma unroll
  for (int nn = 0; nn < 8; ++nn) {
    *reinterpret_cast<uint32_t*>(oa + 8 * nn) = pack_bf162(o[nn][0] * i0, o[nn][1] * i0);
    *reinterpret_cast<uint32_t*>(ob + 8 * nn) = pack_bf162(o[nn][2] * i1, o[nn][3] * i1);
  }
  if (w == 0 && t4 == 0) {
    lse[(size_t)t * kHeads + g] = ls0 > 0.f ? mx0 + log2f(ls0) : -INFINITY;
    lse[(size_t)t * kHeads + g + 8] = ls1 > 0.f ? mx1 + log2f(ls1) : -INFINITY;
  }
}

template <bool kCluster>
__global__ void __launch_bounds__(kMmThreads, 1)
sparse_attn_mma_kernel(const __nv_bfloat16* __restrict__ q_nope, const __nv_bfloat16* __restrict__ q_pe,
                       const __nv_bfloat16* __restrict__ ckv, const __nv_bfloat16* __restrict__ kpe,
                       const int32_t* __restrict__ indices, int64_t index_stride, float scale_log2,
                       __nv_bfloat16* __restrict__ out, float* __restrict__ lse, int tokens, int topk,
                       int64_t num_slots, AtPlan plan, void* ws_raw, int32_t* status) {
  extern __shared__ unsigned char dyn_raw[];
  const uint32_t raw_addr = smem_u32(dyn_raw);
  const uint32_t pad = (128u - (raw_addr & 127u)) & 127u;
  const uint32_t kv_addr = raw_addr + pad;
  const uint32_t p_addr = kv_addr + kMmStages * kMmStageBytes;
  unsigned char* p_ptr = dyn_raw + pad + kMmStages * kMmStageBytes;
  MmShared& sh = *reinterpret_cast<MmShared*>(p_ptr + kMmPBytes);

  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  const int tpt = plan.tiles_per_token;
  const long total = (long)tokens * tpt;
  long w0, w1;
  if (kCluster) {   // plan.per_cta holds the cluster size: rank r takes the r-th share of the token's tiles
    const int csize = plan.per_cta, rank = (int)blockIdx.x % csize;
    const long tok = blockIdx.x / csize;
    w0 = tok * tpt + (long)rank * tpt / csize;
    w1 = tok * tpt + (long)(rank + 1) * tpt / csize;
  } else {
    w0 = (long)blockIdx.x * plan.per_cta;
    w1 = w0 + plan.per_cta < total ? w0 + plan.per_cta : total;
  }
  const int n = (int)(w1 - w0);
  if (!kCluster && n <= 0) return;
  AtPartials part = at_carve(ws_raw, tokens, plan.segs_max);

  // ---------------- gather issue: tile `issued` goes to stage issued % 3 ------------------------
  long ti = w0 / tpt;                 // (token, tile-in-token) of the tile whose indices are requested next
  int ji = (int)(w0 - ti * tpt);
  // indices of the next tile to issue (nv) and of the one after it (nw), two per lane: requested
  // two tiles ahead so that no issue ever waits for its index row (the first two go out together)
  int issued = 0, nv0 = -1, nv1 = -1, nw0 = -1, nw1 = -1;
  auto load_indices = [&](long tt, int jj, int& a, int& b) {
    const int k0 = jj * kAtTile + lane, k1 = k0 + 32;
    a = k0 < topk ? __ldg(indices + (size_t)tt * index_stride + k0) : -1;
    b = k1 < topk ? __ldg(indices + (size_t)tt * index_stride + k1) : -1;
  };
  auto advance = [&]() { if (++ji == tpt) { ji = 0; ++ti; } };
  ptx::grid_dependency_wait();  // the index rows may come from the kernel before us in the stream
  ptx::launch_dependents();     // from here on the next kernel in the stream may run its set-up under our tail
  if (n > 0) { load_indices(ti, ji, nv0, nv1); advance(); }
  if (n > 1) { load_indices(ti, ji, nw0, nw1); advance(); }
  const int sub = lane >> 3, ch = lane & 7;  // row inside a 4-row group, 16-byte chunk of a 128-byte block
  auto issue_tile = [&]() {
    if (issued < n) {
      const int s = issued % kMmStages;
      int v0 = nv0, v1 = nv1;
      nv0 = nw0; nv1 = nw1;
      if (issued + 2 < n) { load_indices(ti, ji, nw0, nw1); advance(); }
      if (v0 >= num_slots || v1 >= num_slots) {
        raise_status(status, DSA_STATUS_BAD_SLOT);
        if (v0 >= num_slots) v0 = -1;
        if (v1 >= num_slots) v1 = -1;
      }
      if (v0 < 0) v0 = -1;
      if (v1 < 0) v1 = -1;
      const bool live = __any_sync(0xffffffffu, v0 >= 0 || v1 >= 0);
      const uint32_t dst0 = kv_addr + s * kMmStageBytes;
#pragma unroll
      for (int gi = 0; gi < 2; ++gi) {       // this warp copies row groups w and w + 8
        const int r = 4 * (w + 8 * gi) + sub;
        const int a = __shfl_sync(0xffffffffu, v0, r & 31), b = __shfl_sync(0xffffffffu, v1, r & 31);
        const int sl = r < 32 ? a : b;
        if (live) {
          const uint32_t nbytes = sl >= 0 ? 16u : 0u;
          const __nv_bfloat16* src_c = ckv + ((size_t)(sl >= 0 ? sl : 0) * kCkv + ch * 8);
          const __nv_bfloat16* src_p = kpe + ((size_t)(sl >= 0 ? sl : 0) * kKpe + ch * 8);
          const uint32_t dst = dst0 + r * 128 + ((ch ^ (r & 7)) << 4);
#pragma unroll
          for (int kb = 0; kb < 8; ++kb) ptx::cp_async16(dst + kb * kMmBlockBytes, src_c + kb * 64, nbytes);
          ptx::cp_async16(dst + 8 * kMmBlockBytes, src_p, nbytes);
        }
        if (ch == 0) sh.idx[s][r] = sl;
      }
      if (tid == 0) sh.live[s] = live ? 1 : 0;
    }
    cp_async_commit();  // always: keeps "all but the newest group" == "tile i has landed"
    ++issued;
  };
  // q of the first token is requested before the first two tiles, into the third stage, so that
  // its latency overlaps theirs
  auto stage_q = [&](long tt, uint32_t qs) {
    for (int c = tid; c < kHeads * 72; c += kMmThreads) {
      const int h = c / 72, jj = c - h * 72;
      const __nv_bfloat16* src = jj < 64 ? q_nope + ((size_t)(tt * kHeads + h) * kCkv + jj * 8)
                                         : q_pe + ((size_t)(tt * kHeads + h) * kKpe + (jj - 64) * 8);
      ptx::cp_async16(qs + h * 1168 + jj * 16, src, 16);
    }
    cp_async_commit();
  };
  if (n > 0) stage_q(w0 / tpt, kv_addr + 2 * kMmStageBytes);
  issue_tile();
  issue_tile();

  // ---------------- per-token state --------------------------------------------------------------
  uint32_t qa[36][4];          // A fragments of q: k-step ks covers columns 16 ks .. 16 ks + 15
  float o[8][4];               // O[heads g / g+8][columns 64 w + 8 n + 2 t4, +1]
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  if (kCluster) {   // a rank without tiles still takes part in the merge
#pragma unroll
    for (int nn = 0; nn < 8; ++nn) o[nn][0] = o[nn][1] = o[nn][2] = o[nn][3] = 0.f;
  }
  long t = w0 / tpt, cur_t = -1;
  int j = (int)(w0 - t * tpt) - 1;

  for (int i = 0; i < n; ++i) {
    if (++j == tpt) { j = 0; ++t; }
    const bool new_token = t != cur_t;
    cp_async_wait_group<1>();   // tile i has landed (only the newest group, tile i+1, may be pending)
    __syncthreads();            // ... for every thread; and everyone is done with tile i-1
    if (new_token) {
      // q of the new token: staged once, coalesced, in the stage that tile i-1 has just left (it is
      // handed to tile i+2 right after), then read as the 36 A fragments by every warp.  Rows of
      // 1152 B at a pitch of 1168 B keep the ldmatrix reads conflict-free.
      const uint32_t qs = kv_addr + ((i + 2) % kMmStages) * kMmStageBytes;
      if (i > 0) {   // (the first token's q was requested before the loop and has landed with tile 0)
        stage_q(t, qs);
        cp_async_wait_group<0>();
        __syncthreads();
      }
      const uint32_t qrow = qs + ((lane & 7) + ((lane >> 3) & 1) * 8) * 1168 + (lane >> 4) * 16;
#pragma unroll
      for (int ks = 0; ks < 36; ++ks) ldsm_x4(qrow + ks * 32, qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3]);
#pragma unroll
      for (int nn = 0; nn < 8; ++nn) o[nn][0] = o[nn][1] = o[nn][2] = o[nn][3] = 0.f;
      m0 = m1 = -INFINITY;
      l0 = l1 = 0.f;
      cur_t = t;
      __syncthreads();          // the staging area may now be overwritten by tile i+2
    }
    issue_tile();               // tile i+2 -> the stage tile i-1 used
    const int s = i % kMmStages;
    if (sh.live[s]) {
      const uint32_t sa = kv_addr + s * kMmStageBytes;
      // ---- S = Q . K^T for rows 8w .. 8w+7 -----------------------------------------------------
      // four accumulator chains (one per k-step of a column block): a single chain of 36
      // dependent mma.sync would be latency-bound
      float sacc[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
      float sc[4] = {0.f, 0.f, 0.f, 0.f}, sd[4] = {0.f, 0.f, 0.f, 0.f};
      {
        const int row_l = 8 * w + (lane & 7);
        const uint32_t brow = sa + row_l * 128;
        const int rx = row_l & 7, quad = lane >> 3;
#pragma unroll
        for (int kb = 0; kb < 9; ++kb) {
#pragma unroll
          for (int kk = 0; kk < 2; ++kk) {
            uint32_t r0, r1, r2, r3;
            ldsm_x4(brow + kb * kMmBlockBytes + (((kk * 4 + quad) ^ rx) << 4), r0, r1, r2, r3);
            if (kk == 0) {
              hmma_16816(sacc, qa[kb * 4], r0, r1);
              hmma_16816(sb, qa[kb * 4 + 1], r2, r3);
            } else {
              hmma_16816(sc, qa[kb * 4 + 2], r0, r1);
              hmma_16816(sd, qa[kb * 4 + 3], r2, r3);
            }
          }
        }
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) sacc[e] = (sacc[e] + sb[e]) + (sc[e] + sd[e]);
      const int ra = 8 * w + 2 * t4;
      const bool va = sh.idx[s][ra] >= 0, vb = sh.idx[s][ra + 1] >= 0;
      const float x0 = va ? sacc[0] * scale_log2 : -INFINITY, x1 = vb ? sacc[1] * scale_log2 : -INFINITY;
      const float x2 = va ? sacc[2] * scale_log2 : -INFINITY, x3 = vb ? sacc[3] * scale_log2 : -INFINITY;
      const bool need = fmaxf(x0, x1) > m0 + kMmRescaleGap || fmaxf(x2, x3) > m1 + kMmRescaleGap;
      // P^T[head][row]: rows 8w..8w+7 are 16-byte chunk w of the head's 128-byte line
      uint32_t* pa0 = reinterpret_cast<uint32_t*>(p_ptr + g * 128 + ((w ^ (g & 7)) << 4) + t4 * 4);
      uint32_t* pa1 = reinterpret_cast<uint32_t*>(p_ptr + (g + 8) * 128 + ((w ^ (g & 7)) << 4) + t4 * 4);
      float u0 = m0 == -INFINITY ? 0.f : m0, u1 = m1 == -INFINITY ? 0.f : m1;
      float p0 = exp2f(x0 - u0), p1 = exp2f(x1 - u0), p2 = exp2f(x2 - u1), p3 = exp2f(x3 - u1);
      // optimistic: publish P with the running max as it is; the same barrier that makes P visible
      // tells whether some logit exceeded the max by more than 2^8 (rare)
      *pa0 = pack_bf162(p0, p1);
      *pa1 = pack_bf162(p2, p3);
      if (__syncthreads_or(need)) {
        // refresh the running max of every head over the tile, rescale the accumulators, redo P
        float v0 = fmaxf(x0, x1), v1 = fmaxf(x2, x3);
        v0 = fmaxf(v0, __shfl_xor_sync(0xffffffffu, v0, 1));
        v0 = fmaxf(v0, __shfl_xor_sync(0xffffffffu, v0, 2));
        v1 = fmaxf(v1, __shfl_xor_sync(0xffffffffu, v1, 1));
        v1 = fmaxf(v1, __shfl_xor_sync(0xffffffffu, v1, 2));
        if (t4 == 0) { sh.red[w][g] = v0; sh.red[w][g + 8] = v1; }
        __syncthreads();
        float mx0 = sh.red[0][g], mx1 = sh.red[0][g + 8];
#pragma unroll
        for (int ww = 1; ww < 8; ++ww) { mx0 = fmaxf(mx0, sh.red[ww][g]); mx1 = fmaxf(mx1, sh.red[ww][g + 8]); }
        const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
        const float c0 = n0 == -INFINITY ? 1.f : exp2f(m0 - n0), c1 = n1 == -INFINITY ? 1.f : exp2f(m1 - n1);
#pragma unroll
        for (int nn = 0; nn < 8; ++nn) { o[nn][0] *= c0; o[nn][1] *= c0; o[nn][2] *= c1; o[nn][3] *= c1; }
        l0 *= c0; l1 *= c1;
        m0 = n0; m1 = n1;
        u0 = m0 == -INFINITY ? 0.f : m0; u1 = m1 == -INFINITY ? 0.f : m1;
        p0 = exp2f(x0 - u0); p1 = exp2f(x1 - u0); p2 = exp2f(x2 - u1); p3 = exp2f(x3 - u1);
        *pa0 = pack_bf162(p0, p1);
        *pa1 = pack_bf162(p2, p3);
        __syncthreads();
      }
      l0 += p0 + p1;
      l1 += p2 + p3;
      // ---- O += P . V for columns 64w .. 64w+63 (column block w of the tile) ---------------------
      {
        const int hrow = (lane & 7) + ((lane >> 3) & 1) * 8, half = lane >> 4;
        const uint32_t pa = p_addr + hrow * 128;
        const uint32_t vbase = sa + w * kMmBlockBytes;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          uint32_t a[4];
          ldsm_x4(pa + (((ks * 2 + half) ^ (hrow & 7)) << 4), a[0], a[1], a[2], a[3]);
          const int vrow = ks * 16 + hrow;
          const uint32_t va_addr = vbase + vrow * 128;
#pragma unroll
          for (int np = 0; np < 4; ++np) {
            uint32_t r0, r1, r2, r3;
            ldsm_x4_trans(va_addr + (((np * 2 + half) ^ (vrow & 7)) << 4), r0, r1, r2, r3);
            hmma_16816(o[2 * np], a, r0, r1);
            hmma_16816(o[2 * np + 1], a, r2, r3);
          }
        }
      }
    }
    if (!kCluster && (j == tpt - 1 || i == n - 1)) {
      // ------------------ end of this CTA's segment of token t ------------------------------------
      float s0 = l0, s1 = l1;
      s0 += __shfl_xor_sync(0xffffffffu, s0, 1);
      s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
      s1 += __shfl_xor_sync(0xffffffffu, s1, 1);
      s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
      __syncthreads();  // sh.red may still be read by a slow warp of a refresh above
      if (t4 == 0) { sh.red[w][g] = s0; sh.red[w][g + 8] = s1; }
      __syncthreads();
      float lt0 = 0.f, lt1 = 0.f;
#pragma unroll
      for (int ww = 0; ww < 8; ++ww) { lt0 += sh.red[ww][g]; lt1 += sh.red[ww][g + 8]; }
      const long first_tile = t * tpt, last_tile = first_tile + tpt - 1;
      const int cta_first = (int)(first_tile / plan.per_cta), cta_last = (int)(last_tile / plan.per_cta);
      const int n_seg = cta_last - cta_first + 1, seg = (int)blockIdx.x - cta_first;
      const int col = 64 * w + 2 * t4;
      if (n_seg == 1) {
        const float i0 = lt0 > 0.f ? 1.f / lt0 : 0.f, i1 = lt1 > 0.f ? 1.f / lt1 : 0.f;
        __nv_bfloat16* oa = out + ((size_t)t * kHeads + g) * kCkv + col;
        __nv_bfloat16* ob = oa + 8 * kCkv;
#pragma unroll
        for (int nn = 0; nn < 8; ++nn) {
          *reinterpret_cast<uint32_t*>(oa + 8 * nn) = pack_bf162(o[nn][0] * i0, o[nn][1] * i0);
          *reinterpret_cast<uint32_t*>(ob + 8 * nn) = pack_bf162(o[nn][2] * i1, o[nn][3] * i1);
        }
        if (w == 0 && t4 == 0) {
          lse[(size_t)t * kHeads + g] = lt0 > 0.f ? m0 + log2f(lt0) : -INFINITY;
          lse[(size_t)t * kHeads + g + 8] = lt1 > 0.f ? m1 + log2f(lt1) : -INFINITY;
        }
      } else {
        float* pa = part.acc + (((size_t)t * plan.segs_max + seg) * kHeads + g) * kCkv + col;
        float* pb = pa + 8 * kCkv;
#pragma unroll
        for (int nn = 0; nn < 8; ++nn) {
          *reinterpret_cast<float2*>(pa + 8 * nn) = make_float2(o[nn][0], o[nn][1]);
          *reinterpret_cast<float2*>(pb + 8 * nn) = make_float2(o[nn][2], o[nn][3]);
        }
        if (w == 0 && t4 == 0) {
          const size_t base = ((size_t)t * plan.segs_max + seg) * kHeads;
          part.m[base + g] = lt0 > 0.f ? m0 : -INFINITY;
          part.l[base + g] = lt0;
          part.m[base + g + 8] = lt1 > 0.f ? m1 : -INFINITY;
          part.l[base + g + 8] = lt1;
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) {
          const int old = atomicAdd(&part.counters[t], 1);
          sh.is_last = old == n_seg - 1;
          if (sh.is_last) part.counters[t] = 0;  // ready for the next call
        }
        __syncthreads();
        if (sh.is_last) {
          __threadfence();
          mm_merge_segments(part, t, n_seg, plan.segs_max, o, out, lse, w, g, t4);
        }
      }
    }
  }
  cp_async_wait_group<0>();
  if (kCluster) {
    // ---------------- merge across the token's cluster through distributed shared memory ----------
    // Column block b (64 output columns = what warp b of every CTA holds) is merged by rank b % c:
    // every warp sends its 16 x 64 fp32 block to that rank, every CTA sends its (m, l) to all.
    cg::cluster_group cluster = cg::this_cluster();
    const int csize = plan.per_cta, rank = (int)cluster.block_rank();
    const long tok = blockIdx.x / csize;
    float s0 = l0, s1 = l1;
    s0 += __shfl_xor_sync(0xffffffffu, s0, 1);
    s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
    s1 += __shfl_xor_sync(0xffffffffu, s1, 1);
    s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
    __syncthreads();   // every warp is done with the stages and with sh.red
    // peers write into this CTA's stage memory: they may start once every CTA of the cluster has
    // left its tile loop (arrive here, wait just before the first remote store)
    if (csize > 1) cluster.barrier_arrive();
    if (t4 == 0) { sh.red[w][g] = s0; sh.red[w][g + 8] = s1; }
    __syncthreads();
    float lt0 = 0.f, lt1 = 0.f;
#pragma unroll
    for (int ww = 0; ww < 8; ++ww) { lt0 += sh.red[ww][g]; lt1 += sh.red[ww][g + 8]; }
    const float mm0 = lt0 > 0.f ? m0 : -INFINITY, mm1 = lt1 > 0.f ? m1 : -INFINITY;
    // exchange area at the start of the stage memory of the RECEIVING CTA:
    //   xo[src rank][local block][16 heads][64 cols] fp32, then xml[src rank][2][16] (m, l)
    float* xo_local = reinterpret_cast<float*>(dyn_raw + pad);
    float* xml_local = xo_local + 8 * kHeads * 64;
    const int dst_rank = w % csize, blk_local = w / csize, blocks_per_rank = 8 / csize;
    if (csize > 1) {
      cluster.barrier_wait();
      if (dst_rank != rank) {
        float* remote = cluster.map_shared_rank(xo_local, dst_rank) +
                        ((size_t)(rank * blocks_per_rank + blk_local) * kHeads) * 64;
#pragma unroll
        for (int nn = 0; nn < 8; ++nn) {
          *reinterpret_cast<float2*>(remote + g * 64 + 8 * nn + 2 * t4) = make_float2(o[nn][0], o[nn][1]);
          *reinterpret_cast<float2*>(remote + (g + 8) * 64 + 8 * nn + 2 * t4) = make_float2(o[nn][2], o[nn][3]);
        }
      }
      if (w == 0 && t4 == 0) {
        for (int d = 0; d < csize; ++d) {
          if (d == rank) continue;
          float* r = cluster.map_shared_rank(xml_local, d) + rank * 2 * kHeads;
          r[g] = mm0; r[g + 8] = mm1;
          r[kHeads + g] = lt0; r[kHeads + g + 8] = lt1;
        }
      }
      cluster.sync();
    }
    float mx0 = mm0, mx1 = mm1, ls0 = lt0, ls1 = lt1;
    const bool merger = dst_rank == rank;
    for (int sr = 0; sr < csize; ++sr) {
      if (sr == rank) continue;
      const float* ml = xml_local + sr * 2 * kHeads;
      const float ms0 = ml[g], ms1 = ml[g + 8], lg0 = ml[kHeads + g], lg1 = ml[kHeads + g + 8];
      const float n0 = fmaxf(mx0, ms0), n1 = fmaxf(mx1, ms1);
      const float c0 = mx0 == -INFINITY ? 0.f : exp2f(mx0 - n0), c1 = mx1 == -INFINITY ? 0.f : exp2f(mx1 - n1);
      const float f0 = ms0 == -INFINITY ? 0.f : exp2f(ms0 - n0), f1 = ms1 == -INFINITY ? 0.f : exp2f(ms1 - n1);
      if (merger) {
        const float* src = xo_local + ((size_t)(sr * blocks_per_rank + blk_local) * kHeads) * 64;
#pragma unroll
        for (int nn = 0; nn < 8; ++nn) {
          const float2 va = *reinterpret_cast<const float2*>(src + g * 64 + 8 * nn + 2 * t4);
          const float2 vb = *reinterpret_cast<const float2*>(src + (g + 8) * 64 + 8 * nn + 2 * t4);
          o[nn][0] = o[nn][0] * c0 + va.x * f0;
          o[nn][1] = o[nn][1] * c0 + va.y * f0;
          o[nn][2] = o[nn][2] * c1 + vb.x * f1;
          o[nn][3] = o[nn][3] * c1 + vb.y * f1;
        }
      }
      ls0 = ls0 * c0 + lg0 * f0;
      ls1 = ls1 * c1 + lg1 * f1;
      mx0 = n0;
      mx1 = n1;
    }
    if (merger) {
      const float i0 = ls0 > 0.f ? 1.f / ls0 : 0.f, i1 = ls1 > 0.f ? 1.f / ls1 : 0.f;
      const int col = 64 * w + 2 * t4;
      __nv_bfloat16* oa = out + ((size_t)tok * kHeads + g) * kCkv + col;
      __nv_bfloat16* ob = oa + 8 * kCkv;
#pragma unroll
      for (int nn = 0; nn < 8; ++nn) {
        *reinterpret_cast<uint32_t*>(oa + 8 * nn) = pack_bf162(o[nn][0] * i0, o[nn][1] * i0);
        *reinterpret_cast<uint32_t*>(ob + 8 * nn) = pack_bf162(o[nn][2] * i1, o[nn][3] * i1);
      }
    }
    if (rank == 0 && w == 0 && t4 == 0) {
      lse[(size_t)tok * kHeads + g] = ls0 > 0.f ? mx0 + log2f(ls0) : -INFINITY;
      lse[(size_t)tok * kHeads + g + 8] = ls1 > 0.f ? mx1 + log2f(ls1) : -INFINITY;
    }
  }
}

// Cluster size for the one-cluster-per-token split, or 0 when the contiguous-range split is the
// better fit.  Candidates are the largest power of two (<= 8) that keeps tokens * size within the
// SMs, leaves every CTA at least four tiles and fits in ONE wave of clusters.  The choice follows
// a cost model fitted to per-call times at 12-120 tokens x 2048 rows (microseconds after the
// common start-up): cluster = 1.65 * tiles per CTA; contiguous = 1.86 * tiles per SM + 8, the 8
// being the partial flush, the q re-staging at token boundaries and the L2 round trips of the
// last-arriver merge.  An 8-CTA cluster always wins where it fits (16.7 against 20.6 us at 12
// tokens, 16 against 29 us at one).
// Clusters of `csize` CTAs of this kernel that can be resident at once (a cluster needs all its
// SMs inside one GPC, so this is less than SMs / csize for the larger sizes); queried once.
static int mm_max_active_clusters(int csize) {
  static std::atomic<int> cache[kMaxDevices][9];   // per device: 0 = not asked yet, -1 = query failed
  const int dev = current_device();
  std::atomic<int> uncached{0};
  std::atomic<int>& slot = (dev >= 0 && dev < kMaxDevices) ? cache[dev][csize] : uncached;
  if (slot.load(std::memory_order_relaxed) == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(csize * 64));
    cfg.blockDim = dim3(kMmThreads);
    cfg.dynamicSmemBytes = kMmDynBytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)csize;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, sparse_attn_mma_kernel<true>, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = -1;
    }
    slot.store(n, std::memory_order_relaxed);
  }
  const int n = slot.load(std::memory_order_relaxed);
  return n > 0 ? n : 0;
}

static int mm_cluster_size(int tokens, int tiles_per_token, int sms) {
  int c = 1;
  while (c < 8 && (long)tokens * c * 2 <= sms && tiles_per_token / (c * 2) >= 4) c *= 2;
  while (c > 1 && tokens > mm_max_active_clusters(c)) c /= 2;   // one wave of clusters only
  if ((long)tokens * c > sms) return 0;
  if (c == 8) return c;
  const double est_cluster = 1.65 * (double)((tiles_per_token + c - 1) / c);
  const double est_contiguous = 1.86 * (double)tokens * tiles_per_token / sms + 8.0;
  return est_cluster <= est_contiguous ? c : 0;
}

cudaError_t launch_sparse_attn_mma(const void* q_nope, const void* q_pe, const void* ckv,
                                   const void* kpe, const int32_t* indices, int64_t index_stride,
                                   float sm_scale, void* out, float* lse, int tokens, int topk,
                                   int64_t num_slots, void* ws, int32_t* status, cudaStream_t stream) {
  static std::atomic<uint64_t> smem_opted_a{0}, smem_opted_b{0};
  {
    cudaError_t e = opt_in_dynamic_smem(reinterpret_cast<const void*>(sparse_attn_mma_kernel<false>),
                                        kMmDynBytes, smem_opted_a);
    if (e == cudaSuccess)
      e = opt_in_dynamic_smem(reinterpret_cast<const void*>(sparse_attn_mma_kernel<true>), kMmDynBytes,
                              smem_opted_b);
    if (e != cudaSuccess) return e;
  }
  static int cluster_ok = -1;
  if (cluster_ok < 0) {   // DSA_ATT_CLUSTER=0 forces the contiguous-range split (for A/B timing)
    const char* e = getenv("DSA_ATT_CLUSTER");
    cluster_ok = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  AtPlan plan = at_make_plan(tokens, topk, sm_count());
  const int csize = cluster_ok ? mm_cluster_size(tokens, plan.tiles_per_token, sm_count()) : 0;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kMmThreads);
  cfg.dynamicSmemBytes = kMmDynBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled();
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (csize > 0) {
    plan.per_cta = csize;   // the kernel reads the cluster size from here
    cfg.gridDim = dim3((unsigned)(tokens * csize));
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = (unsigned)csize;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, sparse_attn_mma_kernel<true>,
                              static_cast<const __nv_bfloat16*>(q_nope),
                              static_cast<const __nv_bfloat16*>(q_pe),
                              static_cast<const __nv_bfloat16*>(ckv),
                              static_cast<const __nv_bfloat16*>(kpe), indices, index_stride,
                              sm_scale * kMmLog2e, static_cast<__nv_bfloat16*>(out), lse, tokens, topk,
                              num_slots, plan, ws, status);
  }
  cfg.gridDim = dim3((unsigned)plan.grid);
  return cudaLaunchKernelEx(&cfg, sparse_attn_mma_kernel<false>,
                            static_cast<const __nv_bfloat16*>(q_nope),
                            static_cast<const __nv_bfloat16*>(q_pe),
                            static_cast<const __nv_bfloat16*>(ckv),
                            static_cast<const __nv_bfloat16*>(kpe), indices, index_stride,
                            sm_scale * kMmLog2e, static_cast<__nv_bfloat16*>(out), lse, tokens, topk,
                            num_slots, plan, ws, status);
}

}  // namespace dsa
