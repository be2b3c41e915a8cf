// Shared device/host helpers for the dsa_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/dsa_b200.h"

namespace dsa {

constexpr int kPage = DSA_PAGE_SIZE;
constexpr int kIdxHeads = DSA_INDEX_HEADS;
constexpr int kIdxDim = DSA_INDEX_DIM;
constexpr int kPageBytes = DSA_INDEX_PAGE_BYTES;
constexpr int kPageDataBytes = kPage * kIdxDim;  // 8192
constexpr int kTopK = DSA_TOPK;
constexpr int kHeads = DSA_ATTN_HEADS;
constexpr int kCkv = DSA_CKV_DIM;
constexpr int kKpe = DSA_KPE_DIM;

// Upper bound on polls of any device-side wait.  Each poll is a try_wait with a hardware
// suspend-time hint, so this is far longer than any legitimate wait, yet a lost arrival ends
// the kernel with DSA_STATUS_WAIT_TIMEOUT instead of hanging the GPU.
constexpr uint32_t kMaxPolls = 1u << 22;

__device__ __forceinline__ void raise_status(int32_t* status, uint32_t bits) {
  if (status != nullptr) atomicOr(reinterpret_cast<unsigned int*>(status), bits);
}

__device__ __forceinline__ float e4m3_to_float(uint8_t v) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(v), __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}

// Order-preserving map fp32 -> u32: a > b (as floats, -0 < +0) <=> key(a) > key(b).
__device__ __forceinline__ uint32_t float_to_ordered(float f) {
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Size of the per-token arrival-counter region at the start of every attention workspace layout.
// The counters must be zero between calls (the last arriver resets its own), so no layout may ever
// put partial results where another call's counters live: the region has one fixed size for every
// token count that uses counters at all (splitting a token over CTAs stops far below 4096 tokens).
__host__ __device__ inline size_t attn_counter_region_bytes(int tokens) {
  const size_t need = (((size_t)tokens * 4 + 255) / 256) * 256;
  return need < 16384 ? 16384 : need;
}

__device__ __forceinline__ float ordered_to_float(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k ^ 0x80000000u) : ~k);
}

// Per-request score histograms (decode shapes): the scorer counts every score into 4096 bins over
// the top 12 bits of its order-preserving key, the selection kernel starts from the finished
// histogram and puts it back to zero.  The region sits in front of the score rows of the indexer
// workspace and has one fixed size whatever the batch, so that it is zero between calls.
constexpr int kHistMaxBatch = 1024;       // larger batches take the min/max path
constexpr int kHistBins = 4096;
constexpr size_t kHistRegionBytes = (size_t)kHistMaxBatch * kHistBins * sizeof(uint32_t);

// Where the selection sends a finished index row in a head-sharded layer: every rank's staging
// buffer of (id, epoch) pairs as seen from this GPU (entry `rank` unused).  world <= 1: nothing is sent.
constexpr int kRowSendMaxWorld = 8;
struct RowSend {
  uint2* stage[kRowSendMaxWorld];
  int world, rank, row_offset, row_width;
  uint32_t epoch;
};
// Store row `index` (row_width ids at `row`, complete and visible to this CTA) into every peer's
// staging buffer as (id, epoch) pairs, 16 bytes per store; by all threads of the calling CTA.
__device__ __forceinline__ void send_row_pairs(const RowSend& xs, const int32_t* row, int index) {
  const int units = xs.row_width / 2;
  for (int u = threadIdx.x; u < units; u += blockDim.x) {
    const int2 v = __ldcg(reinterpret_cast<const int2*>(row) + u);
    const uint4 packed = make_uint4((uint32_t)v.x, xs.epoch, (uint32_t)v.y, xs.epoch);
    // (constant indices: the table stays in the kernel's parameter space, no local copy)
#pragma unroll
    for (int p = 0; p < kRowSendMaxWorld; ++p) {
      if (p < xs.world && p != xs.rank)
        reinterpret_cast<uint4*>(xs.stage[p] + (size_t)index * xs.row_width)[u] = packed;
    }
  }
}
// This rank's own staging buffer.
__device__ __forceinline__ uint2* own_stage(const RowSend& xs) {
  uint2* p = xs.stage[0];
#pragma unroll
  for (int r = 1; r < kRowSendMaxWorld; ++r)
    if (r == xs.rank) p = xs.stage[r];
  return p;
}

// -inf and NaN scores are ranked as this value by the selection (and by the scorer's min / max).
constexpr float kScoreFloor = -3.0e38f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

}  // namespace dsa
