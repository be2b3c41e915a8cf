// Producers of the two paged caches the DSA path reads: the FP8 index-key pages and the bf16
// ckv/kpe pages.  Both are scatter writes of whole token rows to global slot ids
// (slot = page * 64 + position), HBM-bound and tiny next to the readers.
//
// Index-key page layout (unpacked by the reference's dequant_fp8_kv_cache,
// archive/dsa_topk_indexer_fp8_h64_d128_topk2048_ps64/solution/triton/indexer_baseline.py:16-36):
// 8448 bytes per page = 64 rows of 128 e4m3 bytes, then 64 fp32 scales; key = e4m3 * scale.
// Quantisation is per token: scale = max(|k|, 1e-12) / 448, byte = rn_e4m3(k / scale).
#include "common.cuh"

namespace dsa {

namespace {

constexpr int kWriteThreads = 256;
constexpr int kWriteWarps = kWriteThreads / 32;

template <typename T>
__device__ __forceinline__ float4 load_key4(const T* row, int lane);

template <>
__device__ __forceinline__ float4 load_key4<float>(const float* row, int lane) {
  return reinterpret_cast<const float4*>(row)[lane];
}

template <>
__device__ __forceinline__ float4 load_key4<__nv_bfloat16>(const __nv_bfloat16* row, int lane) {
  const uint2 raw = reinterpret_cast<const uint2*>(row)[lane];
  const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
  const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  return make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
}

__device__ __forceinline__ uint32_t to_e4m3(float v) {
  return static_cast<uint32_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}

// One warp per token: a lane owns 4 of the 128 components, the warp reduces |k| to its maximum,
// and the 128 quantised bytes leave as one coalesced 128-byte row.
template <typename T>
__global__ void __launch_bounds__(kWriteThreads)
index_cache_write_kernel(const T* __restrict__ keys, int64_t key_stride,
                         const int32_t* __restrict__ slots, uint8_t* __restrict__ cache, int tokens,
                         int64_t num_slots, int32_t* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  for (int t = blockIdx.x * kWriteWarps + (threadIdx.x >> 5); t < tokens;
       t += gridDim.x * kWriteWarps) {
    const int32_t slot = slots[t];
    if (slot < 0) continue;  // -1: token not cached
    if (slot >= num_slots) {
      if (lane == 0) raise_status(status, DSA_STATUS_BAD_SLOT);
      continue;
    }
    const float4 v = load_key4<T>(keys + static_cast<int64_t>(t) * key_stride, lane);
    float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    const float scale = fmaxf(amax, 1e-12f) / 448.0f;
    const uint32_t packed = to_e4m3(v.x / scale) | (to_e4m3(v.y / scale) << 8) |
                            (to_e4m3(v.z / scale) << 16) | (to_e4m3(v.w / scale) << 24);
    uint8_t* page = cache + static_cast<int64_t>(slot / kPage) * kPageBytes;
    const int pos = slot % kPage;
    reinterpret_cast<uint32_t*>(page + pos * kIdxDim)[lane] = packed;
    if (lane == 0) reinterpret_cast<float*>(page + kPageDataBytes)[pos] = scale;
  }
}

// One warp per token: 64 + 8 chunks of 16 bytes (1024-byte ckv row, 128-byte kpe row).
__global__ void __launch_bounds__(kWriteThreads)
kv_cache_append_kernel(const uint4* __restrict__ ckv, int64_t ckv_stride16,
                       const uint4* __restrict__ kpe, int64_t kpe_stride16,
                       const int32_t* __restrict__ slots, uint4* __restrict__ ckv_cache,
                       uint4* __restrict__ kpe_cache, int tokens, int64_t num_slots,
                       int32_t* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  for (int t = blockIdx.x * kWriteWarps + (threadIdx.x >> 5); t < tokens;
       t += gridDim.x * kWriteWarps) {
    const int32_t slot = slots[t];
    if (slot < 0) continue;
    if (slot >= num_slots) {
      if (lane == 0) raise_status(status, DSA_STATUS_BAD_SLOT);
      continue;
    }
    const uint4* src = ckv + static_cast<int64_t>(t) * ckv_stride16;
    uint4* dst = ckv_cache + static_cast<int64_t>(slot) * (kCkv * 2 / 16);
    const uint4 a = src[lane], b = src[lane + 32];
    uint4 c = make_uint4(0, 0, 0, 0);
    if (lane < kKpe * 2 / 16) c = kpe[static_cast<int64_t>(t) * kpe_stride16 + lane];
    dst[lane] = a;
    dst[lane + 32] = b;
    if (lane < kKpe * 2 / 16) kpe_cache[static_cast<int64_t>(slot) * (kKpe * 2 / 16) + lane] = c;
  }
}

int write_grid(int tokens) {
  const int blocks = (tokens + kWriteWarps - 1) / kWriteWarps;
  return blocks < 1 ? 1 : (blocks > 148 * 8 ? 148 * 8 : blocks);
}

}  // namespace

cudaError_t launch_index_cache_write(const void* keys, int key_dtype, int64_t key_stride,
                                     const int32_t* slots, void* cache, int tokens,
                                     int64_t num_slots, int32_t* status, cudaStream_t stream) {
  uint8_t* out = static_cast<uint8_t*>(cache);
  if (key_dtype == 0) {
    index_cache_write_kernel<float><<<write_grid(tokens), kWriteThreads, 0, stream>>>(
        static_cast<const float*>(keys), key_stride, slots, out, tokens, num_slots, status);
  } else {
    index_cache_write_kernel<__nv_bfloat16><<<write_grid(tokens), kWriteThreads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(keys), key_stride, slots, out, tokens, num_slots, status);
  }
  return cudaGetLastError();
}

cudaError_t launch_kv_cache_append(const void* ckv, int64_t ckv_stride, const void* kpe,
                                   int64_t kpe_stride, const int32_t* slots, void* ckv_cache,
                                   void* kpe_cache, int tokens, int64_t num_slots, int32_t* status,
                                   cudaStream_t stream) {
  kv_cache_append_kernel<<<write_grid(tokens), kWriteThreads, 0, stream>>>(
      static_cast<const uint4*>(ckv), ckv_stride / 8, static_cast<const uint4*>(kpe),
      kpe_stride / 8, slots, static_cast<uint4*>(ckv_cache), static_cast<uint4*>(kpe_cache), tokens,
      num_slots, status);
  return cudaGetLastError();
}

}  // namespace dsa
