// Plain CUDA-core scorer for the FP8 indexer.  It exists as an on-device cross-check for the
// tensor-core scorer at sizes the CPU oracle cannot reach in reasonable time: products of e4m3
// values are exact in fp32 and are summed here with ordinary fp32 FMAs.
//
// score[b,t] = scale[t] * sum_h w[b,h] * relu( sum_d q[b,h,d] * k[t,d] )
// (reference: indexer_baseline.py:75-80; the per-token scale is factored out of the dot product,
//  which is valid because relu(s*x) = s*relu(x) for s >= 0).
#include "common.cuh"

namespace dsa {

constexpr int kSimtThreads = 256;
constexpr int kSimtPagesPerCta = 8;

__global__ void __launch_bounds__(kSimtThreads)
indexer_score_simt_kernel(const uint8_t* __restrict__ q_fp8, const uint8_t* __restrict__ k_cache,
                          const float* __restrict__ weights, const int32_t* __restrict__ seq_lens,
                          const int32_t* __restrict__ block_table, int64_t bt_stride,
                          float* __restrict__ scores, int64_t score_stride, int num_pages,
                          int32_t* status) {
  extern __shared__ float smem[];
  float* qs = smem;                           // [128 d][64 h]
  float* ks = qs + kIdxDim * kIdxHeads;       // [64 tok][129]
  float* part = ks + kPage * (kIdxDim + 1);   // [4][64]
  float* ws = part + 4 * kPage;               // [64]

  const int b = blockIdx.y;
  const int len = seq_lens[b];
  const int n_pages = (len + kPage - 1) / kPage;
  const int first = blockIdx.x * kSimtPagesPerCta;
  if (first >= n_pages) return;
  const int tid = threadIdx.x;

  for (int i = tid; i < kIdxHeads * kIdxDim; i += kSimtThreads) {
    int h = i / kIdxDim, d = i % kIdxDim;
    qs[d * kIdxHeads + h] = e4m3_to_float(q_fp8[(size_t)b * kIdxHeads * kIdxDim + i]);
  }
  if (tid < kIdxHeads) ws[tid] = weights[(size_t)b * kIdxHeads + tid];

  const int tok = tid & 63, hq = tid >> 6;
  const int last = min(first + kSimtPagesPerCta, n_pages);
  for (int p = first; p < last; ++p) {
    __syncthreads();
    int page = block_table[(size_t)b * bt_stride + p];
    bool ok = page >= 0 && page < num_pages;
    if (!ok) {
      if (tid == 0) raise_status(status, DSA_STATUS_BAD_PAGE);
      page = 0;
    }
    const uint8_t* src = k_cache + (size_t)page * kPageBytes;
    {
      // 8192 bytes: each thread converts 32 consecutive bytes of one token row.
      const uint4* v = reinterpret_cast<const uint4*>(src) + tid * 2;
      uint4 a = v[0], c = v[1];
      uint32_t w32[8] = {a.x, a.y, a.z, a.w, c.x, c.y, c.z, c.w};
      int t = (tid * 32) / kIdxDim, d0 = (tid * 32) % kIdxDim;
#pragma unroll
      for (int j = 0; j < 32; ++j)
        ks[t * (kIdxDim + 1) + d0 + j] = e4m3_to_float((w32[j >> 2] >> (8 * (j & 3))) & 0xff);
    }
    __syncthreads();
    float acc[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) acc[j] = 0.f;
    for (int d = 0; d < kIdxDim; ++d) {
      float kv = ks[tok * (kIdxDim + 1) + d];
      const float4* q4 = reinterpret_cast<const float4*>(qs + d * kIdxHeads + hq * 16);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float4 q = q4[j];
        acc[4 * j + 0] = fmaf(kv, q.x, acc[4 * j + 0]);
        acc[4 * j + 1] = fmaf(kv, q.y, acc[4 * j + 1]);
        acc[4 * j + 2] = fmaf(kv, q.z, acc[4 * j + 2]);
        acc[4 * j + 3] = fmaf(kv, q.w, acc[4 * j + 3]);
      }
    }
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) s = fmaf(ws[hq * 16 + j], fmaxf(acc[j], 0.f), s);
    part[hq * kPage + tok] = s;
    __syncthreads();
    if (hq == 0) {
      int t = p * kPage + tok;
      if (t < len) {
        float total = (part[tok] + part[kPage + tok]) + (part[2 * kPage + tok] + part[3 * kPage + tok]);
        float scale = reinterpret_cast<const float*>(src + kPageDataBytes)[tok];
        scores[(size_t)b * score_stride + t] = ok ? total * scale : -INFINITY;
      }
    }
  }
}

cudaError_t launch_indexer_score_simt(const void* q_fp8, const void* k_cache, const float* weights,
                                      const int32_t* seq_lens, const int32_t* block_table,
                                      int64_t bt_stride, float* scores, int64_t score_stride,
                                      int batch, int num_pages, int max_pages, int32_t* status,
                                      cudaStream_t stream) {
  size_t smem = sizeof(float) * (kIdxDim * kIdxHeads + kPage * (kIdxDim + 1) + 4 * kPage + kIdxHeads);
  cudaError_t e = cudaFuncSetAttribute(indexer_score_simt_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  dim3 grid((max_pages + kSimtPagesPerCta - 1) / kSimtPagesPerCta, batch);
  indexer_score_simt_kernel<<<grid, kSimtThreads, smem, stream>>>(
      static_cast<const uint8_t*>(q_fp8), static_cast<const uint8_t*>(k_cache), weights, seq_lens,
      block_table, bt_stride, scores, score_stride, num_pages, status);
  return cudaGetLastError();
}

}  // namespace dsa
