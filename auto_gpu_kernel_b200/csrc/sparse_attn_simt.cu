// CUDA-core sparse MLA attention (split over the selected rows, last-arriver merge).  Kept as the
// on-device cross-check of the tensor-core kernel: plain fp32 FMAs over the same gathered rows.
//
//   logit[h,k] = (q_nope[h].ckv[idx[k]] + q_pe[h].kpe[idx[k]]) * sm_scale     idx == -1 -> masked
//   lse[h]     = log2( sum_k e^{logit[h,k]} )                                   (base 2)
//   out[h]     = softmax_k(logit[h,:]) @ ckv[idx[:]]                            -> bf16
// (reference: sparse_baseline.py:18-45).  A token with no valid index gets out = 0, lse = -inf.
#include "common.cuh"

namespace dsa {

constexpr int kAttThreads = 256;
constexpr int kAttTile = 32;                 // gathered rows per step
constexpr int kRowElems = kCkv + kKpe;       // 576
constexpr int kRowPad = kRowElems + 8;       // 16 B pad: conflict-free 16 B row reads
constexpr float kLog2e = 1.4426950408889634f;

struct AttWorkspace {
  int32_t* counters;  // [tokens] arrival counters, zero between calls
  float* m;           // [tokens][splits][16]
  float* l;           // [tokens][splits][16]
  float* acc;         // [tokens][splits][16][512]
};

__host__ __device__ inline size_t att_counter_bytes(int tokens) {
  return attn_counter_region_bytes(tokens);
}

__host__ __device__ inline AttWorkspace att_carve(void* ws, int tokens, int splits) {
  AttWorkspace w;
  char* p = static_cast<char*>(ws);
  w.counters = reinterpret_cast<int32_t*>(p);
  p += att_counter_bytes(tokens);
  w.m = reinterpret_cast<float*>(p);
  p += (size_t)tokens * splits * kHeads * 4;
  w.l = reinterpret_cast<float*>(p);
  p += (size_t)tokens * splits * kHeads * 4;
  w.acc = reinterpret_cast<float*>(p);
  return w;
}

// Merge the per-split partial results of one token.  Executed by the CTA that arrived last, so it
// never waits.  256 threads: thread -> (head = tid/16, 32 output columns).
__device__ void att_merge(const AttWorkspace& w, int t, int splits, __nv_bfloat16* out, float* lse,
                          int tid) {
  const int h = tid >> 4, c0 = (tid & 15) * 32;
  float mx = -INFINITY;
  for (int s = 0; s < splits; ++s) mx = fmaxf(mx, w.m[((size_t)t * splits + s) * kHeads + h]);
  float acc[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) acc[j] = 0.f;
  float lsum = 0.f;
  if (mx != -INFINITY) {
    for (int s = 0; s < splits; ++s) {
      size_t o = ((size_t)t * splits + s) * kHeads + h;
      float ms = w.m[o];
      if (ms == -INFINITY) continue;
      float f = exp2f(ms - mx);
      lsum += w.l[o] * f;
      const float4* a = reinterpret_cast<const float4*>(w.acc + o * kCkv + c0);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float4 v = a[j];
        acc[4 * j + 0] += v.x * f; acc[4 * j + 1] += v.y * f;
        acc[4 * j + 2] += v.z * f; acc[4 * j + 3] += v.w * f;
      }
    }
  }
  float inv = lsum > 0.f ? 1.f / lsum : 0.f;
  __nv_bfloat16* o = out + ((size_t)t * kHeads + h) * kCkv + c0;
#pragma unroll
  for (int j = 0; j < 32; j += 2)
    *reinterpret_cast<__nv_bfloat162*>(o + j) = __floats2bfloat162_rn(acc[j] * inv, acc[j + 1] * inv);
  if ((tid & 15) == 0) lse[(size_t)t * kHeads + h] = lsum > 0.f ? mx + log2f(lsum) : -INFINITY;
}

__global__ void __launch_bounds__(kAttThreads)
sparse_attn_simt_kernel(const __nv_bfloat16* __restrict__ q_nope, const __nv_bfloat16* __restrict__ q_pe,
                        const __nv_bfloat16* __restrict__ ckv, const __nv_bfloat16* __restrict__ kpe,
                        const int32_t* __restrict__ indices, int64_t index_stride, float scale_log2,
                        __nv_bfloat16* __restrict__ out, float* __restrict__ lse, int topk,
                        int64_t num_slots, int splits, void* ws_raw, int tokens, int32_t* status) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* qs = reinterpret_cast<float*>(smem_raw);                       // [16][576]
  __nv_bfloat16* kt = reinterpret_cast<__nv_bfloat16*>(qs + kHeads * kRowElems);  // [32][584]
  float* ps = reinterpret_cast<float*>(kt + kAttTile * kRowPad);        // [16][32]
  float* corr = ps + kHeads * kAttTile;                                 // [16]
  int* rows = reinterpret_cast<int*>(corr + kHeads);                    // [32]
  __shared__ int is_last;

  const int t = blockIdx.x, split = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int per = (topk + splits - 1) / splits;
  const int k_begin = split * per, k_end = min(topk, k_begin + per);

  for (int i = tid; i < kHeads * kRowElems; i += kAttThreads) {
    int h = i / kRowElems, d = i % kRowElems;
    qs[i] = d < kCkv ? __bfloat162float(q_nope[((size_t)t * kHeads + h) * kCkv + d])
                     : __bfloat162float(q_pe[((size_t)t * kHeads + h) * kKpe + (d - kCkv)]);
  }

  const int h0 = warp * 2;  // this warp owns heads h0, h0+1
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float acc[2][16];
#pragma unroll
  for (int j = 0; j < 16; ++j) acc[0][j] = acc[1][j] = 0.f;

  for (int k0 = k_begin; k0 < k_end; k0 += kAttTile) {
    __syncthreads();
    if (tid < kAttTile) {
      int k = k0 + tid;
      int r = k < k_end ? indices[(size_t)t * index_stride + k] : -1;
      if (r >= num_slots) { raise_status(status, DSA_STATUS_BAD_SLOT); r = -1; }
      rows[tid] = r;
    }
    __syncthreads();
    // gather 32 rows x 72 16-byte chunks (64 of ckv, 8 of kpe)
    for (int c = tid; c < kAttTile * 72; c += kAttThreads) {
      int r = c / 72, j = c % 72;
      int slot = rows[r];
      uint4 v = make_uint4(0, 0, 0, 0);
      if (slot >= 0) {
        v = j < 64 ? __ldg(reinterpret_cast<const uint4*>(ckv + (size_t)slot * kCkv) + j)
                   : __ldg(reinterpret_cast<const uint4*>(kpe + (size_t)slot * kKpe) + (j - 64));
      }
      *reinterpret_cast<uint4*>(kt + r * kRowPad + j * 8) = v;
    }
    __syncthreads();
    // logits: lane = row, warp = 2 heads
    {
      float s0 = 0.f, s1 = 0.f;
      const __nv_bfloat16* kr = kt + lane * kRowPad;
      const float* qa = qs + h0 * kRowElems;
      const float* qb = qa + kRowElems;
      for (int d = 0; d < kRowElems; d += 8) {
        uint4 raw = *reinterpret_cast<const uint4*>(kr + d);
        const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 kv = __bfloat1622float2(k2[j]);
          s0 = fmaf(kv.x, qa[d + 2 * j], s0); s0 = fmaf(kv.y, qa[d + 2 * j + 1], s0);
          s1 = fmaf(kv.x, qb[d + 2 * j], s1); s1 = fmaf(kv.y, qb[d + 2 * j + 1], s1);
        }
      }
      const bool valid = rows[lane] >= 0;
      float x[2] = {valid ? s0 * scale_log2 : -INFINITY, valid ? s1 * scale_log2 : -INFINITY};
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float mx = x[e];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float m_new = fmaxf(m_run[e], mx);
        float m_use = m_new == -INFINITY ? 0.f : m_new;
        float p = exp2f(x[e] - m_use);
        float sum = p;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        float c = exp2f(m_run[e] - m_use);  // 0 when m_run is -inf
        l_run[e] = l_run[e] * c + sum;
        m_run[e] = m_new;
        ps[(h0 + e) * kAttTile + lane] = p;
        if (lane == 0) corr[h0 + e] = c;
      }
    }
    __syncwarp();
    // PV: lane owns columns 64*j + 2*lane, +1 for j = 0..7
    {
      const float c0 = corr[h0], c1 = corr[h0 + 1];
#pragma unroll
      for (int j = 0; j < 16; ++j) { acc[0][j] *= c0; acc[1][j] *= c1; }
      for (int r = 0; r < kAttTile; ++r) {
        const float p0 = ps[h0 * kAttTile + r], p1 = ps[(h0 + 1) * kAttTile + r];
        const __nv_bfloat16* kr = kt + r * kRowPad + 2 * lane;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float2 kv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(kr + 64 * j));
          acc[0][2 * j] = fmaf(p0, kv.x, acc[0][2 * j]); acc[0][2 * j + 1] = fmaf(p0, kv.y, acc[0][2 * j + 1]);
          acc[1][2 * j] = fmaf(p1, kv.x, acc[1][2 * j]); acc[1][2 * j + 1] = fmaf(p1, kv.y, acc[1][2 * j + 1]);
        }
      }
    }
  }

  if (splits == 1) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      float inv = l_run[e] > 0.f ? 1.f / l_run[e] : 0.f;
      __nv_bfloat16* o = out + ((size_t)t * kHeads + h0 + e) * kCkv + 2 * lane;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        *reinterpret_cast<__nv_bfloat162*>(o + 64 * j) =
            __floats2bfloat162_rn(acc[e][2 * j] * inv, acc[e][2 * j + 1] * inv);
      if (lane == 0)
        lse[(size_t)t * kHeads + h0 + e] = l_run[e] > 0.f ? m_run[e] + log2f(l_run[e]) : -INFINITY;
    }
    return;
  }

  AttWorkspace w = att_carve(ws_raw, tokens, splits);
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    size_t o = ((size_t)t * splits + split) * kHeads + h0 + e;
    float* a = w.acc + o * kCkv + 2 * lane;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      *reinterpret_cast<float2*>(a + 64 * j) = make_float2(acc[e][2 * j], acc[e][2 * j + 1]);
    if (lane == 0) { w.m[o] = m_run[e]; w.l[o] = l_run[e]; }
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    int old = atomicAdd(&w.counters[t], 1);
    is_last = old == splits - 1;
    if (is_last) w.counters[t] = 0;  // ready for the next call
  }
  __syncthreads();
  if (is_last) {
    __threadfence();
    att_merge(w, t, splits, out, lse, tid);
  }
}

int att_pick_splits(int tokens, int topk) {
  int s = 1;
  while (s < 16 && tokens * s < 296 && topk / (s * 2) >= kAttTile) s *= 2;
  return s;
}

size_t att_workspace_bytes(int tokens, int splits) {
  return att_counter_bytes(tokens) + (size_t)tokens * splits * kHeads * (2 + kCkv) * 4;
}

cudaError_t launch_sparse_attn_simt(const void* q_nope, const void* q_pe, const void* ckv,
                                    const void* kpe, const int32_t* indices, int64_t index_stride,
                                    float sm_scale, void* out, float* lse, int tokens, int topk,
                                    int64_t num_slots, int splits, void* ws, int32_t* status,
                                    cudaStream_t stream) {
  size_t smem = sizeof(float) * kHeads * kRowElems + sizeof(__nv_bfloat16) * kAttTile * kRowPad +
                sizeof(float) * (kHeads * kAttTile + kHeads) + sizeof(int) * kAttTile;
  cudaError_t e = cudaFuncSetAttribute(sparse_attn_simt_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  dim3 grid(tokens, splits);
  sparse_attn_simt_kernel<<<grid, kAttThreads, smem, stream>>>(
      static_cast<const __nv_bfloat16*>(q_nope), static_cast<const __nv_bfloat16*>(q_pe),
      static_cast<const __nv_bfloat16*>(ckv), static_cast<const __nv_bfloat16*>(kpe), indices,
      index_stride, sm_scale * kLog2e, static_cast<__nv_bfloat16*>(out), lse, topk, num_slots,
      splits, ws, tokens, status);
  return cudaGetLastError();
}

}  // namespace dsa
