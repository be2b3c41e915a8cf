// Work split shared by the sparse-attention kernels: the (token, 64-row tile) sequence is cut into
// equal contiguous ranges, one per CTA; a token covered by several CTAs ("segments") leaves one
// partial result per segment in the caller's workspace and is merged by the last arriver.
#pragma once

#include "common.cuh"

namespace dsa {

constexpr int kAtTile = 64;

struct AtPlan {
  int tiles_per_token;  // ceil(topk / 64)
  int per_cta;          // tiles per CTA range
  int grid;
  int segs_max;         // partial slots per token in the workspace
};

struct AtPartials {
  int32_t* counters;  // [tokens], zero between calls
  float* m;           // [tokens][segs_max][16]
  float* l;           // [tokens][segs_max][16]
  float* acc;         // [tokens][segs_max][16][512]
};

__host__ __device__ inline size_t at_counter_bytes(int tokens) {
  return attn_counter_region_bytes(tokens);
}
__host__ __device__ inline AtPartials at_carve(void* ws, int tokens, int segs_max) {
  AtPartials w;
  char* p = static_cast<char*>(ws);
  w.counters = reinterpret_cast<int32_t*>(p);
  p += at_counter_bytes(tokens);
  w.m = reinterpret_cast<float*>(p);
  p += (size_t)tokens * segs_max * kHeads * 4;
  w.l = reinterpret_cast<float*>(p);
  p += (size_t)tokens * segs_max * kHeads * 4;
  w.acc = reinterpret_cast<float*>(p);
  return w;
}

// (A split that gives ranges containing a token start fewer tiles was measured equal to this
// uniform one -- 40.5-42 us against 41.7 us at 64 tokens -- and is not kept: what the boundary
// CTAs lose is barrier and round-trip latency, which the cluster-per-token split removes.)
inline AtPlan at_make_plan(int tokens, int topk, int sms) {
  AtPlan p;
  p.tiles_per_token = (topk + kAtTile - 1) / kAtTile;
  const long total = (long)tokens * p.tiles_per_token;
  p.grid = (int)(total < sms ? total : sms);
  if (p.grid < 1) p.grid = 1;
  if (tokens >= 4 * p.grid) {  // whole tokens per CTA: no partial results at all
    p.per_cta = p.tiles_per_token * ((tokens + p.grid - 1) / p.grid);
    p.segs_max = 1;
  } else {
    p.per_cta = (int)((total + p.grid - 1) / p.grid);
    // a token may be cut into at most 32 segments
    const int min_per = p.tiles_per_token <= 32 ? 1 : (p.tiles_per_token + 30) / 31;
    if (p.per_cta < min_per) p.per_cta = min_per;
    int s = (p.tiles_per_token + p.per_cta - 1) / p.per_cta + 1;
    p.segs_max = s < p.tiles_per_token ? s : p.tiles_per_token;
    if (p.segs_max > 32) p.segs_max = 32;
  }
  p.grid = (int)((total + p.per_cta - 1) / p.per_cta);
  return p;
}

inline size_t at_tc_workspace_bytes(int tokens, int topk, int sms) {
  AtPlan p = at_make_plan(tokens, topk, sms);
  return at_counter_bytes(tokens) + (size_t)tokens * p.segs_max * kHeads * (2 + kCkv) * 4;
}

}  // namespace dsa
