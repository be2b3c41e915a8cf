// Work split shared by the sparse-attention kernels: the (token, 64-row tile) sequence is cut into
// equal contiguous ranges, one per CTA; a token covered by several CTAs ("segments") leaves one
// partial result per segment in the caller's workspace and is merged by the last arriver.
#pragma once

#include "common.cuh"

namespace dsa {

constexpr int kAtTile = 64;

constexpr int kAtMaxGrid = 192;

struct AtPlan {
  int tiles_per_token;  // ceil(topk / 64)
  int per_cta;          // tiles per CTA range (uniform split)
  int grid;
  int segs_max;         // partial slots per token in the workspace
  // Cost-balanced split (used by the mma.sync kernel when `balanced` is set): CTA c owns the tiles
  // [starts[c], starts[c+1]).  Starting a token inside a range costs about one tile (its q has to be
  // staged and the pipeline drains), so ranges that contain a token start get one tile less.
  int balanced;
  int starts[kAtMaxGrid + 1];
};

// CTA that owns tile `w` under the balanced split (largest c with starts[c] <= w).
__host__ __device__ inline int at_owner(const AtPlan& p, long w) {
  int lo = 0, hi = p.grid;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (p.starts[mid] <= w) lo = mid; else hi = mid;
  }
  return lo;
}

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

inline AtPlan at_make_plan(int tokens, int topk, int sms, double start_cost = 1.0) {
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
    // a token may be cut into at most 32 segments (size of the merge scratch in shared memory)
    const int min_per = p.tiles_per_token <= 32 ? 1 : (p.tiles_per_token + 30) / 31;
    if (p.per_cta < min_per) p.per_cta = min_per;
    int s = (p.tiles_per_token + p.per_cta - 1) / p.per_cta + 1;
    p.segs_max = s < p.tiles_per_token ? s : p.tiles_per_token;
    if (p.segs_max > 32) p.segs_max = 32;
  }
  p.grid = (int)((total + p.per_cta - 1) / p.per_cta);
  p.balanced = 0;
  if (p.segs_max > 1 && p.grid <= kAtMaxGrid && p.per_cta >= 4) {
    // cost of a token = its tiles + 1 (the token start); cut the cost axis into `grid` equal parts
    const int tpt = p.tiles_per_token;
    const double token_cost = tpt + start_cost, budget = tokens * token_cost / p.grid;
    int worst = 1, segs_of_token = 0;
    long prev_token = -1;
    p.starts[0] = 0;
    for (int c = 1; c < p.grid; ++c) {
      const double x = budget * c;
      const long t = (long)(x / token_cost);
      const double rem = x - t * token_cost;
      long w = t * tpt + (rem <= start_cost ? 0 : (long)(rem - start_cost + 0.999999));
      if (w <= p.starts[c - 1]) w = p.starts[c - 1] + 1;
      if (w > total - (p.grid - c)) w = total - (p.grid - c);
      p.starts[c] = (int)w;
    }
    p.starts[p.grid] = (int)total;
    for (int c = 0; c < p.grid; ++c) {   // segments per token: count the CTAs that touch each token
      const long t_first = p.starts[c] / tpt, t_last = ((long)p.starts[c + 1] - 1) / tpt;
      for (long t = t_first; t <= t_last; ++t) {
        segs_of_token = (t == prev_token) ? segs_of_token + 1 : 1;
        prev_token = t;
        if (segs_of_token > worst) worst = segs_of_token;
      }
    }
    if (worst <= 32) {
      p.balanced = 1;
      if (worst > p.segs_max) p.segs_max = worst;
    }
  }
  return p;
}

inline size_t at_tc_workspace_bytes(int tokens, int topk, int sms) {
  AtPlan p = at_make_plan(tokens, topk, sms);
  return at_counter_bytes(tokens) + (size_t)tokens * p.segs_max * kHeads * (2 + kCkv) * 4;
}

}  // namespace dsa
