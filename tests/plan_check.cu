// Host-only check of the attention work split (attn_plan.cuh): prints one line per violated
// invariant and exits non-zero if any.  Built and run by tests/test_attn_plan.py; no GPU needed.
#include <cstdio>

#include "../auto_gpu_kernel_b200/csrc/attn_plan.cuh"

int main() {
  int bad = 0, cases = 0;
  const int sms_list[] = {1, 4, 132, 148, 160};
  const int topk_list[] = {1, 63, 64, 65, 512, 2048, 4096, 8192};
  for (int sms : sms_list)
    for (int topk : topk_list)
      for (int tokens = 1; tokens <= 1200; tokens += (tokens < 160 ? 1 : 37)) {
        ++cases;
        const dsa::AtPlan p = dsa::at_make_plan(tokens, topk, sms);
        const long total = (long)tokens * p.tiles_per_token;
        auto fail = [&](const char* what) {
          ++bad;
          printf("T=%d topk=%d sms=%d: %s (grid %d per_cta %d segs_max %d)\n", tokens, topk, sms, what,
                 p.grid, p.per_cta, p.segs_max);
        };
        if (p.tiles_per_token != (topk + 63) / 64) fail("tiles per token");
        if (p.grid < 1 || p.per_cta < 1) fail("empty plan");
        if ((long)p.grid * p.per_cta < total) fail("ranges do not cover all tiles");
        if ((long)(p.grid - 1) * p.per_cta >= total) fail("a CTA without tiles");
        if (p.segs_max < 1 || p.segs_max > 32) fail("segment slots out of range");
        // the largest number of CTA ranges that any token's tiles fall into
        int worst = 1;
        for (long t = 0; t < tokens; ++t) {
          const long first = t * p.tiles_per_token, last = first + p.tiles_per_token - 1;
          const int segs = (int)(last / p.per_cta - first / p.per_cta) + 1;
          if (segs > worst) worst = segs;
        }
        if (worst > p.segs_max) fail("a token is cut into more segments than there are slots");
        if (dsa::at_tc_workspace_bytes(tokens, topk, sms) <
            dsa::at_counter_bytes(tokens) + (size_t)tokens * worst * dsa::kHeads * (2 + dsa::kCkv) * 4)
          fail("workspace smaller than the partials need");
      }
  printf("%d cases, %d violations\n", cases, bad);
  return bad ? 1 : 0;
}
