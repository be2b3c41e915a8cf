"""Run one kernel of the DSA path on a seeded synthetic case and print its mean device time.

    python -m auto_gpu_kernel_b200.run_case scorer    --batch 32 --context 32768 --iters 25
    python -m auto_gpu_kernel_b200.run_case select    --batch 64 --context 32768
    python -m auto_gpu_kernel_b200.run_case indexer   --batch 64 --context 32768
    python -m auto_gpu_kernel_b200.run_case attention --batch 64 --context 8192 --variant 0
    python -m auto_gpu_kernel_b200.run_case block     --batch 64 --context 32768
    python -m auto_gpu_kernel_b200.run_case prefill   --batch 4096 --context 16384
    python -m auto_gpu_kernel_b200.run_case mma-rate         (issue cost of tcgen05.mma / mma.sync shapes)

Meant for profilers (the launches of one kernel in a small process) and for quick A/B timing.
The time printed is CUDA-event time over `--iters` back-to-back launches after `--warmup` ones.
`--no-pdl` turns programmatic dependent launch off so that per-kernel durations reported by a
profiler do not include the time a dependent kernel spends waiting for its predecessor.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def measure_mma_rate(dev, kind, m, n, iters=2880):
    """(issue cycles, completion cycles) per instruction of `dsa_selftest_mma_rate` (see the header)."""
    import torch
    from . import _lib, workspace
    lib = _lib.load()
    cycles = torch.zeros(2, dtype=torch.int64, device=dev)
    sink = torch.zeros(1, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = lib.dsa_selftest_mma_rate(kind, m, n, iters, cycles.data_ptr(), sink.data_ptr(),
                                       workspace.status_word(dev).data_ptr(),
                                       torch.cuda.current_stream(dev).cuda_stream)
    _lib.check(rc, "dsa_selftest_mma_rate")
    torch.cuda.synchronize(dev)
    workspace.check_status(dev)
    per = iters * (8 * m if kind == 2 else 1)      # mma.sync: 8 per warp and iteration, m warps
    return cycles[0].item() / per, cycles[1].item() / per


def mma_rate(dev) -> int:
    """Cost of one tensor-core instruction, per SM: tcgen05.mma (one issuing thread) for the shapes
    the kernels use or could use, and mma.sync m16n8k16 issued from 4 / 8 / 16 warps."""
    rows = []
    for kind, name in ((0, "tcgen05 bf16"), (1, "tcgen05 e4m3")):
        for m in (64, 128):
            for n in (16, 64, 128, 256):
                issue, done = measure_mma_rate(dev, kind, m, n)
                rows.append({"instr": name, "m": m, "n": n, "issue_cycles": round(issue, 1),
                             "complete_cycles": round(done, 1)})
    for warps in (4, 8, 16):
        _, done = measure_mma_rate(dev, 2, warps, 0, iters=2000)
        rows.append({"instr": "mma.sync m16n8k16 bf16", "warps": warps, "cycles_per_instr_per_sm": round(done, 2),
                     "mac_per_clk_per_sm": round(2048 / done)})
    for r in rows:
        print(json.dumps(r))
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("case", choices=["scorer", "select", "indexer", "attention", "block", "prefill", "mma-rate"])
    ap.add_argument("--batch", type=int, default=64, help="requests (= query tokens)")
    ap.add_argument("--context", type=int, default=32768, help="tokens per request")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--variant", type=int, default=0,
                    help="scorer/prefill: 0 tcgen05, 1 CUDA-core, 2 streaming tcgen05 kernel; "
                         "attention: 0 mma.sync, 1 CUDA-core, 2 tcgen05")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-pdl", action="store_true")
    args = ap.parse_args(argv)
    if args.no_pdl:
        os.environ["DSA_PDL"] = "0"   # read once by the library, before its first launch

    import torch
    from . import indexer, sparse_attention, workspace, inputs as wl

    if not torch.cuda.is_available():
        print("run_case: no CUDA device", file=sys.stderr)
        return 2
    dev = torch.device("cuda", 0)
    if args.case == "mma-rate":
        return mma_rate(dev)
    lens = [args.context] * args.batch

    if args.case in ("scorer", "select", "indexer"):
        inp = wl.make_indexer_inputs(lens, seed=args.seed, device=dev)
        a = inp.args()
        if args.case == "scorer":
            out = indexer.scores(*a, variant=args.variant)
            fn = lambda: indexer.scores(*a, variant=args.variant, out=out)
        elif args.case == "select":
            rows = indexer.scores(*a, variant=0)
            topk = torch.empty(args.batch, indexer.TOPK, dtype=torch.int32, device=dev)
            fn = lambda: indexer.select(rows, inp.seq_lens, inp.block_table, topk)
        else:
            topk = torch.empty(args.batch, indexer.TOPK, dtype=torch.int32, device=dev)
            fn = lambda: indexer.kernel(*a, topk)
        moved = inp.k_index_cache_fp8.numel()
    elif args.case == "prefill":
        # chunked prefill: `batch` query rows after a prefix of `context` tokens, all rows reading
        # the same pages (block_table row stride 0); row i sees context + i + 1 tokens
        inp = wl.make_shared_prefix_indexer_inputs(args.context, args.batch, seed=args.seed, device=dev)
        shared = inp.block_table[:1].expand(args.batch, -1)
        a = (inp.q_index_fp8, inp.k_index_cache_fp8, inp.weights, inp.seq_lens, shared)
        out = indexer.scores(*a, variant=args.variant)
        fn = lambda: indexer.scores(*a, variant=args.variant, out=out)
        moved = int(inp.seq_lens.sum()) * 2 * 64 * 128   # flops, reported in the gb_per_s field as GFLOP/s
    elif args.case == "attention":
        inp = wl.make_attention_inputs(lens, seed=args.seed, device=dev)
        out = torch.empty_like(inp.q_nope)
        lse = torch.empty(inp.q_nope.shape[:2], dtype=torch.float32, device=dev)
        fn = lambda: sparse_attention.kernel(*inp.args(), out, lse, variant=args.variant)
        moved = int((inp.sparse_indices >= 0).sum()) * 1152
    else:
        blk = wl.make_decode_block_inputs(lens, seed=args.seed, device=dev)
        a = blk.indexer.args()
        topk = torch.empty(args.batch, indexer.TOPK, dtype=torch.int32, device=dev)
        out = torch.empty_like(blk.q_nope)
        lse = torch.empty(blk.q_nope.shape[:2], dtype=torch.float32, device=dev)

        def fn():
            indexer.kernel(*a, topk)
            sparse_attention.kernel(blk.q_nope, blk.q_pe, blk.ckv_cache, blk.kpe_cache, topk,
                                    blk.sm_scale, out, lse)
        moved = blk.indexer.k_index_cache_fp8.numel() + args.batch * min(args.context, 2048) * 1152

    for _ in range(max(args.warmup, 1)):
        fn()
    torch.cuda.synchronize(dev)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.iters):
        fn()
    t1.record()
    torch.cuda.synchronize(dev)
    status = workspace.check_status(dev)
    us = t0.elapsed_time(t1) * 1e3 / args.iters
    print(json.dumps({"case": args.case, "batch": args.batch, "context": args.context,
                      "variant": args.variant, "iters": args.iters, "us_per_iter": round(us, 2),
                      "key_or_row_bytes": moved, "gb_per_s": round(moved / us / 1e3, 1),
                      "pdl": not args.no_pdl, "status": status}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
