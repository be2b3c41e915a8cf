#!/usr/bin/env python
"""Benchmark of the DSA decode block (FP8 top-k indexer -> sparse MLA attention) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One "step" = one call of the indexer followed by one call of sparse attention over the indices it
produced, on the headline decode point: B = 64 requests per GPU, context 32768, page size
64, top-k 2048.  With N > 1 (torchrun, one rank per GPU) requests are sharded: every rank owns its
own 64 requests and their cache pages, there is no data-path collective, and the reported time is
the maximum over ranks (weak scaling).  Prints ONE JSON line on rank 0.

`--impl reference` times the CPU restatement of the reference's PyTorch definitions (oracle/) on
the host cores instead, on a stated sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

BATCH = 64
CONTEXT = 32768
TOPK = 2048
SCORER_DRAM_BYTES_PER_TOKEN = (138860544 + 1302784) / (32 * 32768)
METRIC = "us/call: DSA indexer + sparse attn, decode B=64 ctx 32K"
WORKLOAD = "dsa_decode_block B=64/GPU ctx=32768 ps=64 topk=2048 (indexer 64h fp8 -> sparse MLA 16h bf16)"


# ------------------------------------------------------------------------------ algorithmic work
def indexer_bytes(lens):
    """132 B per cached token + block_table + q + w + seq_len + index row out, per request."""
    return sum(132 * n + 4 * ((n + 63) // 64) + 8192 + 256 + 4 + 8192 for n in lens)


def attention_bytes(tokens, valid=TOPK):
    """1152 B per selected row + q (18432) + indices (8192) + out (16384) + lse (64), per token."""
    return tokens * (valid * 1152 + 18432 + 8192 + 16384 + 64)


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        peaks = json.loads(path.read_text())
        return float(peaks["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ------------------------------------------------------------------------------ clocks sampling
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        top = sorted(sm)[len(sm) // 2:]           # samples under load (idle gaps read lower)
        return {"sm_mhz": statistics.median(top), "sm_max_mhz": max(mx), "samples": len(sm),
                "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------ CPU legs
def cpu_reference_step(block, requests):
    """One pass of the oracle (CPU restatement of the reference) over `requests` requests."""
    sys.path.insert(0, str(ROOT / "oracle"))
    import dsa_oracle as oracle
    idx = block.indexer
    sel = slice(0, requests)
    topk = oracle.indexer_topk(idx.q_index_fp8[sel], idx.k_index_cache_fp8, idx.weights[sel],
                               idx.seq_lens[sel], idx.block_table[sel])
    oracle.sparse_attention(block.q_nope[sel], block.q_pe[sel], block.ckv_cache, block.kpe_cache,
                            topk, block.sm_scale)


def time_cpu(block_cpu, requests, steps, warmup):
    torch.set_num_threads(os.cpu_count() or 1)
    for _ in range(warmup):
        cpu_reference_step(block_cpu, requests)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        cpu_reference_step(block_cpu, requests)
        times.append(time.perf_counter() - t0)
    return statistics.median(times)


def block_to_cpu(block):
    from auto_gpu_kernel_b200 import inputs as wl
    return wl.DecodeBlockInputs(block.indexer.to("cpu"), block.q_nope.cpu(), block.q_pe.cpu(),
                                block.ckv_cache.cpu(), block.kpe_cache.cpu(), block.sm_scale)


# ------------------------------------------------------------------------------ head-sharded block
def run_head_sharded(args, rank, world, dev):
    """The full-block layout: B = 128 requests, ctx uniform in [16K, 64K]; the indexer is
    request-sharded, its int32 [B, 2048] index rows are all-gathered (NCCL), attention runs for all
    tokens on every rank for that rank's 16 heads over replicated ckv/kpe caches."""
    import torch.distributed as dist
    from auto_gpu_kernel_b200 import dist as dsa_dist, inputs as wl, workspace
    batch = 128
    lens = wl.uniform_lengths(batch, 16384, 65536, seed=0)
    block = wl.make_decode_block_inputs(lens, seed=0, device=dev)      # identical on every rank
    idx = block.indexer
    gen = torch.Generator(device=dev).manual_seed(100 + rank)           # this rank's 16 heads
    q_nope = (torch.randn(batch, 16, 512, generator=gen, device=dev) * 0.1).to(torch.bfloat16)
    q_pe = (torch.randn(batch, 16, 64, generator=gen, device=dev) * 0.1).to(torch.bfloat16)
    mine = dsa_dist.shard_range(batch, rank, world)
    counts = [len(dsa_dist.shard_range(batch, r, world)) for r in range(world)]
    sel = slice(mine.start, mine.stop)
    local_args = (idx.q_index_fp8[sel].contiguous(), idx.k_index_cache_fp8, idx.weights[sel].contiguous(),
                  idx.seq_lens[sel].contiguous(), idx.block_table[sel].contiguous())
    local_idx = torch.empty(len(mine), TOPK, dtype=torch.int32, device=dev)
    out = torch.empty(batch, 16, 512, dtype=torch.bfloat16, device=dev)
    lse = torch.empty(batch, 16, dtype=torch.float32, device=dev)

    def step():
        dsa_dist.decode_block_head_sharded(local_args, counts, q_nope, q_pe, block.ckv_cache,
                                           block.kpe_cache, block.sm_scale, out, lse,
                                           local_indices=local_idx)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    workspace.check_status(dev)
    sampler = ClockSampler(dev.index)
    barrier()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    t_load = time.perf_counter()
    while time.perf_counter() - t_load < 1.2:
        for _ in range(10):
            step()
        torch.cuda.synchronize()
    clocks = sampler.stop()
    clocks["window"] = "timed steps, then the same steps repeated for 1.2 s"
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        us = t.item() / args.steps * 1e3
        my_tokens = sum(lens[i] for i in mine)
        line = {"metric": "us/layer: full DSA block, 128 heads = 16/GPU, decode B=128 ctx 16-64K",
                "value": us, "unit": "us", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": us / 1e3, "higher_is_better": False, "scaling": "strong",
                "vs_baseline": None, "dtype": "fp8(e4m3)+bf16, fp32 accumulate", "data": "synthetic",
                "config": {"workload": "dsa_full_block B=128 ctx~U[16K,64K] heads=16/GPU",
                           "indexer": f"request-sharded, {len(mine)} requests / {my_tokens} cached tokens on rank 0",
                           "collective": "all_gather int32 [128,2048] (1 MiB)" if world > 1 else "none (1 GPU)",
                           "attention": "head-sharded, all 128 tokens per rank, caches replicated"},
                "impl": "b200", "gpu_launches": 3 * args.steps, "clocks": clocks}
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


# ------------------------------------------------------------------------------ main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--layout", default="requests", choices=["requests", "heads"],
                    help="requests: every rank owns its requests, no collective (default, the headline "
                         "metric); heads: the full 128-head block -- indexer request-sharded, "
                         "all-gather of the index rows, attention head-sharded")
    ap.add_argument("--batch", type=int, default=BATCH, help=argparse.SUPPRESS)
    ap.add_argument("--context", type=int, default=CONTEXT, help=argparse.SUPPRESS)
    ap.add_argument("--cpu-requests", type=int, default=16, help=argparse.SUPPRESS)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    from auto_gpu_kernel_b200 import inputs as wl

    lens = [args.context] * args.batch
    config = {"workload": WORKLOAD, "batch_per_gpu": args.batch, "context": args.context,
              "page_size": 64, "topk": TOPK, "sharding": "requests (no collective)",
              "l2": "inputs exceed L2: 278 MB key cache streamed + 151 MB gathered from a 2.4 GB cache per step"}

    if args.impl == "reference":
        if rank != 0:
            return 0
        n_req = min(args.cpu_requests, args.batch)
        block = wl.make_decode_block_inputs(lens[:n_req], seed=0, device="cpu")
        sec = time_cpu(block, n_req, max(1, args.steps), args.warmup)
        us = sec * 1e6 * (args.batch / n_req)
        cores = os.cpu_count() or 1
        sample = (f"{n_req} of {args.batch} requests per step (indexer + attention), time scaled x"
                  f"{args.batch / n_req:g}; median of {max(1, args.steps)} steps")
        line = {"metric": METRIC, "value": us, "unit": "us", "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": us / 1e3,
                "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": config, "impl": "reference",
                "cpu_baseline": {"value": us, "unit": "us", "cores": cores, "kind": "port",
                                 "sample": sample},
                "e2e": {"value": us, "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line))
        return 0

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (the b200 arm has no CPU path)")
    from auto_gpu_kernel_b200 import indexer, sparse_attention, workspace
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    if args.layout == "heads":
        return run_head_sharded(args, rank, world, dev)

    block = wl.make_decode_block_inputs(lens, seed=rank, device=dev)
    idx = block.indexer
    topk = torch.empty(args.batch, TOPK, dtype=torch.int32, device=dev)
    out = torch.empty(args.batch, 16, 512, dtype=torch.bfloat16, device=dev)
    lse = torch.empty(args.batch, 16, dtype=torch.float32, device=dev)
    score_buf = torch.empty(args.batch, (idx.block_table.shape[1] * 64 + 127) // 128 * 128,
                            dtype=torch.float32, device=dev)

    def step():
        indexer.kernel(*idx.args(), topk)
        sparse_attention.kernel(block.q_nope, block.q_pe, block.ckv_cache, block.kpe_cache, topk,
                                block.sm_scale, out, lse)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def ev():
        return torch.cuda.Event(enable_timing=True)

    for _ in range(args.warmup):
        step()
    workspace.check_status(dev)

    # ---- timed region: exactly K steps between two events on the launching stream ----------------
    # (no event inside a step: the three kernels of a step are chained by programmatic dependent
    #  launch and an event record between them would serialise them)
    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    t_begin, t_end = ev(), ev()
    barrier()
    t_begin.record()
    for _ in range(args.steps):
        step()
    t_end.record()
    barrier()
    total_ms = t_begin.elapsed_time(t_end)
    # the timed region lasts a few milliseconds, far less than nvidia-smi's sampling period: keep
    # the very same steps running for 1.2 s so that the clock samples are taken under this load
    t_load = time.perf_counter()
    while time.perf_counter() - t_load < 1.2:
        for _ in range(20):
            step()
        torch.cuda.synchronize()
    clocks = sampler.stop()
    clocks["window"] = "timed steps, then the same steps repeated for 1.2 s"
    workspace.check_status(dev)

    # ---- per-stage times: the same K steps with an event between the two operator calls ----------
    marks = [(ev(), ev(), ev()) for _ in range(args.steps)]
    torch.cuda.synchronize()
    for a, b, c in marks:
        a.record()
        indexer.kernel(*idx.args(), topk)
        b.record()
        sparse_attention.kernel(block.q_nope, block.q_pe, block.ckv_cache, block.kpe_cache, topk,
                                block.sm_scale, out, lse)
        c.record()
    torch.cuda.synchronize()
    idx_us = statistics.mean(a.elapsed_time(b) for a, b, _ in marks) * 1e3
    att_us = statistics.mean(b.elapsed_time(c) for _, b, c in marks) * 1e3

    # ---- dominant kernel alone (indexer scorer), same inputs, K launches -------------------------
    for _ in range(3):
        indexer.scores(*idx.args(), variant=0, out=score_buf)
    torch.cuda.synchronize()
    k0, k1 = ev(), ev()
    k0.record()
    for _ in range(args.steps):
        indexer.scores(*idx.args(), variant=0, out=score_buf)
    k1.record()
    torch.cuda.synchronize()
    score_us = k0.elapsed_time(k1) / args.steps * 1e3

    # ---- end to end through the public operators with host buffers -------------------------------
    # HostDecodeStep owns pinned input/result slabs; the caller's per-step tensors are written into
    # its pinned views (here once: the same synthetic step is repeated) and every run() copies
    # them to the device, runs both operators and copies indices, output and LSE back.
    from auto_gpu_kernel_b200.host_step import HostDecodeStep
    host = HostDecodeStep(idx.k_index_cache_fp8, block.ckv_cache, block.kpe_cache, args.batch,
                          idx.block_table.shape[1], block.sm_scale)
    host.inputs.q_index_fp8.copy_(idx.q_index_fp8.view(torch.uint8))
    host.inputs.weights.copy_(idx.weights)
    host.inputs.seq_lens.copy_(idx.seq_lens)
    host.inputs.block_table.copy_(idx.block_table)
    host.inputs.q_nope.copy_(block.q_nope)
    host.inputs.q_pe.copy_(block.q_pe)
    torch.cuda.synchronize()
    h2d, d2h = host.h2d_bytes, host.d2h_bytes

    def e2e_step():
        host.run()   # synchronises: the caller reads the result every step

    for _ in range(3):
        e2e_step()
    barrier()
    e0, e1 = ev(), ev()
    e0.record()
    for _ in range(args.steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)

    times = torch.tensor([total_ms, e2e_ms, idx_us, att_us, score_us], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms, idx_us, att_us, score_us = times.tolist()

    line = None
    if rank == 0:
        peak, peak_kind = measured_peaks()
        us = total_ms / args.steps * 1e3
        algo = indexer_bytes(lens)
        achieved = algo / (score_us * 1e-6) / 1e9
        att_algo = attention_bytes(args.batch)
        line = {
            "metric": METRIC, "value": us, "unit": "us", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": us / 1e3, "higher_is_better": False,
            "scaling": "weak", "vs_baseline": None, "dtype": "fp8(e4m3)+bf16, fp32 accumulate",
            "data": "synthetic", "config": config, "impl": "b200",
            "stages": {"indexer_us": idx_us, "sparse_attention_us": att_us,
                       "attention_hbm_gbs": att_algo / (att_us * 1e-6) / 1e9,
                       "attention_frac_of_peak": att_algo / (att_us * 1e-6) / 1e9 / peak},
            "roofline": {"kernel": "indexer_score_tc_kernel", "bound": "hbm", "achieved": achieved,
                         "peak": peak, "peak_source": f"{peak_kind} copy bandwidth", "unit": "GB/s",
                         "frac": achieved / peak, "us_per_launch": score_us,
                         "algorithmic_bytes": algo, "traffic": None},
            "e2e": {"value": e2e_ms / args.steps * 1e3, "unit": "us", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h,
                    "note": "HostDecodeStep.run(): per-step inputs (q, weights, seq_lens, block_table, q_nope, "
                            "q_pe) from pinned host memory, results (indices, output, lse) read back; the paged "
                            "caches are device-resident state"},
            "gpu_launches": 3 * args.steps,
            "clocks": clocks,
        }
        # DRAM traffic of the scorer from one ncu capture (profiles/indexer_score_tc_B32_ctx32K.md):
        # 138.87 MB read + 1.69 MB written for 32 x 32768 cached tokens; it grows with the tokens
        # streamed, so it is scaled to this launch by the token count.
        line["roofline"]["traffic"] = SCORER_DRAM_BYTES_PER_TOKEN * sum(lens)
        if world == 1:
            n_req = min(args.cpu_requests, args.batch)
            cpu_block = wl.make_decode_block_inputs(lens[:n_req], seed=0, device="cpu")
            sec = time_cpu(cpu_block, n_req, steps=3, warmup=1)
            line["cpu_baseline"] = {
                "value": sec * 1e6 * (args.batch / n_req), "unit": "us", "cores": os.cpu_count() or 1,
                "kind": "port",
                "sample": f"{n_req} of {args.batch} requests (indexer + attention), time scaled x"
                          f"{args.batch / n_req:g}; median of 3 steps"}
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
