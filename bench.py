#!/usr/bin/env python
"""Benchmark of the DSA hot path (FP8 top-k indexer -> sparse MLA attention) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
                    [--workload headline|cfg1|cfg2|cfg3|cfg4] [--compare]

Workloads (one JSON line each, same schema; the default is the headline):
  headline  one decode step = indexer call + attention call over the indexer's own indices,
            B = 64 requests per GPU, context 32768, page size 64, top-k 2048.  With N > 1 every
            rank owns its own 64 requests and cache pages (weak scaling, no data-path collective);
            the line then also carries, under `stages`, the head-sharded full block (cfg4) with
            its all-gather and a cfg2 shard, timed with the same protocol.
  cfg1      sparse attention alone, T = 64 tokens, contexts uniform in [8K, 32K].
  cfg2      indexer alone, B = 256 requests, contexts uniform in [32K, 128K], requests sharded
            over the N GPUs (strong scaling).
  cfg3      chunked prefill: 16K prefix + 4096-token chunk, indexer + attention, query tokens
            sharded over the N GPUs.
  cfg4      the full 128-head block: B = 128, contexts uniform in [16K, 64K]; indexer
            request-sharded, one all-gather of the int32 [128, 2048] index rows, attention
            head-sharded (16 heads per GPU) over replicated caches.

Timing: W >= 3 warm-up steps, then exactly K steps between two CUDA events on the launching
stream, bracketed by a barrier + synchronize, maximum over ranks.  Inputs are larger than L2.

`--impl reference` times the reference's own PyTorch definitions (baseline/_ref, copied there by
baseline/fetch_reference.py; kind "reference") on the host cores, or the CPU restatement in
oracle/ when those files are absent (kind "port"), on a stated sample of the same workload.
`--compare` (1 GPU) adds a `comparators` object: the reference's Gluon/Triton GPU kernels from
baseline/_ref timed beside this library's on the same inputs (spin-free dispatches only).
"""
from __future__ import annotations

import argparse
import importlib.util
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
REF_DIR = ROOT / "baseline" / "_ref"

BATCH = 64
CONTEXT = 32768
TOPK = 2048
# DRAM bytes per cached token of the scorer, from one ncu capture of 32 x 32768 tokens
# (138.87 MB read + 1.30 MB written); traffic grows with the tokens streamed.
SCORER_DRAM_BYTES_PER_TOKEN = (138860544 + 1302784) / (32 * 32768)
DTYPE = "fp8(e4m3)+bf16, fp32 accumulate"


# ------------------------------------------------------------------------------ algorithmic work
def indexer_bytes(lens):
    """132 B per cached token + block_table + q + w + seq_len + index row out, per request."""
    return sum(132 * n + 4 * ((n + 63) // 64) + 8192 + 256 + 4 + 8192 for n in lens)


def attention_bytes(tokens, valid=TOPK):
    """1152 B per selected row + q (18432) + indices (8192) + out (16384) + lse (64), per token."""
    return tokens * (valid * 1152 + 18432 + 8192 + 16384 + 64)


def measured_peaks():
    """(HBM GB/s, dense bf16 TFLOP/s, source)."""
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        peaks = json.loads(path.read_text())
        return float(peaks["hbm_gbs"]), float(peaks["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


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


# ------------------------------------------------------------------------------ timing protocol
class Ranks:
    """Rank bookkeeping + the barrier that brackets every timed region."""

    def __init__(self):
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.dev = None

    def init(self):
        import torch.distributed as dist
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1 and not dist.is_initialized():
            dist.init_process_group("nccl", device_id=self.dev)

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, values):
        t = torch.tensor(list(values), dtype=torch.float64, device=self.dev)
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    def finish(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
            dist.destroy_process_group()


def ev():
    return torch.cuda.Event(enable_timing=True)


def timed_us(step, steps, warmup, ranks, sampler=None):
    """Mean microseconds per step: W warm-ups, then exactly K steps between two events.

    The K steps of a decode workload last a millisecond or two, so a host hiccup (another rank's
    process start, the clock sampler's) would otherwise show up as device time.  Two precautions:
    the sampler is started -- and given time to come up -- before the warm-up, and the first event
    is recorded behind a short device-side delay, during which the host has already queued the K
    steps: the device then runs them back to back, as a serving loop that runs ahead of the GPU does."""
    if sampler is not None:
        sampler.start()
        time.sleep(0.4)
    for _ in range(max(warmup, 3)):
        step()
    ranks.barrier()
    e0, e1 = ev(), ev()
    ranks.barrier()
    torch.cuda._sleep(int(min(4.0e-3, max(1.0e-3, steps * 6.0e-5)) * 1.9e9))   # 1-4 ms of device time
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    ranks.barrier()
    return e0.elapsed_time(e1) * 1e3 / steps


def sample_clocks(step, sampler, batches=None):
    """The timed region lasts milliseconds, less than nvidia-smi's sampling period: keep the very
    same steps running for 1.2 s so that the clock samples are taken under this load.  A step that
    holds an exchange between ranks is repeated `batches` x 20 times instead, the same count on
    every rank."""
    t0 = time.perf_counter()
    done = 0
    while (time.perf_counter() - t0 < 1.2) if batches is None else (done < batches):
        for _ in range(20):
            step()
        torch.cuda.synchronize()
        done += 1
    clocks = sampler.stop()
    clocks["window"] = "timed steps, then the same steps repeated for 1.2 s"
    return clocks


def e2e_us(host_tensors, dev_tensors, run, results, steps, ranks):
    """The same step through the public operators with HOST buffers: every step copies the per-step
    inputs from pinned memory, runs, copies the results back to pinned memory and synchronises."""
    pinned_in = [t.cpu().pin_memory() for t in host_tensors]
    pinned_out = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in results]

    def step():
        for src, dst in zip(pinned_in, dev_tensors):
            dst.copy_(src, non_blocking=True)
        run()
        for src, dst in zip(results, pinned_out):
            dst.copy_(src, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    us = timed_us(step, steps, 3, ranks)
    h2d = sum(t.numel() * t.element_size() for t in pinned_in)
    d2h = sum(t.numel() * t.element_size() for t in pinned_out)
    return us, h2d, d2h


# ------------------------------------------------------------------------------ CPU legs
def load_reference():
    """(indexer_kernel, attention_kernel, kind): the reference's own definitions when present."""
    def from_path(name):
        spec = importlib.util.spec_from_file_location(f"dsa_ref_{name}", REF_DIR / f"{name}.py")
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod.kernel

    if (REF_DIR / "indexer_baseline.py").exists() and (REF_DIR / "sparse_baseline.py").exists():
        return from_path("indexer_baseline"), from_path("sparse_baseline"), "reference"
    sys.path.insert(0, str(ROOT / "oracle"))
    import dsa_oracle as oracle

    def idx_kernel(q, cache, w, lens, table, out):
        out.copy_(oracle.indexer_topk(q, cache, w, lens, table))

    def att_kernel(qn, qp, ckv, kpe, idx, scale, out, lse):
        o, l = oracle.sparse_attention(qn, qp, ckv, kpe, idx, scale)
        out.copy_(o); lse.copy_(l)

    return idx_kernel, att_kernel, "port"


def cpu_step_seconds(indexer_args, attention_args, steps, warmup):
    """Median seconds of one CPU pass: indexer (if given) then attention (if given; when both are
    given the attention reads the indexer's indices)."""
    idx_kernel, att_kernel, kind = load_reference()
    torch.set_num_threads(os.cpu_count() or 1)
    topk = None
    if indexer_args is not None:
        topk = torch.empty(indexer_args[0].shape[0], TOPK, dtype=torch.int32)

    def step():
        if indexer_args is not None:
            idx_kernel(*indexer_args, topk)
        if attention_args is not None:
            qn, qp, ckv, kpe, idx, scale = attention_args
            rows = topk if idx is None else idx
            out = torch.empty(qn.shape, dtype=torch.bfloat16)
            lse = torch.empty(qn.shape[:2], dtype=torch.float32)
            att_kernel(qn, qp, ckv, kpe, rows, scale, out, lse)

    for _ in range(warmup):
        step()
    times = []
    for _ in range(max(1, steps)):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    return statistics.median(times), kind


# ------------------------------------------------------------------------------ workloads
class Workload:
    """A named configuration: builds its device inputs, runs one step, knows its CPU sample."""
    name = ""
    metric = ""
    scaling = "weak"

    def __init__(self, args, ranks):
        self.args, self.ranks = args, ranks

    def config(self):
        raise NotImplementedError


class Headline(Workload):
    name = "headline"
    metric = "us/call: DSA indexer + sparse attn, decode B=64 ctx 32K"

    def config(self):
        a = self.args
        return {"workload": f"dsa_decode_block B={a.batch}/GPU ctx={a.context} ps=64 topk=2048 "
                            "(indexer 64h fp8 -> sparse MLA 16h bf16)",
                "batch_per_gpu": a.batch, "context": a.context, "page_size": 64, "topk": TOPK,
                "sharding": "requests (no collective)",
                "l2": "inputs exceed L2: 278 MB key cache streamed + 151 MB gathered from a 2.4 GB cache per step"}

    def cpu_sample(self, n_req):
        from auto_gpu_kernel_b200 import inputs as wl
        a = self.args
        block = wl.make_decode_block_inputs([a.context] * n_req, seed=0, device="cpu")
        idx = block.indexer
        return (idx.args(), (block.q_nope, block.q_pe, block.ckv_cache, block.kpe_cache, None, block.sm_scale),
                a.batch / n_req, f"{n_req} of {a.batch} requests (indexer + attention), time scaled x{a.batch / n_req:g}")


# ------------------------------------------------------------------------------ reference arm
def run_reference_arm(args, ranks):
    """The CPU implementation of the path on the host cores, bounded sample of the same workload."""
    if ranks.rank != 0:
        return 0
    from auto_gpu_kernel_b200 import inputs as wl
    name = args.workload
    if name == "headline":
        w = Headline(args, ranks)
        idx_args, att_args, scale, sample = w.cpu_sample(min(args.cpu_requests, args.batch))
        metric, config, scaling = w.metric, w.config(), "weak"
    elif name == "cfg1":
        lens = wl.uniform_lengths(64, 8192, 32768, seed=1)[:16]
        inp = wl.make_attention_inputs(lens, seed=1, device="cpu")
        idx_args, att_args, scale = None, inp.args(), 4.0
        sample = "16 of 64 tokens, time scaled x4"
        metric, config, scaling = CFG1_METRIC, cfg1_config(), "weak"
    elif name == "cfg2":
        lens = wl.uniform_lengths(256, 32768, 131072, seed=2)
        pick = lens[:4]
        inp = wl.make_indexer_inputs(pick, seed=2, device="cpu")
        idx_args, att_args, scale = inp.args(), None, sum(lens) / sum(pick)
        sample = f"4 of 256 requests ({sum(pick)} of {sum(lens)} cached tokens), time scaled x{scale:.1f} by tokens"
        metric, config, scaling = CFG2_METRIC, cfg2_config(args.gpus), "strong"
    elif name == "cfg3":
        inp = wl.make_shared_prefix_indexer_inputs(prefix_len=16384, chunk_len=32, seed=4, device="cpu")
        att = wl.make_attention_inputs([16400] * 32, seed=4, device="cpu")
        idx_args = inp.args()
        att_args = (att.q_nope, att.q_pe, att.ckv_cache, att.kpe_cache, att.sparse_indices, att.sm_scale)
        scale = 4096 / 32
        sample = "32 of 4096 query rows (first rows of the chunk; indexer + attention), time scaled x128"
        metric, config, scaling = CFG3_METRIC, cfg3_config(args.gpus), "strong"
    else:
        lens = wl.uniform_lengths(128, 16384, 65536, seed=0)[:8]
        block = wl.make_decode_block_inputs(lens, seed=0, device="cpu")
        idx_args = block.indexer.args()
        att_args = (block.q_nope, block.q_pe, block.ckv_cache, block.kpe_cache, None, block.sm_scale)
        scale = 128 / 8 * 8   # 8 of 128 requests, 16 of 128 heads
        sample = "8 of 128 requests, 16 of 128 heads, time scaled x128"
        metric, config, scaling = CFG4_METRIC, cfg4_config(args.gpus), "strong"
    sec, kind = cpu_step_seconds(idx_args, att_args, max(1, args.steps), args.warmup)
    us = sec * 1e6 * scale
    cores = os.cpu_count() or 1
    line = {"metric": metric, "value": us, "unit": "us", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": us / 1e3, "higher_is_better": False,
            "scaling": scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config, "impl": "reference",
            "cpu_baseline": {"value": us, "unit": "us", "cores": cores, "kind": kind,
                             "sample": f"{sample}; median of {max(1, args.steps)} steps"},
            "e2e": {"value": us, "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))
    return 0


def cpu_baseline_for(idx_args, att_args, scale, sample):
    sec, kind = cpu_step_seconds(idx_args, att_args, steps=3, warmup=1)
    return {"value": sec * 1e6 * scale, "unit": "us", "cores": os.cpu_count() or 1, "kind": kind,
            "sample": f"{sample}; median of 3 steps"}


# ------------------------------------------------------------------------------ multi-GPU pieces
def head_sharded_setup(ranks, batch=128, lo=16384, hi=65536):
    """cfg4: B requests (contexts uniform in [lo, hi]); indexer request-sharded, all-gather of the
    index rows, attention of all tokens for this rank's 16 heads over replicated caches."""
    from auto_gpu_kernel_b200 import dist as dsa_dist, inputs as wl
    dev, rank, world = ranks.dev, ranks.rank, ranks.world
    lens = wl.uniform_lengths(batch, lo, hi, seed=0)
    block = wl.make_decode_block_inputs(lens, seed=0, device=dev)      # identical on every rank
    idx = block.indexer
    gen = torch.Generator(device=dev).manual_seed(100 + rank)           # this rank's 16 heads
    q_nope = (torch.randn(batch, 16, 512, generator=gen, device=dev) * 0.1).to(torch.bfloat16)
    q_pe = (torch.randn(batch, 16, 64, generator=gen, device=dev) * 0.1).to(torch.bfloat16)
    counts = [len(dsa_dist.shard_range(batch, r, world)) for r in range(world)]
    mine = dsa_dist.shard_range(batch, rank, world)
    sel = slice(mine.start, mine.stop)
    local_args = (idx.q_index_fp8[sel].contiguous(), idx.k_index_cache_fp8, idx.weights[sel].contiguous(),
                  idx.seq_lens[sel].contiguous(), idx.block_table[sel].contiguous())
    plan = dsa_dist.HeadShardedPlan(counts, rank, dev)
    out = torch.empty(batch, 16, 512, dtype=torch.bfloat16, device=dev)
    lse = torch.empty(batch, 16, dtype=torch.float32, device=dev)

    def make_step(p):
        def step():
            dsa_dist.decode_block_head_sharded(local_args, counts, q_nope, q_pe, block.ckv_cache,
                                               block.kpe_cache, block.sm_scale, out, lse, plan=p)
        return step

    def gather_only():
        plan.gather()

    # the same exchange as pushes into the peers' buffers by the library's own kernel (no NCCL in
    # the data path); set up collectively, so a failure is the same on every rank
    push_plan, push_error = None, None
    if world > 1:
        try:
            push_plan = dsa_dist.PeerPushPlan(counts, rank, dev)
        except Exception as exc:   # noqa: BLE001 - reported in the JSON line
            push_error = f"{type(exc).__name__}: {exc}"[:200]
        # all ranks or none (PeerPushPlan agrees on its own outcome; this covers anything else)
        every = [None] * world
        torch.distributed.all_gather_object(every, push_error)
        if any(e is not None for e in every) and push_plan is not None:
            push_plan.abandon()
            push_plan = None
        push_error = next((e for e in every if e is not None), None)
    my_tokens = sum(lens[i] for i in mine)
    return make_step(plan), gather_only, {"requests_on_rank0": len(mine), "cached_tokens_on_rank0": my_tokens,
                                          "lens": lens, "local_args": local_args,
                                          "attention": (q_nope, q_pe, block.ckv_cache, block.kpe_cache, block.sm_scale),
                                          "out": out, "lse": lse, "plan": plan, "push_plan": push_plan,
                                          "push_error": push_error,
                                          "push_step": make_step(push_plan) if push_plan is not None else None,
                                          "push_only": push_plan.gather if push_plan is not None else None}


def cfg2_setup(ranks, batch=256, lo=32768, hi=131072):
    """cfg2: B requests sharded over the ranks (strong scaling); every rank builds only its shard."""
    from auto_gpu_kernel_b200 import dist as dsa_dist, indexer, inputs as wl
    lens = wl.uniform_lengths(batch, lo, hi, seed=2)
    mine = dsa_dist.shard_range(batch, ranks.rank, ranks.world)
    my_lens = [lens[i] for i in mine]
    inp = wl.make_indexer_inputs(my_lens, seed=2 + ranks.rank, device=ranks.dev)
    topk = torch.empty(len(my_lens), TOPK, dtype=torch.int32, device=ranks.dev)

    def step():
        indexer.kernel(*inp.args(), topk)

    return step, lens, my_lens, inp, topk


CFG1_METRIC = "us/call: DSA sparse MLA attention decode, T=64, ctx 8-32K"
CFG2_METRIC = "us/call: DSA FP8 indexer decode, B=256, ctx 32-128K, request-sharded"
CFG3_METRIC = "us/call: DSA chunked prefill (16K prefix + 4096-token chunk), indexer + sparse attn, token-sharded"
CFG4_METRIC = "us/layer: full DSA block, 128 heads = 16/GPU, decode B=128 ctx 16-64K"


def cfg1_config():
    return {"workload": "dsa_sparse_attention_decode T=64 ctx~U[8K,32K] topk=2048 16 heads",
            "l2": "inputs exceed L2: 151 MB gathered per call from a 1.5 GB ckv/kpe cache"}


def cfg2_config(gpus):
    return {"workload": "dsa_indexer_decode B=256 ctx~U[32K,128K] topk=2048",
            "sharding": f"requests over {gpus} GPU(s), no collective",
            "l2": "inputs exceed L2: 2.7 GB of key pages streamed per call (whole job)"}


def cfg3_config(gpus):
    return {"workload": "dsa_chunked_prefill prefix=16384 chunk=4096 (row i sees 16384+i+1 tokens)",
            "sharding": f"query tokens over {gpus} GPU(s), key pages replicated, no collective",
            "l2": "key pages (2.7 MB) and ckv/kpe (23.6 MB) are L2-resident by nature of the workload; "
                  "the scorer is tensor-bound, the attention gathers 9.7 GB from L2 per call"}


def cfg4_config(gpus):
    return {"workload": "dsa_full_block B=128 ctx~U[16K,64K] heads=16/GPU",
            "indexer": "request-sharded", "collective": "all_gather int32 [128,2048] (1 MiB)" if gpus > 1 else "none (1 GPU)",
            "attention": "head-sharded, all 128 tokens per rank, caches replicated",
            "l2": "inputs exceed L2: 0.68 GB of key pages (whole job) + 302 MB gathered per rank from a 5.9 GB cache"}


def fp8_peak_tflops(dev):
    """Dense FP8 rate of this GPU measured the way the bf16 peak was: torch._scaled_mm 8192^3."""
    n = 8192
    a = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn)
    b = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn).t()
    one = torch.ones((), device=dev)
    try:
        for _ in range(3):
            torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        best = float("inf")
        for _ in range(10):
            e0, e1 = ev(), ev()
            e0.record()
            torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        return 2 * n ** 3 / (best * 1e-3) / 1e12, "torch._scaled_mm e4m3 8192^3, best of 10, this run"
    except Exception as exc:   # noqa: BLE001 -- report and fall back to twice the bf16 figure
        return None, f"_scaled_mm failed ({type(exc).__name__}): using 2 x bf16 peak"


# ------------------------------------------------------------------------------ comparators
def run_comparators(args, ranks):
    """The reference's GPU kernels (baseline/_ref) beside this library's, same inputs, same events.
    Only dispatches that take no in-kernel spin barrier: the second-generation attention at
    T = 64 (4 splits x 64 tokens = 256 CTAs > 144: true-last-CTA merge) and at T = 256 (no split),
    the second-generation indexer at B = 64 x 8191 tokens (its 13-bit position field ends there;
    64 x 4 chunks > 128: the unfused sort + merge pair, not the flag-synchronised kernel) and on
    short rows (one fill kernel), the contest submissions' indexer (no barrier in the file) and
    their attention at T <= 2.  A kernel that fails to build or launch on this box is recorded with
    the error text."""
    from auto_gpu_kernel_b200 import indexer, inputs as wl, sparse_attention
    dev = ranks.dev
    result = {}

    def load(name):
        spec = importlib.util.spec_from_file_location(f"dsa_ref_{name}", REF_DIR / f"{name}.py")
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod

    def time_pair(label, ours, theirs_name, theirs_call, check):
        entry = {"b200_us": timed_us(ours, args.steps, args.warmup, ranks)}
        try:
            mod = load(theirs_name)
            fn = lambda: theirs_call(mod)   # noqa: E731
            fn()                              # JIT
            torch.cuda.synchronize()
            entry["reference_us"] = timed_us(fn, args.steps, args.warmup, ranks)
            entry["reference_kernel"] = f"baseline/_ref/{theirs_name}.py::kernel"
            entry["agreement"] = check()
        except Exception as exc:   # noqa: BLE001 -- a JIT failure on this box is a result, not a crash
            entry["unavailable"] = f"{type(exc).__name__}: {str(exc)[:300]}"
        result[label] = entry

    if not (REF_DIR / "fable_attention.py").exists():
        return {"unavailable": "baseline/_ref is empty: run baseline/fetch_reference.py on a checkout of the reference"}

    def attention_pair(label, theirs, lens, seed, pad_tail=0):
        att = wl.make_attention_inputs(lens, seed=seed, device=dev, pad_tail=pad_tail)
        n = len(lens)
        out_a, lse_a = torch.empty_like(att.q_nope), torch.empty(n, 16, dtype=torch.float32, device=dev)
        out_b, lse_b = torch.empty_like(att.q_nope), torch.empty(n, 16, dtype=torch.float32, device=dev)
        time_pair(label, lambda: sparse_attention.kernel(*att.args(), out_a, lse_a), theirs,
                  lambda mod: mod.kernel(*att.args(), out_b, lse_b),
                  lambda: {"max_abs_out": float((out_a.float() - out_b.float()).abs().max()),
                           "max_abs_lse": float((lse_a - lse_b).nan_to_num(neginf=0.0).abs().max())})

    def indexer_pair(label, theirs, lens, seed, note):
        inp = wl.make_indexer_inputs(lens, seed=seed, device=dev)
        top_a = torch.empty(len(lens), TOPK, dtype=torch.int32, device=dev)
        top_b = torch.empty(len(lens), TOPK, dtype=torch.int32, device=dev)

        def overlap():
            a, b = top_a.cpu(), top_b.cpu()
            same = sum(len(set(x.tolist()) & set(y.tolist())) for x, y in zip(a, b))
            want = sum(min(n, TOPK) + (1 if n < TOPK else 0) for n in lens)   # the -1 pad counts once
            return {"mean_set_overlap": same / max(want, 1), "note": note}

        time_pair(label, lambda: indexer.kernel(*inp.args(), top_a), theirs,
                  lambda mod: mod.kernel(*inp.args(), top_b), overlap)

    # ---- the configurations of this benchmark ------------------------------------------------------
    # second-generation attention at cfg1: 64 tokens x 4 splits = 256 CTAs > 144 -> true-last-CTA merge
    attention_pair("attention_cfg1_T64", "fable_attention", wl.uniform_lengths(64, 8192, 32768, seed=1), 1)
    # ... and at 256 tokens, where it does not split at all (one CTA per token, no merge)
    attention_pair("attention_T256_ctx8K", "fable_attention", [8192] * 256, 2)
    # second-generation indexer at the longest context its 13-bit position field allows
    indexer_pair("indexer_B64_ctx8191", "fable_indexer", [8191] * 64, 7,
                 "the reference ranks by the top 19 key bits, this library exactly")
    # ---- contest-like shapes (B <= 31, contexts up to 5806, tail-padded index rows) ---------------
    # the contest submissions; only their dispatches without a spin barrier: the indexer (none in
    # the file), the attention at T <= 2 (every CTA recomputes the logits, no exchange)
    gen = torch.Generator().manual_seed(11)
    ragged = [int(x) for x in torch.randint(2049, 5807, (31,), generator=gen)]
    ragged[0], ragged[7], ragged[19] = 5806, 94, 1500
    indexer_pair("indexer_contest_B31_ctx5806", "indexer_fused", ragged, 11,
                 "both exact; rows of at most 2048 tokens are emitted whole by both")
    short = [int(x) for x in torch.randint(1, 2049, (16,), generator=gen)]
    indexer_pair("indexer_contest_B16_short", "indexer_fused", short, 12, "no scoring: every token is selected")
    indexer_pair("indexer_contest_B16_short_gen2", "fable_indexer", short, 12, "no scoring: every token is selected")
    attention_pair("attention_contest_T2_padded", "sparse_fused", [33, 1200], 13)
    return result


# ------------------------------------------------------------------------------ b200 arm
def run_headline(args, ranks):
    from auto_gpu_kernel_b200 import indexer, inputs as wl, sparse_attention, workspace
    dev, world = ranks.dev, ranks.world
    w = Headline(args, ranks)
    lens = [args.context] * args.batch
    block = wl.make_decode_block_inputs(lens, seed=ranks.rank, device=dev)
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

    # ---- timed region: exactly K steps between two events on the launching stream ----------------
    # (no event inside a step: the kernels of a step are chained by programmatic dependent launch
    #  and an event record between them would serialise them)
    sampler = ClockSampler(ranks.local)
    step_us = timed_us(step, args.steps, args.warmup, ranks, sampler)
    clocks = sample_clocks(step, sampler)
    workspace.check_status(dev)

    # ---- per-stage times -----------------------------------------------------------------------------
    # (a) each operator alone, K calls back to back (its kernels chained by dependent launch, as in
    #     the step); (b) the K steps again with an event between the two operator calls: an event
    #     record breaks the dependent-launch chain, so (b) adds a launch gap per operator and is
    #     reported for reference only
    idx_us = timed_us(lambda: indexer.kernel(*idx.args(), topk), args.steps, 3, ranks)
    att_us = timed_us(lambda: sparse_attention.kernel(block.q_nope, block.q_pe, block.ckv_cache, block.kpe_cache,
                                                      topk, block.sm_scale, out, lse), args.steps, 3, ranks)
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
    idx_sep_us = statistics.mean(a.elapsed_time(b) for a, b, _ in marks) * 1e3
    att_sep_us = statistics.mean(b.elapsed_time(c) for _, b, c in marks) * 1e3

    # ---- dominant kernel alone (indexer scorer), same inputs, K launches -------------------------
    score_us = timed_us(lambda: indexer.scores(*idx.args(), variant=0, out=score_buf), args.steps, 3, ranks)

    # ---- end to end through the public host-buffer call -------------------------------------------
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
    e2e = timed_us(host.run, args.steps, 3, ranks)   # run() synchronises: the caller reads the result every step

    stages = {"indexer_us": idx_us, "sparse_attention_us": att_us}
    extra_keys, extra_vals = [], []
    launches_per_step = 3
    if world > 1:
        # the one collective of the path, and the strong-scaled long-context indexer, in the same record
        hs_step, gather_only, info = head_sharded_setup(ranks)
        hs_us = timed_us(hs_step, args.steps, args.warmup, ranks)
        ag_us = timed_us(gather_only, args.steps, args.warmup, ranks)
        workspace.check_status(dev)
        hsp_us = timed_us(info["push_step"], args.steps, args.warmup, ranks) if info["push_step"] else 0.0
        push_us = timed_us(info["push_only"], args.steps, args.warmup, ranks) if info["push_only"] else 0.0
        try:
            workspace.check_status(dev)
        except RuntimeError:      # a poll ran out on this rank: the pushed layer is reported as not measured
            hsp_us = push_us = float("inf")
        if info["push_plan"] is not None:
            info["push_plan"].close()
        del hs_step, gather_only, info
        torch.cuda.empty_cache()
        c2_step, c2_lens, _, _, _ = cfg2_setup(ranks)
        c2_us = timed_us(c2_step, max(5, args.steps // 2), args.warmup, ranks)
        extra_keys = ["head_sharded_us", "allgather_us", "head_sharded_push_us", "push_us", "cfg2_us"]
        extra_vals = [hs_us, ag_us, hsp_us, push_us, c2_us]
        workspace.check_status(dev)

    vals = ranks.max_over_ranks([step_us, e2e, idx_us, att_us, score_us, idx_sep_us, att_sep_us] + extra_vals)
    vals = [0.0 if v == float("inf") else v for v in vals]
    step_us, e2e, idx_us, att_us, score_us, idx_sep_us, att_sep_us = vals[:7]
    if ranks.rank != 0:
        return None
    peak, _, peak_kind = measured_peaks()
    algo = indexer_bytes(lens)
    achieved = algo / (score_us * 1e-6) / 1e9
    att_algo = attention_bytes(args.batch)
    stages.update({"indexer_us": idx_us, "sparse_attention_us": att_us,
                   "indexer_hbm_gbs": algo / (idx_us * 1e-6) / 1e9,
                   "indexer_frac_of_peak": algo / (idx_us * 1e-6) / 1e9 / peak,
                   "attention_hbm_gbs": att_algo / (att_us * 1e-6) / 1e9,
                   "attention_frac_of_peak": att_algo / (att_us * 1e-6) / 1e9 / peak,
                   "step_frac_of_peak": (algo + att_algo) / (step_us * 1e-6) / 1e9 / peak})
    stages["indexer_separated_us"] = idx_sep_us
    stages["sparse_attention_separated_us"] = att_sep_us
    stages["note"] = ("*_us: the operator alone, K calls back to back; *_separated_us: inside the step with an "
                      "event between the operators (breaks the dependent-launch chain)")
    for k, v in zip(extra_keys, vals[7:]):
        stages[k] = v
    if extra_keys:
        stages["head_sharded"] = ("cfg4: B=128 ctx~U[16K,64K], indexer request-sharded, int32 [128,2048] index rows "
                                  "exchanged, attention 16 heads/GPU; head_sharded_us / allgather_us with the NCCL "
                                  "all_gather, head_sharded_push_us / push_us with the library's own exchange kernel "
                                  "(0 = could not be set up)")
        stages["cfg2"] = f"B=256 ctx~U[32K,128K], {256 // world} requests per GPU (strong scaling)"
    line = {
        "metric": w.metric, "value": step_us, "unit": "us", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": step_us / 1e3, "higher_is_better": False,
        "scaling": "weak", "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
        "config": w.config(), "impl": "b200", "stages": stages,
        "roofline": {"kernel": "indexer_score_tc_kernel", "bound": "hbm", "achieved": achieved,
                     "peak": peak, "peak_source": f"{peak_kind} copy bandwidth", "unit": "GB/s",
                     "frac": achieved / peak, "us_per_launch": score_us, "algorithmic_bytes": algo,
                     "traffic": SCORER_DRAM_BYTES_PER_TOKEN * sum(lens)},
        "e2e": {"value": e2e, "unit": "us", "h2d_bytes_per_step": host.h2d_bytes,
                "d2h_bytes_per_step": host.d2h_bytes,
                "note": "HostDecodeStep.run(): per-step inputs (q, weights, seq_lens, block_table, q_nope, "
                        "q_pe) from pinned host memory, results (indices, output, lse) read back; the paged "
                        "caches are device-resident state"},
        "gpu_launches": launches_per_step * args.steps, "clocks": clocks,
    }
    if world == 1:
        idx_args, att_args, scale, sample = w.cpu_sample(min(args.cpu_requests, args.batch))
        line["cpu_baseline"] = cpu_baseline_for(idx_args, att_args, scale, sample)
    return line


def run_cfg1(args, ranks):
    from auto_gpu_kernel_b200 import inputs as wl, sparse_attention, workspace
    dev = ranks.dev
    lens = wl.uniform_lengths(64, 8192, 32768, seed=1 + ranks.rank)
    att = wl.make_attention_inputs(lens, seed=1 + ranks.rank, device=dev)
    out, lse = torch.empty_like(att.q_nope), torch.empty(64, 16, dtype=torch.float32, device=dev)
    step = lambda: sparse_attention.kernel(*att.args(), out, lse)   # noqa: E731
    sampler = ClockSampler(ranks.local)
    us = timed_us(step, args.steps, args.warmup, ranks, sampler)
    clocks = sample_clocks(step, sampler)
    workspace.check_status(dev)
    dq, dp, di = att.q_nope.clone(), att.q_pe.clone(), att.sparse_indices.clone()
    e2e, h2d, d2h = e2e_us([att.q_nope, att.q_pe, att.sparse_indices], [dq, dp, di],
                           lambda: sparse_attention.kernel(dq, dp, att.ckv_cache, att.kpe_cache, di, att.sm_scale, out, lse),
                           [out, lse], args.steps, ranks)
    us, e2e = ranks.max_over_ranks([us, e2e])
    if ranks.rank != 0:
        return None
    peak, _, kind = measured_peaks()
    algo = attention_bytes(64)
    line = base_line(CFG1_METRIC, us, args, ranks, "weak", cfg1_config(), clocks, 1)
    line["roofline"] = {"kernel": "sparse_attn_mma_kernel", "bound": "hbm", "achieved": algo / (us * 1e-6) / 1e9,
                        "peak": peak, "peak_source": f"{kind} copy bandwidth", "unit": "GB/s",
                        "frac": algo / (us * 1e-6) / 1e9 / peak, "us_per_launch": us,
                        "algorithmic_bytes": algo, "traffic": None}
    line["e2e"] = {"value": e2e, "unit": "us", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                   "note": "q_nope, q_pe and the index rows from pinned host memory, output and LSE read back"}
    if ranks.world == 1:
        sub = wl.make_attention_inputs(lens[:16], seed=1, device="cpu")
        line["cpu_baseline"] = cpu_baseline_for(None, sub.args(), 4.0, "16 of 64 tokens, time scaled x4")
    return line


def base_line(metric, us, args, ranks, scaling, config, clocks, launches_per_step):
    return {"metric": metric, "value": us, "unit": "us", "n_gpus": ranks.world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": us / 1e3, "higher_is_better": False,
            "scaling": scaling, "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
            "config": config, "impl": "b200", "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks}


def run_cfg2(args, ranks):
    from auto_gpu_kernel_b200 import indexer, inputs as wl, workspace
    step, lens, my_lens, inp, topk = cfg2_setup(ranks)
    sampler = ClockSampler(ranks.local)
    us = timed_us(step, args.steps, args.warmup, ranks, sampler)
    clocks = sample_clocks(step, sampler)
    workspace.check_status(ranks.dev)
    width = (inp.block_table.shape[1] * 64 + 127) // 128 * 128
    score_buf = torch.empty(len(my_lens), width, dtype=torch.float32, device=ranks.dev)
    score_us = timed_us(lambda: indexer.scores(*inp.args(), variant=0, out=score_buf), args.steps, 3, ranks)
    dq, dw, dl, dt = inp.q_index_fp8.clone(), inp.weights.clone(), inp.seq_lens.clone(), inp.block_table.clone()
    e2e, h2d, d2h = e2e_us([inp.q_index_fp8.view(torch.uint8), inp.weights, inp.seq_lens, inp.block_table],
                           [dq.view(torch.uint8), dw, dl, dt],
                           lambda: indexer.kernel(dq, inp.k_index_cache_fp8, dw, dl, dt, topk),
                           [topk], args.steps, ranks)
    us, score_us, e2e = ranks.max_over_ranks([us, score_us, e2e])
    if ranks.rank != 0:
        return None
    peak, _, kind = measured_peaks()
    algo_all, algo_mine = indexer_bytes(lens), indexer_bytes(my_lens)
    line = base_line(CFG2_METRIC, us, args, ranks, "strong", cfg2_config(ranks.world), clocks, 2)
    line["stages"] = {"indexer_us": us, "scorer_us": score_us,
                      "whole_job_hbm_gbs": algo_all / (us * 1e-6) / 1e9,
                      "indexer_frac_of_peak_per_gpu": algo_mine / (us * 1e-6) / 1e9 / peak}
    line["roofline"] = {"kernel": "indexer_score_tc_kernel", "bound": "hbm",
                        "achieved": algo_mine / (score_us * 1e-6) / 1e9, "peak": peak,
                        "peak_source": f"{kind} copy bandwidth", "unit": "GB/s",
                        "frac": algo_mine / (score_us * 1e-6) / 1e9 / peak, "us_per_launch": score_us,
                        "algorithmic_bytes": algo_mine, "traffic": SCORER_DRAM_BYTES_PER_TOKEN * sum(my_lens)}
    line["e2e"] = {"value": e2e, "unit": "us", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                   "note": "q, weights, seq_lens, block_table from pinned host memory, index rows read back"}
    if ranks.world == 1:
        pick = lens[:4]
        sub = wl.make_indexer_inputs(pick, seed=2, device="cpu")
        line["cpu_baseline"] = cpu_baseline_for(sub.args(), None, sum(lens) / sum(pick),
                                                f"4 of 256 requests, time scaled x{sum(lens) / sum(pick):.1f} by cached tokens")
    return line


def run_cfg3(args, ranks):
    from auto_gpu_kernel_b200 import dist as dsa_dist, indexer, inputs as wl, sparse_attention, workspace
    dev = ranks.dev
    prefix, chunk = 16384, 4096
    inp = wl.make_shared_prefix_indexer_inputs(prefix_len=prefix, chunk_len=chunk, seed=4, device=dev)
    mine = dsa_dist.shard_range(chunk, ranks.rank, ranks.world)      # this rank's query tokens
    sel = slice(mine.start, mine.stop)
    n = len(mine)
    shared = inp.block_table[:1].expand(n, -1)
    q, wts, lens = inp.q_index_fp8[sel].contiguous(), inp.weights[sel].contiguous(), inp.seq_lens[sel].contiguous()
    pages = inp.k_index_cache_fp8.shape[0]
    gen = torch.Generator(device=dev).manual_seed(8)
    ckv = torch.randn(pages, 64, 512, generator=gen, device=dev).to(torch.bfloat16)
    kpe = torch.randn(pages, 64, 64, generator=gen, device=dev).to(torch.bfloat16)
    qn = (torch.randn(chunk, 16, 512, generator=gen, device=dev) * 0.1).to(torch.bfloat16)[sel].contiguous()
    qp = (torch.randn(chunk, 16, 64, generator=gen, device=dev) * 0.1).to(torch.bfloat16)[sel].contiguous()
    topk = torch.empty(n, TOPK, dtype=torch.int32, device=dev)
    out, lse = torch.empty_like(qn), torch.empty(n, 16, dtype=torch.float32, device=dev)
    scale = 192 ** -0.5
    width = (inp.block_table.shape[1] * 64 + 127) // 128 * 128
    score_buf = torch.empty(n, width, dtype=torch.float32, device=dev)

    def step():
        indexer.kernel(q, inp.k_index_cache_fp8, wts, lens, shared, topk)
        sparse_attention.kernel(qn, qp, ckv, kpe, topk, scale, out, lse)

    sampler = ClockSampler(ranks.local)
    us = timed_us(step, args.steps, args.warmup, ranks, sampler)
    clocks = sample_clocks(step, sampler)
    workspace.check_status(dev)
    score_us = timed_us(lambda: indexer.scores(q, inp.k_index_cache_fp8, wts, lens, shared, variant=0, out=score_buf),
                        args.steps, 3, ranks)
    idx_us = timed_us(lambda: indexer.kernel(q, inp.k_index_cache_fp8, wts, lens, shared, topk), args.steps, 3, ranks)
    att_us = timed_us(lambda: sparse_attention.kernel(qn, qp, ckv, kpe, topk, scale, out, lse), args.steps, 3, ranks)
    dq, dw, dl, dn, dp = q.clone(), wts.clone(), lens.clone(), qn.clone(), qp.clone()

    def e2e_run():
        indexer.kernel(dq, inp.k_index_cache_fp8, dw, dl, shared, topk)
        sparse_attention.kernel(dn, dp, ckv, kpe, topk, scale, out, lse)

    e2e, h2d, d2h = e2e_us([q.view(torch.uint8), wts, lens, qn, qp], [dq.view(torch.uint8), dw, dl, dn, dp],
                           e2e_run, [out, lse], max(3, args.steps // 2), ranks)
    fp8_peak, fp8_how = fp8_peak_tflops(dev) if ranks.rank == 0 else (None, "")
    us, score_us, idx_us, att_us, e2e = ranks.max_over_ranks([us, score_us, idx_us, att_us, e2e])
    if ranks.rank != 0:
        return None
    hbm, bf16, kind = measured_peaks()
    if fp8_peak is None:
        fp8_peak = 2 * bf16
    my_tokens = int(lens.sum())
    flops = 2 * 64 * 128 * my_tokens                       # scorer, this rank
    att_flops = 2 * 16 * TOPK * (576 + 512) * n            # attention, this rank
    gathered = n * TOPK * 1152
    line = base_line(CFG3_METRIC, us, args, ranks, "strong", cfg3_config(ranks.world), clocks, 3)
    line["stages"] = {"indexer_us": idx_us, "scorer_us": score_us, "select_us": idx_us - score_us,
                      "sparse_attention_us": att_us,
                      "attention_tflops": att_flops / (att_us * 1e-6) / 1e12,
                      "attention_frac_of_bf16_peak": att_flops / (att_us * 1e-6) / 1e12 / bf16,
                      "attention_l2_gather_gbs": gathered / (att_us * 1e-6) / 1e9,
                      "attention_bound": "gather from L2 (each token has its own 2048 rows): reported against both roofs"}
    line["roofline"] = {"kernel": "indexer_score_prefill_kernel", "bound": "tensor",
                        "achieved": flops / (score_us * 1e-6) / 1e12, "peak": fp8_peak,
                        "peak_source": fp8_how, "unit": "TFLOP/s",
                        "frac": flops / (score_us * 1e-6) / 1e12 / fp8_peak, "us_per_launch": score_us,
                        "algorithmic_flops": flops, "traffic": None,
                        "frac_of_2x_bf16_burst": flops / (score_us * 1e-6) / 1e12 / (2 * bf16)}
    line["e2e"] = {"value": e2e, "unit": "us", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                   "note": "chunk queries (index q, weights, lengths, q_nope, q_pe) from pinned host memory, output and LSE read back"}
    if ranks.world == 1:
        sub = wl.make_shared_prefix_indexer_inputs(prefix_len=prefix, chunk_len=32, seed=4, device="cpu")
        att = wl.make_attention_inputs([16400] * 32, seed=4, device="cpu")
        line["cpu_baseline"] = cpu_baseline_for(sub.args(), att.args(), chunk / 32,
                                                "32 of 4096 query rows (indexer + attention), time scaled x128")
    return line


def run_cfg4(args, ranks):
    from auto_gpu_kernel_b200 import indexer, sparse_attention, workspace
    nccl_step, gather_only, info = head_sharded_setup(ranks)
    push_step, push_only = info["push_step"], info["push_only"]
    # the layer as the library runs it: index rows pushed by its own kernel where that could be
    # set up, otherwise (and always at one GPU) the NCCL all-gather
    step = push_step if push_step is not None else nccl_step
    sampler = ClockSampler(ranks.local)
    us = timed_us(step, args.steps, args.warmup, ranks, sampler)
    (us_all,) = ranks.max_over_ranks([us])
    batches = None if ranks.world == 1 else max(1, int(1.2e6 / (20.0 * max(us_all, 1.0))))
    clocks = sample_clocks(step, sampler, batches)
    workspace.check_status(ranks.dev)
    nccl_us = timed_us(nccl_step, args.steps, args.warmup, ranks) if push_step is not None else us
    ag_us = timed_us(gather_only, args.steps, 3, ranks) if ranks.world > 1 else 0.0
    push_us = timed_us(push_only, args.steps, 3, ranks) if push_only is not None else 0.0
    workspace.check_status(ranks.dev)
    plan = info["plan"]
    idx_us = timed_us(lambda: indexer.kernel(*info["local_args"], plan.local_rows), args.steps, 3, ranks)
    qn, qp, ckv, kpe, scale = info["attention"]
    att_us = timed_us(lambda: sparse_attention.kernel(qn, qp, ckv, kpe, plan.all_rows, scale, info["out"], info["lse"]),
                      args.steps, 3, ranks)
    us, nccl_us, ag_us, push_us, idx_us, att_us = ranks.max_over_ranks([us, nccl_us, ag_us, push_us, idx_us, att_us])
    if info["push_plan"] is not None:
        info["push_plan"].close()
    if ranks.rank != 0:
        return None
    peak, _, kind = measured_peaks()
    att_algo = attention_bytes(128)
    line = base_line(CFG4_METRIC, us, args, ranks, "strong", cfg4_config(ranks.world), clocks, 3)
    line["config"]["indexer"] = (f"request-sharded, {info['requests_on_rank0']} requests / "
                                 f"{info['cached_tokens_on_rank0']} cached tokens on rank 0")
    if ranks.world > 1:
        line["config"]["collective"] = (
            "index rows int32 [128,2048] (1 MiB) pushed into the peers' buffers by dsa_index_rows_exchange "
            "(plain stores over NVLink, bounded wait); the NCCL all_gather of the same rows is timed beside it"
            if push_step is not None else
            f"all_gather int32 [128,2048] (1 MiB); peer push unavailable: {info['push_error']}")
    line["stages"] = {"indexer_us": idx_us, "allgather_us": ag_us, "push_us": push_us,
                      "layer_with_nccl_allgather_us": nccl_us, "layer_with_push_us": us if push_step is not None else None,
                      "sparse_attention_us": att_us,
                      "attention_frac_of_peak": att_algo / (att_us * 1e-6) / 1e9 / peak}
    line["roofline"] = {"kernel": "sparse_attn_mma_kernel", "bound": "hbm",
                        "achieved": att_algo / (att_us * 1e-6) / 1e9, "peak": peak,
                        "peak_source": f"{kind} copy bandwidth", "unit": "GB/s",
                        "frac": att_algo / (att_us * 1e-6) / 1e9 / peak, "us_per_launch": att_us,
                        "algorithmic_bytes": att_algo, "traffic": None}
    return line


RUNNERS = {"headline": run_headline, "cfg1": run_cfg1, "cfg2": run_cfg2, "cfg3": run_cfg3, "cfg4": run_cfg4}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="headline", choices=sorted(RUNNERS))
    ap.add_argument("--layout", default=None, choices=["requests", "heads"],
                    help="older spelling: `--layout heads` = `--workload cfg4`")
    ap.add_argument("--compare", action="store_true",
                    help="1 GPU: also time the reference's GPU kernels from baseline/_ref (`comparators`)")
    ap.add_argument("--batch", type=int, default=BATCH, help=argparse.SUPPRESS)
    ap.add_argument("--context", type=int, default=CONTEXT, help=argparse.SUPPRESS)
    ap.add_argument("--cpu-requests", type=int, default=16, help=argparse.SUPPRESS)
    args = ap.parse_args()
    if args.layout == "heads":
        args.workload = "cfg4"
    ranks = Ranks()

    if args.impl == "reference":
        return run_reference_arm(args, ranks)

    args.warmup = max(args.warmup, 3)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (the b200 arm has no CPU path)")
    ranks.init()
    line = RUNNERS[args.workload](args, ranks)
    if ranks.rank == 0 and line is not None:
        if args.compare and ranks.world == 1:
            line["comparators"] = run_comparators(args, ranks)
        print(json.dumps(line))
    ranks.finish()
    return 0


if __name__ == "__main__":
    sys.exit(main())
