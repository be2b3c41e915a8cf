"""A local stand-in for the evaluator the reference's harness drives.  TEST INFRASTRUCTURE.

The reference benchmarks a solution through flashinfer-bench (`Benchmark(...).run_all()`, called
from kbench/flashinfer.py:96-141), a third-party package that is not part of its tree: it imports
the solution's entry file, calls `kernel(<definition inputs...>, <pre-allocated outputs...>)`
positionally on every workload (destination-passing style, kopt/init.py:87-96), compares with the
definition's PyTorch reference and times warm-up + iterations x trials with CUDA events
(defaults in kbench/adapters/flashinfer.py:35-37: 3 warm-ups, 50 iterations, 5 trials).

This module does the same for a *packed solution directory* (auto_gpu_kernel_b200.pack) over
seeded synthetic workloads, with the oracle as the definition's reference, and returns records with
the fields of kbench's `WorkloadResult` (kbench/results.py:11-19).
"""
from __future__ import annotations

import importlib.util
import statistics
import time
from dataclasses import dataclass
from pathlib import Path

import torch

import dsa_oracle as oracle
from auto_gpu_kernel_b200 import inputs as wl


@dataclass
class WorkloadResult:                      # same fields as kbench/results.py:11-19
    workload_id: str
    status: str                            # "passed" | "failed" | "error"
    latency_ms: float | None = None
    reference_latency_ms: float | None = None
    max_abs_error: float | None = None
    max_rel_error: float | None = None
    log: str | None = None


def load_entry(solution_dir, entry_point: str):
    """`entry_point` is "<file>::<symbol>" as in config.toml (kbench/config.py:135-138)."""
    file_name, symbol = entry_point.split("::")
    path = Path(solution_dir) / file_name
    spec = importlib.util.spec_from_file_location(f"packed_{path.stem}", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return getattr(mod, symbol)


def _time_ms(fn, warmup, iterations, trials):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    samples = []
    for _ in range(trials):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iterations):
            fn()
        b.record()
        torch.cuda.synchronize()
        samples.append(a.elapsed_time(b) / iterations)
    return statistics.median(samples)


def evaluate_indexer(kernel, workloads, device, warmup=3, iterations=20, trials=3):
    """workloads: {id: (seq_lens, seed)}.  Correctness = the acceptance rule of the definition
    (exact set where the boundary gap allows, see oracle.check_topk_row)."""
    out = []
    for wid, (lens, seed) in workloads.items():
        inp = wl.make_indexer_inputs(lens, seed=seed, device=device)
        topk = torch.full((len(lens), wl.TOPK), -7, dtype=torch.int32, device=device)
        try:
            kernel(*inp.args(), topk)      # positional, outputs last, nothing returned
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            rows = [r.cpu() for r in oracle.indexer_scores(*inp.args())]
            ref_ms = (time.perf_counter() - t0) * 1e3
            cpu = inp.to("cpu")
            bad = [b for b, row in enumerate(rows)
                   if not oracle.check_topk_row(row, cpu.block_table[b], int(cpu.seq_lens[b]),
                                                topk[b].cpu())["ok"]]
            lat = _time_ms(lambda: kernel(*inp.args(), topk), warmup, iterations, trials)
            out.append(WorkloadResult(wid, "failed" if bad else "passed", lat, ref_ms, 0.0, 0.0,
                                      f"rows failing the set rule: {bad}" if bad else None))
        except Exception as exc:           # the evaluator records errors, it does not raise
            out.append(WorkloadResult(wid, "error", log=repr(exc)))
    return out


def evaluate_attention(kernel, workloads, device, warmup=3, iterations=20, trials=3,
                       atol=1e-2, rtol=1e-2):
    """workloads: {id: (seq_lens, seed, pad_tail)}."""
    out = []
    for wid, (lens, seed, pad_tail) in workloads.items():
        inp = wl.make_attention_inputs(lens, seed=seed, device=device, pad_tail=pad_tail)
        o = torch.empty_like(inp.q_nope)
        lse = torch.empty(inp.q_nope.shape[:2], dtype=torch.float32, device=device)
        try:
            kernel(*inp.args(), o, lse)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            ref_o, ref_l = oracle.sparse_attention(*inp.args(), output=torch.empty_like(o),
                                                   lse=torch.empty_like(lse))
            torch.cuda.synchronize()
            ref_ms = (time.perf_counter() - t0) * 1e3
            err = (o.float() - ref_o.float()).abs()
            rel = err / ref_o.float().abs().clamp_min(1e-6)
            ok = bool((err <= atol + rtol * ref_o.float().abs()).all()) and \
                bool(torch.allclose(lse, ref_l, atol=1e-3, rtol=1e-3))
            lat = _time_ms(lambda: kernel(*inp.args(), o, lse), warmup, iterations, trials)
            out.append(WorkloadResult(wid, "passed" if ok else "failed", lat, ref_ms,
                                      float(err.max()), float(rel[err > atol].max()) if (err > atol).any() else 0.0))
        except Exception as exc:
            out.append(WorkloadResult(wid, "error", log=repr(exc)))
    return out
