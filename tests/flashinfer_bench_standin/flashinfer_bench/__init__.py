"""Stand-in for the third-party `flashinfer_bench` package.  TEST INFRASTRUCTURE.

The reference's harness (`kbench bench` / `kbench ab`, backend "local") evaluates a solution
through flashinfer-bench, which is not part of its tree and not installed here.  This package
offers exactly the names kbench imports (kbench/flashinfer.py:47-49, :77, :86-141) -- BuildSpec,
agents.pack_solution_from_files, data.SupportedBindings, TraceSet, BenchmarkConfig, Benchmark --
so that the unmodified kbench runs end to end on a packed solution directory:

  * a "trace set" is a directory with one `definitions.json`:
        {"<definition name>": {"kind": "indexer" | "attention",
                               "workloads": [{"uuid": "...", "seq_lens": [...], "seed": 0,
                                              "pad_tail": 0}, ...]}}
    (seeded synthetic workloads; the contest trace set is not redistributable);
  * a solution is the text of its files; `Benchmark.run_all` writes them to a scratch directory,
    imports the entry file, calls `kernel(<inputs...>, <pre-allocated outputs...>)` on every
    workload, checks against the definition's reference (the CPU oracle) and times with CUDA
    events -- the work is done by tests/local_evaluator.py.
"""
from __future__ import annotations

import enum
import json
import tempfile
from dataclasses import dataclass, field
from pathlib import Path


@dataclass
class BuildSpec:
    language: str
    target_hardware: list
    entry_point: str
    binding: object = None


@dataclass
class BenchmarkConfig:
    warmup_runs: int = 3
    iterations: int = 100
    num_trials: int = 5
    profile_baseline: bool = False


@dataclass
class Definition:
    name: str
    kind: str


@dataclass
class Workload:
    uuid: str
    seq_lens: list
    seed: int = 0
    pad_tail: int = 0


@dataclass
class Solution:
    name: str
    definition: str
    author: str
    spec: BuildSpec
    files: dict


class EvaluationStatus(enum.Enum):
    PASSED = "passed"
    FAILED = "failed"
    ERROR = "error"


@dataclass
class Performance:
    latency_ms: float | None
    reference_latency_ms: float | None


@dataclass
class Correctness:
    max_absolute_error: float | None
    max_relative_error: float | None


@dataclass
class Evaluation:
    status: EvaluationStatus
    log: str | None
    performance: Performance | None
    correctness: Correctness | None


@dataclass
class Trace:
    workload: Workload
    evaluation: Evaluation | None


@dataclass
class TraceSet:
    root: Path
    definitions: dict = field(default_factory=dict)
    solutions: dict = field(default_factory=dict)
    workloads: dict = field(default_factory=dict)
    traces: dict = field(default_factory=dict)

    @classmethod
    def from_path(cls, path):
        root = Path(path)
        raw = json.loads((root / "definitions.json").read_text())
        defs = {name: Definition(name, d["kind"]) for name, d in raw.items()}
        work = {name: [Workload(w["uuid"], list(w["seq_lens"]), int(w.get("seed", 0)),
                                int(w.get("pad_tail", 0))) for w in d["workloads"]]
                for name, d in raw.items()}
        return cls(root=root, definitions=defs, workloads=work)


class Benchmark:
    def __init__(self, trace_set: TraceSet, config: BenchmarkConfig):
        self.trace_set, self.config = trace_set, config

    def run_all(self, dump_traces: bool = True) -> TraceSet:
        import torch
        import local_evaluator as ev          # tests/local_evaluator.py
        cfg = self.config
        out = {}
        for name, definition in self.trace_set.definitions.items():
            traces = []
            for solution in self.trace_set.solutions.get(name, []):
                with tempfile.TemporaryDirectory() as tmp:
                    for rel, text in solution.files.items():
                        path = Path(tmp) / rel
                        path.parent.mkdir(parents=True, exist_ok=True)
                        path.write_text(text)
                    kernel = ev.load_entry(tmp, solution.spec.entry_point)
                    loads = self.trace_set.workloads.get(name, [])
                    if definition.kind == "indexer":
                        results = ev.evaluate_indexer(kernel, {w.uuid: (w.seq_lens, w.seed) for w in loads},
                                                      torch.device("cuda", 0), cfg.warmup_runs, cfg.iterations,
                                                      cfg.num_trials)
                    else:
                        results = ev.evaluate_attention(
                            kernel, {w.uuid: (w.seq_lens, w.seed, w.pad_tail) for w in loads},
                            torch.device("cuda", 0), cfg.warmup_runs, cfg.iterations, cfg.num_trials)
                by_id = {w.uuid: w for w in loads}
                for r in results:
                    traces.append(Trace(by_id[r.workload_id], Evaluation(
                        EvaluationStatus(r.status), r.log,
                        Performance(r.latency_ms, r.reference_latency_ms) if r.latency_ms is not None else None,
                        Correctness(r.max_abs_error, r.max_rel_error) if r.max_abs_error is not None else None)))
            out[name] = traces
        return TraceSet(root=self.trace_set.root, definitions=self.trace_set.definitions,
                        solutions=self.trace_set.solutions, workloads=self.trace_set.workloads, traces=out)
