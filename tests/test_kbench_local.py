"""`kbench bench` / `kbench ab` of the UNMODIFIED reference harness (copied to baseline/_ref/kbench by
baseline/fetch_reference.py), backend "local", on the packed solution directory, with
tests/flashinfer_bench_standin in place of the third-party evaluator: the drop-in boundary
exercised from the harness's own command line down to the kernels (kbench/cli.py:33-48 ->
adapters/flashinfer.py:42-85 -> backends/local.py:12-24 -> kbench/flashinfer.py:73-141)."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

from auto_gpu_kernel_b200 import build, pack

ROOT = Path(__file__).resolve().parent.parent
KBENCH = ROOT / "baseline" / "_ref"
STANDIN = ROOT / "tests" / "flashinfer_bench_standin"
IDX_DEF = "dsa_topk_indexer_fp8_h64_d128_topk2048_ps64"
ATT_DEF = "dsa_sparse_attention_h16_ckv512_kpe64_topk2048_ps64"

needs_kbench = pytest.mark.skipif(not (KBENCH / "kbench" / "cli.py").exists(),
                                  reason="baseline/_ref/kbench missing: run baseline/fetch_reference.py")


def _project(tmp_path, definition, entry):
    """A kbench project: config.toml, solution/b200/ (the packed directory), a synthetic trace set."""
    root = tmp_path / "project"
    pack.pack(root / "solution" / "b200")
    traces = tmp_path / "traces"
    traces.mkdir()
    (traces / "definitions.json").write_text(json.dumps({
        IDX_DEF: {"kind": "indexer", "workloads": [
            {"uuid": "idx-small", "seq_lens": [94, 700, 2048], "seed": 1},
            {"uuid": "idx-contest-max", "seq_lens": [5806, 3000, 120, 2500], "seed": 2},
            {"uuid": "idx-long", "seq_lens": [40000, 2049], "seed": 3}]},
        ATT_DEF: {"kind": "attention", "workloads": [
            {"uuid": "att-padded", "seq_lens": [33, 500, 5000], "seed": 4},
            {"uuid": "att-full", "seq_lens": [9000] * 8, "seed": 5}]}}))
    (root / "config.toml").write_text(f'''
[kernel]
definition = "{definition}"
language = "triton"
source_dir = "b200"
entry_point = "{entry}"

[remote]
backend = "local"
gpu = "B200"

[remote.data]
local_path = "{traces}"

[bench]
warmup_runs = 1
iterations = 3
num_trials = 1
''')
    return root


def _env():
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join(str(p) for p in (KBENCH, STANDIN, ROOT / "tests", ROOT / "oracle", ROOT))
    env.pop("KBENCH_ROOT", None)
    return env


@needs_kbench
def test_standin_offers_what_kbench_imports(tmp_path):
    """No GPU: kbench's own packing step runs against the stand-in."""
    code = (
        "import tempfile\n"
        "from kbench.flashinfer import _pack\n"
        "from kbench.job import Job\n"
        "job = Job(definition='d', language='triton', entry_point='indexer.py::kernel',\n"
        "          sources={}, data_path='/nowhere')\n"
        "with tempfile.TemporaryDirectory() as tmp:\n"
        "    sol = _pack(job, {'indexer.py': 'def kernel(): pass', 'pkg/x.cu': '// x'}, tmp)\n"
        "assert sorted(sol.files) == ['indexer.py', 'pkg/x.cu'] and sol.spec.binding is None\n"
        "from flashinfer_bench import Benchmark, BenchmarkConfig, TraceSet\n"
        "print('ok')\n")
    proc = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=_env(),
                          cwd=str(tmp_path), timeout=120)
    assert proc.returncode == 0 and proc.stdout.strip() == "ok", proc.stdout + proc.stderr


@needs_kbench
@pytest.mark.gpu
@pytest.mark.parametrize("definition,entry", [(IDX_DEF, "indexer.py::kernel"), (ATT_DEF, "attention.py::kernel")],
                         ids=["indexer", "attention"])
def test_kbench_bench_runs_the_packed_solution(tmp_path, definition, entry):
    root = _project(tmp_path, definition, entry)
    lib = build.build()                      # the packed sources are the same: reuse the built library
    out = tmp_path / "result.json"
    proc = subprocess.run([sys.executable, "-m", "kbench.cli", "bench", "--json", str(out),
                           "--env", f"DSA_B200_LIB={lib}"],
                          capture_output=True, text=True, env=_env(), cwd=str(root), timeout=900)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    summary = json.loads(out.read_text())["summary"]
    assert summary["definition"] == definition and summary["backend"] == "local"
    assert summary["num_workloads"] >= 2 and summary["num_passed"] == summary["num_workloads"]
    assert summary["mean_latency_ms"] > 0
    history = (root / ".kopt" / "bench.jsonl").read_text().strip().splitlines()
    assert len(history) == 1 and json.loads(history[0])["num_passed"] == summary["num_workloads"]


@needs_kbench
@pytest.mark.gpu
def test_kbench_ab_compares_two_candidates(tmp_path):
    root = _project(tmp_path, IDX_DEF, "indexer.py::kernel")
    lib = build.build()
    other = tmp_path / "candidate_b.py"
    other.write_text((root / "solution" / "b200" / "indexer.py").read_text() + "\n# candidate B\n")
    proc = subprocess.run([sys.executable, "-m", "kbench.cli", "ab", "--a", str(other), "--quick",
                           "--env", f"DSA_B200_LIB={lib}"],
                          capture_output=True, text=True, env=_env(), cwd=str(root), timeout=900)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
