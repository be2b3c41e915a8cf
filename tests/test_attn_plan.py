"""Host logic of the attention work split: the planner's invariants over a sweep of token counts,
index widths and SM counts (compiled with nvcc, runs on the CPU)."""
import shutil
import subprocess
from pathlib import Path

import pytest

HERE = Path(__file__).resolve().parent


def test_contiguous_split_invariants(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        pytest.skip("nvcc not available")
    exe = tmp_path / "plan_check"
    build = subprocess.run([nvcc, "-std=c++17", "-O1", "-o", str(exe), str(HERE / "plan_check.cu")],
                           capture_output=True, text=True, timeout=300)
    assert build.returncode == 0, build.stdout + build.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stdout[-2000:]
    assert "0 violations" in run.stdout
