"""`bench.py --impl reference` on the host cores: one JSON line with the keys the driver reads, for a
workload small enough for the CPU suite (cfg1's attention sample; the indexer samples take
minutes).  With baseline/_ref present the unmodified reference files are timed (kind "reference"),
otherwise the CPU restatement (kind "port")."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_reference_arm_prints_one_json_line():
    proc = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--workload", "cfg1",
                           "--steps", "1", "--warmup", "0"], capture_output=True, text=True, cwd=str(ROOT),
                          timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [l for l in proc.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["unit"] == "us" and line["higher_is_better"] is False
    assert line["value"] > 0 and line["n_gpus"] == 1 and line["gpu_launches"] == 0
    assert line["config"]["workload"].startswith("dsa_sparse_attention_decode")
    base = line["cpu_baseline"]
    have_ref = (ROOT / "baseline" / "_ref" / "sparse_baseline.py").exists()
    assert base["kind"] == ("reference" if have_ref else "port")
    assert base["cores"] >= 1 and "16 of 64 tokens" in base["sample"] and base["value"] == line["value"]
    assert line["e2e"] == {"value": line["value"], "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
