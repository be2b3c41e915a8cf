"""The shippable solution directory: only text files kbench forwards, self-contained, and its
library builds and exports the whole C ABI (no compute without a GPU)."""
import subprocess
import sys
from pathlib import Path

import pytest

from auto_gpu_kernel_b200 import pack

SUFFIXES = {".py", ".cu", ".cuh", ".cpp", ".h", ".hpp", ".txt", ".json", ".toml"}   # kbench/flashinfer.py:17


def test_pack_tree_is_text_only_and_complete(tmp_path):
    written = pack.pack(tmp_path / "sol")
    files = [p for p in (tmp_path / "sol").rglob("*") if p.is_file()]
    assert sorted(str(p.relative_to(tmp_path / "sol")) for p in files) == sorted(written)
    assert all(p.suffix in SUFFIXES for p in files)
    for must in ("indexer.py", "attention.py", "config.toml", "include/dsa_b200.h",
                 "dsa_b200/_lib.py", "dsa_b200/csrc/abi.cu", "dsa_b200/csrc/common.cuh"):
        assert must in written
    for p in files:
        p.read_text()   # decodes as text
    # nothing in the shipped host modules reaches back into this repository
    for p in (tmp_path / "sol" / "dsa_b200").glob("*.py"):
        text = p.read_text()
        assert "auto_gpu_kernel_b200 import" not in text and "import auto_gpu_kernel_b200" not in text
        assert "oracle" not in text


def test_packed_solution_builds_and_exports_abi(tmp_path):
    pack.pack(tmp_path / "sol")
    code = (
        "import sys; sys.path.insert(0, sys.argv[1])\n"
        "import dsa_b200._lib as L\n"
        "lib = L.load()\n"
        "assert str(L.library_path()).startswith(sys.argv[1]), L.library_path()\n"
        "assert lib.dsa_b200_version() == 1\n"
        "import indexer, attention\n"
        "assert callable(indexer.kernel) and callable(attention.kernel)\n"
        "assert indexer.kernel.__module__ == 'dsa_b200.indexer'\n"
        "print('ok', len(L.SIGNATURES))\n"
    )
    proc = subprocess.run([sys.executable, "-c", code, str(tmp_path / "sol")], capture_output=True,
                          text=True, cwd=str(tmp_path), timeout=600)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert proc.stdout.strip().startswith("ok")


@pytest.mark.gpu
def test_packed_solution_runs(tmp_path):
    """The packed entry files, imported from a scratch directory, against the in-tree operators."""
    pack.pack(tmp_path / "sol")
    code = (
        "import sys, torch; sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[2])\n"
        "import indexer, attention\n"
        "from auto_gpu_kernel_b200 import inputs as wl, indexer as ref_idx, sparse_attention as ref_att\n"
        "blk = wl.make_decode_block_inputs([4000, 100, 2500], seed=2, device='cuda')\n"
        "topk = torch.empty(3, 2048, dtype=torch.int32, device='cuda')\n"
        "indexer.kernel(*blk.indexer.args(), topk)\n"
        "want = ref_idx.run(*blk.indexer.args())\n"
        "assert torch.equal(topk.sort(dim=1).values, want.sort(dim=1).values)\n"
        "out = torch.empty_like(blk.q_nope); lse = torch.empty(3, 16, device='cuda')\n"
        "attention.kernel(blk.q_nope, blk.q_pe, blk.ckv_cache, blk.kpe_cache, topk, blk.sm_scale, out, lse)\n"
        "o2, l2 = ref_att.run(blk.q_nope, blk.q_pe, blk.ckv_cache, blk.kpe_cache, topk, blk.sm_scale)\n"
        "torch.cuda.synchronize()\n"
        "assert torch.equal(out.view(torch.int16), o2.view(torch.int16)) and torch.equal(lse, l2)\n"
        "print('ok')\n"
    )
    repo = str(Path(__file__).resolve().parent.parent)
    proc = subprocess.run([sys.executable, "-c", code, str(tmp_path / "sol"), repo],
                          capture_output=True, text=True, cwd=str(tmp_path), timeout=900)
    assert proc.returncode == 0, proc.stdout + proc.stderr
