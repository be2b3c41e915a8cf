#!/usr/bin/env python
"""Copy the reference's own files for the DSA hot path out of a checkout of Dogacel/auto-gpu-kernel
into baseline/_ref/ (git-ignored: the reference's sources are never committed here).

    python baseline/fetch_reference.py [path/to/auto-gpu-kernel]      (default: $DSA_REFERENCE_ROOT)

What is copied, unmodified:
  * the two PyTorch definitions -- archive/dsa_topk_indexer_*/solution/triton/indexer_baseline.py and
    archive/dsa_sparse_attention_*/solution/triton/sparse_baseline.py: `bench.py --impl reference`
    times exactly these on the host cores when they are present (kind "reference"), and the CPU
    restatement in oracle/ otherwise (kind "port");
  * the reference's GPU kernels for the same two definitions -- the contest submissions
    (.../solution/triton/indexer_fused.py, sparse_fused.py) and the second generation
    (archive/fable/dsa_*.py, Triton + Gluon): `bench.py --compare` times them beside this library's
    kernels on the same GPU, same inputs, same event protocol;
  * the `kbench` package: tests/test_kbench_local.py drives `kbench bench` end to end with it.
Nothing of this is imported by the library itself.
"""
from __future__ import annotations

import os
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"
IDX = "archive/dsa_topk_indexer_fp8_h64_d128_topk2048_ps64/solution/triton"
ATT = "archive/dsa_sparse_attention_h16_ckv512_kpe64_topk2048_ps64/solution/triton"
FILES = {
    f"{IDX}/indexer_baseline.py": "indexer_baseline.py",
    f"{IDX}/indexer_fused.py": "indexer_fused.py",
    f"{ATT}/sparse_baseline.py": "sparse_baseline.py",
    f"{ATT}/sparse_fused.py": "sparse_fused.py",
    "archive/fable/dsa_topk_indexer_fp8_h64_d128_topk2048_ps64.py": "fable_indexer.py",
    "archive/fable/dsa_sparse_attention_h16_ckv512_kpe64_topk2048_ps64.py": "fable_attention.py",
}


def fetch(root: Path, dest: Path = DEST) -> list:
    copied = []
    dest.mkdir(parents=True, exist_ok=True)
    for src, name in FILES.items():
        path = root / src
        if not path.is_file():
            raise FileNotFoundError(f"{path} not found: is {root} a checkout of the reference?")
        shutil.copyfile(path, dest / name)
        copied.append(name)
    pkg = root / "kbench"
    if pkg.is_dir():
        shutil.rmtree(dest / "kbench", ignore_errors=True)
        shutil.copytree(pkg, dest / "kbench", ignore=shutil.ignore_patterns("__pycache__"))
        copied.append("kbench/")
    return copied


def main(argv) -> int:
    root = Path(argv[1] if len(argv) > 1 else os.environ.get("DSA_REFERENCE_ROOT", ""))
    if not str(root) or not root.is_dir():
        print(__doc__)
        return 2
    print("\n".join(fetch(root)))
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv))
