"""Write a solution directory that the reference's harness can ship.

    python -m auto_gpu_kernel_b200.pack <dest_dir>

kbench sends a solution as {relative path: text} of the files under `sources` whose suffix is one
of .py .cu .cuh .cpp .h .hpp .txt .json .toml (kbench/flashinfer.py:17-33), and the evaluator
imports `entry_point = "<file>::kernel"` (kbench/config.py:135-138).  A shared library cannot
travel, so the directory holds the CUDA sources and the host modules, and the library is compiled
with nvcc on first import on the evaluator's GPU box:

    <dest>/indexer.py        entry_point = "indexer.py::kernel"     (FP8 top-k indexer)
    <dest>/attention.py      entry_point = "attention.py::kernel"   (sparse MLA attention)
    <dest>/dsa_b200/         host modules (ctypes loader, build, workspace, the two operators)
    <dest>/dsa_b200/csrc/    *.cu, *.cuh
    <dest>/include/dsa_b200.h
    <dest>/config.toml       the [solution]/[build] keys for either entry
"""
from __future__ import annotations

import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
SHIPPABLE = {".py", ".cu", ".cuh", ".cpp", ".h", ".hpp", ".txt", ".json", ".toml"}
HOST_MODULES = ["__init__.py", "_lib.py", "build.py", "workspace.py", "indexer.py",
                "sparse_attention.py"]

ENTRY = '''"""Entry file for flashinfer-bench: `kernel` has the definition's signature
({signature}).
The CUDA sources beside this file are compiled for sm_100a on first use."""
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))

from dsa_b200.{module} import kernel, run  # noqa: E402,F401
'''

CONFIG = '''# Either definition; pick the entry_point that matches [solution].definition.
[solution]
name = "dsa-b200"
definition = "dsa_topk_indexer_fp8_h64_d128_topk2048_ps64"   # or dsa_sparse_attention_h16_ckv512_kpe64_topk2048_ps64
author = "dsa-b200"

[build]
language = "triton"          # kbench's name for "Python entry, no TVM-FFI binding"
entry_point = "indexer.py::kernel"                            # or "attention.py::kernel"
'''


def pack(dest) -> list:
    """Create the directory; returns the relative paths written."""
    dest = Path(dest)
    written = []

    def put(rel: str, text: str):
        path = dest / rel
        if path.suffix not in SHIPPABLE:
            raise ValueError(f"{rel}: suffix {path.suffix} does not travel through kbench")
        path.parent.mkdir(parents=True, exist_ok=True)
        path.write_text(text)
        written.append(rel)

    put("indexer.py", ENTRY.format(
        module="indexer",
        signature="q_index_fp8, k_index_cache_fp8, weights, seq_lens, block_table, topk_indices"))
    put("attention.py", ENTRY.format(
        module="sparse_attention",
        signature="q_nope, q_pe, ckv_cache, kpe_cache, sparse_indices, sm_scale, output, lse"))
    put("config.toml", CONFIG)
    for name in HOST_MODULES:
        put(f"dsa_b200/{name}", (PKG_DIR / name).read_text())
    for src in sorted((PKG_DIR / "csrc").iterdir()):
        if src.suffix in (".cu", ".cuh"):
            put(f"dsa_b200/csrc/{src.name}", src.read_text())
    for hdr in sorted((PKG_DIR.parent / "include").glob("*.h")):
        put(f"include/{hdr.name}", hdr.read_text())
    return written


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    for rel in pack(sys.argv[1]):
        print(rel)
