"""The C-ABI library without a GPU: it builds, loads, exports every symbol include/dsa_b200.h
declares, and its host-side argument checks answer before any CUDA call."""
import ctypes
import re
from pathlib import Path

import pytest

from auto_gpu_kernel_b200 import _lib, build

ROOT = Path(__file__).resolve().parent.parent


def declared_functions():
    text = (ROOT / "include" / "dsa_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dsa_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    names = declared_functions()
    assert names, "no declarations found"
    assert set(names) == set(_lib.SIGNATURES), (names, sorted(_lib.SIGNATURES))


def test_library_builds_and_exports_every_declared_symbol():
    path = build.build()
    raw = ctypes.CDLL(str(path))
    for name in declared_functions():
        assert hasattr(raw, name), f"{name} not exported"
    lib = _lib.load()
    assert lib.dsa_b200_version() == 1


def test_host_side_argument_errors():
    lib = _lib.load()
    # min/max words (512 KB) + 1024 score histograms of 4096 bins + score rows
    assert lib.dsa_indexer_workspace_bytes(64, 512) == 512 * 1024 + 1024 * 4096 * 4 + 64 * 512 * 64 * 4
    assert lib.dsa_indexer_workspace_bytes(1, 1) % 256 == 0
    assert lib.dsa_sparse_attn_workspace_bytes(64, 16, 2048) > 64 * 16 * 512 * 4
    # batch 0 is a no-op; null pointers and bad shapes are reported without touching the device
    assert lib.dsa_indexer_topk(None, None, None, None, None, 0, None, 0, 0, 0, 0, None, 0, None, None) == 0
    assert lib.dsa_indexer_topk(None, None, None, None, None, 0, None, 0, 4, 8, 8, None, 0, None, None) == -1
    assert lib.dsa_indexer_topk(16, 16, 16, 16, 16, 8, 16, 2048, 4, 8, 8, 256, 16, None, None) == -3
    assert lib.dsa_indexer_scores(16, 16, 16, 16, 16, 8, 16, 100, 4, 8, 8, 0, None, None) == -2
    assert lib.dsa_indexer_scores(16, 16, 16, 16, 16, 8, 16, 512, 4, 8, 8, 7, None, None) == -5
    assert lib.dsa_sparse_attn(None, None, None, None, None, 0, 1.0, None, None, 2, 16, 2048, 64, None, 0, None, None) == -1
    assert lib.dsa_sparse_attn(16, 16, 16, 16, 16, 2048, 1.0, 16, 16, 2, 8, 2048, 64, 256, 1 << 30, None, None) == -2
    assert lib.dsa_sparse_attn(16, 16, 16, 16, 16, 2048, 1.0, 16, 16, 2, 16, 2048, 64, 256, 16, None, None) == -3
    assert b"workspace" in lib.dsa_b200_error_string(-3)


def test_check_raises():
    with pytest.raises(RuntimeError, match="null pointer"):
        _lib.check(-1, "x")
