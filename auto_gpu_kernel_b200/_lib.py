"""ctypes binding of libdsa_b200.so -- the only way the package reaches the GPU.

There is no fallback: if the shared library is missing or lacks a symbol declared in
include/dsa_b200.h, importing an operator raises.  Build it with
`python -m auto_gpu_kernel_b200.build` (nvcc, sm_100a).
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

from . import build as _build

_c_int = ctypes.c_int
_c_i64 = ctypes.c_int64
_c_size = ctypes.c_size_t
_ptr = ctypes.c_void_p
_c_float = ctypes.c_float

# name -> (restype, argtypes); mirrors include/dsa_b200.h one to one.
SIGNATURES = {
    "dsa_b200_version": (_c_int, []),
    "dsa_b200_error_string": (ctypes.c_char_p, [_c_int]),
    "dsa_indexer_workspace_bytes": (_c_size, [_c_int, _c_int]),
    "dsa_indexer_topk": (_c_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _c_i64, _ptr, _c_i64, _c_int,
                                  _c_int, _c_int, _ptr, _c_size, _ptr, _ptr]),
    "dsa_indexer_topk_noalloc": (_c_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _c_i64, _ptr, _c_i64, _c_int,
                                          _c_int, _c_int, _ptr, _ptr]),
    "dsa_indexer_scores": (_c_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _c_i64, _ptr, _c_i64, _c_int,
                                    _c_int, _c_int, _c_int, _ptr, _ptr]),
    "dsa_topk_select": (_c_int, [_ptr, _c_i64, _ptr, _ptr, _c_i64, _ptr, _c_i64, _c_int, _c_int,
                                 _ptr, _ptr]),
    "dsa_sparse_attn_workspace_bytes": (_c_size, [_c_int, _c_int, _c_int]),
    "dsa_sparse_attn": (_c_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _c_i64, _c_float, _ptr, _ptr,
                                 _c_int, _c_int, _c_int, _c_i64, _ptr, _c_size, _ptr, _ptr]),
    "dsa_sparse_attn_tcgen05": (_c_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _c_i64, _c_float, _ptr,
                                         _ptr, _c_int, _c_int, _c_int, _c_i64, _ptr, _c_size,
                                         _ptr, _ptr]),
    "dsa_sparse_attn_cuda_core": (_c_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _c_i64, _c_float, _ptr,
                                           _ptr, _c_int, _c_int, _c_int, _c_i64, _ptr, _c_size,
                                           _ptr, _ptr]),
    "dsa_index_cache_write": (_c_int, [_ptr, _c_int, _c_i64, _ptr, _ptr, _c_int, _c_int, _ptr, _ptr]),
    "dsa_kv_cache_append": (_c_int, [_ptr, _c_i64, _ptr, _c_i64, _ptr, _ptr, _ptr, _c_int, _c_i64,
                                     _ptr, _ptr]),
    "dsa_decode_step_host": (_c_int, [_ptr]),
    "dsa_peer_slab_create": (_c_int, [_c_size, _ptr, _ptr]),
    "dsa_peer_slab_open": (_c_int, [_ptr, _ptr]),
    "dsa_peer_slab_close": (_c_int, [_ptr]),
    "dsa_peer_slab_destroy": (_c_int, [_ptr]),
    "dsa_index_rows_exchange": (_c_int, [_ptr, _ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_i64,
                                         _c_int, ctypes.c_uint32, _c_int, ctypes.c_uint64, _ptr, _ptr]),
    "dsa_indexer_topk_send": (_c_int, [_ptr, _ptr, _ptr, _ptr, _ptr, _c_i64, _ptr, _c_i64, _c_int, _c_int,
                                       _c_int, _ptr, _c_size, _ptr, _c_int, _c_int, _c_int,
                                       ctypes.c_uint32, _ptr, _ptr]),
    "dsa_selftest_wait_expiry": (_c_int, [ctypes.c_uint64, _ptr, _ptr, _ptr]),
    "dsa_selftest_mma_rate": (_c_int, [_c_int, _c_int, _c_int, _c_int, _ptr, _ptr, _ptr, _ptr]),
}


class HostStepArgs(ctypes.Structure):
    """Mirror of `dsa_host_step_args` in include/dsa_b200.h (same order, same types)."""
    _fields_ = [
        ("host_in", _ptr), ("dev_in", _ptr), ("in_indexer_bytes", _c_size),
        ("in_attention_bytes", _c_size), ("host_out", _ptr), ("dev_out", _ptr),
        ("out_attention_bytes", _c_size), ("out_indices_bytes", _c_size),
        ("q_index_fp8", _ptr), ("weights", _ptr), ("seq_lens", _ptr), ("block_table", _ptr),
        ("block_table_stride", _c_i64), ("q_nope", _ptr), ("q_pe", _ptr), ("output", _ptr),
        ("lse", _ptr), ("topk_indices", _ptr),
        ("k_index_cache", _ptr), ("ckv_cache", _ptr), ("kpe_cache", _ptr),
        ("batch", _c_int), ("num_pages", _c_int), ("max_pages", _c_int), ("num_slots", _c_i64),
        ("sm_scale", _c_float), ("indexer_workspace", _ptr), ("indexer_workspace_bytes", _c_size),
        ("attention_workspace", _ptr), ("attention_workspace_bytes", _c_size),
        ("status_dev", _ptr), ("stream", _ptr), ("side_stream", _ptr),
        ("ev_first_copy", _ptr), ("ev_q_ready", _ptr), ("ev_indices_ready", _ptr),
    ]


_lib = None


def library_path() -> Path:
    """DSA_B200_LIB if set; else next to this file; else, when that directory is read-only (a
    solution unpacked by an evaluator), a per-source-digest directory under the temp dir."""
    override = os.environ.get("DSA_B200_LIB")
    if override:
        return Path(override)
    if os.access(_build.PKG_DIR, os.W_OK):
        return _build.PKG_DIR / _build.LIB_NAME
    import hashlib
    import tempfile
    digest = hashlib.sha256()
    for src in sorted(_build.CSRC.glob("*.cu*")) + sorted(_build.INCLUDE.glob("*.h")):
        digest.update(src.read_bytes())
    out = Path(tempfile.gettempdir()) / f"dsa_b200_{digest.hexdigest()[:16]}"
    out.mkdir(parents=True, exist_ok=True)
    return out / _build.LIB_NAME


def load(build_if_missing: bool = True):
    """Load (building first when the sources are newer) and type the C ABI.  Raises on failure."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if build_if_missing and "DSA_B200_LIB" not in os.environ and _build.needs_build(path):
        _build.build(path)
    if not path.exists():
        raise RuntimeError(f"{path} is missing: run `python -m auto_gpu_kernel_b200.build`")
    lib = ctypes.CDLL(str(path))
    for name, (res, args) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as exc:
            raise RuntimeError(f"{path} does not export {name}") from exc
        fn.restype = res
        fn.argtypes = args
    if lib.dsa_b200_version() != 1:
        raise RuntimeError(f"{path}: ABI version {lib.dsa_b200_version()} != 1")
    _lib = lib
    return lib


def check(code: int, what: str):
    """Turn a non-zero return code of the C ABI into a RuntimeError."""
    if code != 0:
        text = load().dsa_b200_error_string(code).decode()
        raise RuntimeError(f"{what}: {text} (code {code})")
