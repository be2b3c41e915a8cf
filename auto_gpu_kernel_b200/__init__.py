"""B200 (sm_100a) implementation of the DeepSeek Sparse Attention hot path: the FP8 top-k indexer
and sparse MLA attention, behind the entry signatures of the reference's two `kernel(...)`
definitions.  The compute lives in libdsa_b200.so (hand-written CUDA, C ABI in include/dsa_b200.h);
this package is the thin PyTorch-facing host side."""

from . import indexer, sparse_attention, workspace  # noqa: F401
from .workspace import check_status  # noqa: F401

__all__ = ["indexer", "sparse_attention", "workspace", "check_status"]
