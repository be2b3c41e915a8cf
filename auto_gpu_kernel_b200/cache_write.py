"""Writers of the two paged caches the DSA path reads (the step before the path).

The reference ships no writer: its inputs arrive packed.  The layouts written here are the ones
its readers unpack -- index-key pages by `dequant_fp8_kv_cache`
(archive/dsa_topk_indexer_fp8_h64_d128_topk2048_ps64/solution/triton/indexer_baseline.py:16-36),
ckv/kpe rows by the flat views of
archive/dsa_sparse_attention_h16_ckv512_kpe64_topk2048_ps64/solution/triton/sparse_baseline.py:18-28.
CUDA tensors only; enqueued on the current stream.
"""
from __future__ import annotations

import torch

from . import _lib, workspace


def write_index_keys(keys, slots, k_index_cache_fp8):
    """Quantise `keys` [n,128] (fp32 or bf16) per token (absmax / 448, e4m3) and store token t at
    global slot `slots[t]` (page * 64 + position; -1 skips the token) of the packed
    [P,64,1,132] int8 cache."""
    if not keys.is_cuda:
        raise RuntimeError("dsa cache writer: CUDA tensors required (no CPU path)")
    if keys.dim() != 2 or keys.shape[1] != 128 or keys.dtype not in (torch.float32, torch.bfloat16):
        raise ValueError("keys must be [n,128] float32 or bfloat16")
    if keys.stride(1) != 1:
        raise ValueError("keys rows must be dense")
    if slots.shape != (keys.shape[0],) or slots.dtype != torch.int32 or not slots.is_contiguous():
        raise ValueError("slots must be a contiguous [n] int32 tensor")
    cache = k_index_cache_fp8
    if cache.dim() != 4 or cache.shape[1:] != (64, 1, 132) or cache.element_size() != 1 \
            or not cache.is_contiguous():
        raise ValueError("k_index_cache_fp8 must be a contiguous [P,64,1,132] int8 tensor")
    dev = keys.device
    lib = _lib.load()
    with workspace.device_guard(dev):
        rc = lib.dsa_index_cache_write(
            keys.data_ptr(), 0 if keys.dtype == torch.float32 else 1, keys.stride(0),
            slots.data_ptr(), cache.data_ptr(), keys.shape[0], cache.shape[0],
            workspace.status_word(dev).data_ptr(), workspace.stream_handle(dev))
    _lib.check(rc, "dsa_index_cache_write")


def append_kv(ckv, kpe, slots, ckv_cache, kpe_cache):
    """Store row t of `ckv` [n,512] / `kpe` [n,64] (bf16) at global slot `slots[t]` of the paged
    caches [P,64,512] / [P,64,64] (-1 skips the token)."""
    if not ckv.is_cuda:
        raise RuntimeError("dsa cache writer: CUDA tensors required (no CPU path)")
    n = ckv.shape[0]
    if ckv.shape != (n, 512) or kpe.shape != (n, 64) or ckv.dtype != torch.bfloat16 \
            or kpe.dtype != torch.bfloat16 or ckv.stride(1) != 1 or kpe.stride(1) != 1:
        raise ValueError("ckv must be [n,512] and kpe [n,64], bf16 with dense rows")
    if slots.shape != (n,) or slots.dtype != torch.int32 or not slots.is_contiguous():
        raise ValueError("slots must be a contiguous [n] int32 tensor")
    if ckv_cache.shape[-1] != 512 or kpe_cache.shape[-1] != 64 or not ckv_cache.is_contiguous() \
            or not kpe_cache.is_contiguous() or ckv_cache.dtype != torch.bfloat16 \
            or kpe_cache.dtype != torch.bfloat16:
        raise ValueError("caches must be contiguous bf16 [...,512] / [...,64]")
    num_slots = ckv_cache.numel() // 512
    if kpe_cache.numel() // 64 != num_slots:
        raise ValueError("ckv_cache and kpe_cache hold different numbers of slots")
    dev = ckv.device
    lib = _lib.load()
    with workspace.device_guard(dev):
        rc = lib.dsa_kv_cache_append(
            ckv.data_ptr(), ckv.stride(0), kpe.data_ptr(), kpe.stride(0), slots.data_ptr(),
            ckv_cache.data_ptr(), kpe_cache.data_ptr(), n, num_slots,
            workspace.status_word(dev).data_ptr(), workspace.stream_handle(dev))
    _lib.check(rc, "dsa_kv_cache_append")
