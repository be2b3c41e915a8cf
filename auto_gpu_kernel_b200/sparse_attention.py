"""Sparse MLA attention operator: same entry signature and tensor layouts as the reference's
`kernel(q_nope, q_pe, ckv_cache, kpe_cache, sparse_indices, sm_scale, output, lse)`
(archive/dsa_sparse_attention_h16_ckv512_kpe64_topk2048_ps64/solution/triton/sparse_baseline.py:12),
destination-passing style.  `run(...)` is the value-returning form.

All tensors must be CUDA tensors on one device; there is no CPU path.  A token whose indices are all
-1 gets output 0 and lse -inf (the reference's GPU kernels do the same; its PyTorch definition
yields NaN there).
"""
from __future__ import annotations

import torch

from . import _lib, workspace

HEADS = 16
CKV = 512
KPE = 64


def kernel(q_nope, q_pe, ckv_cache, kpe_cache, sparse_indices, sm_scale, output, lse, variant=0):
    """Write attention output and base-2 LSE in place; enqueued on the current stream, returns None.
    `variant` 0 = default (warp-level mma.sync) kernel, 1 = CUDA-core cross-check kernel, 2 =
    tcgen05/TMEM kernel (not part of the reference signature; positional callers never pass it)."""
    if not q_nope.is_cuda:
        raise RuntimeError("dsa sparse attention: CUDA tensors required (this operator has no CPU path)")
    dev = q_nope.device
    tokens = q_nope.shape[0]
    for name, t in (("q_pe", q_pe), ("ckv_cache", ckv_cache), ("kpe_cache", kpe_cache),
                    ("sparse_indices", sparse_indices), ("output", output), ("lse", lse)):
        if t.device != dev:
            raise RuntimeError(f"dsa sparse attention: {name} is on {t.device}, q_nope on {dev}")
    if q_nope.shape[1:] != (HEADS, CKV) or q_nope.dtype != torch.bfloat16:
        raise ValueError(f"q_nope must be [T,{HEADS},{CKV}] bf16, got {tuple(q_nope.shape)} {q_nope.dtype}")
    if q_pe.shape != (tokens, HEADS, KPE) or q_pe.dtype != torch.bfloat16:
        raise ValueError(f"q_pe must be [T,{HEADS},{KPE}] bf16")
    if ckv_cache.shape[-1] != CKV or ckv_cache.dtype != torch.bfloat16:
        raise ValueError("ckv_cache must be [..., 512] bf16")
    if kpe_cache.shape[-1] != KPE or kpe_cache.dtype != torch.bfloat16:
        raise ValueError("kpe_cache must be [..., 64] bf16")
    slots = ckv_cache.numel() // CKV
    if kpe_cache.numel() // KPE != slots:
        raise ValueError("ckv_cache and kpe_cache hold different numbers of slots")
    if sparse_indices.dim() != 2 or sparse_indices.shape[0] != tokens \
            or sparse_indices.dtype != torch.int32 or sparse_indices.stride(1) != 1:
        raise ValueError("sparse_indices must be [T,topk] int32 with dense rows")
    if output.shape != (tokens, HEADS, CKV) or output.dtype != torch.bfloat16 \
            or lse.shape != (tokens, HEADS) or lse.dtype != torch.float32:
        raise ValueError("output must be [T,16,512] bf16 and lse [T,16] float32")
    for name, t in (("q_nope", q_nope), ("q_pe", q_pe), ("ckv_cache", ckv_cache),
                    ("kpe_cache", kpe_cache), ("output", output), ("lse", lse)):
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
    if tokens == 0:
        return None
    topk = sparse_indices.shape[1]
    lib = _lib.load()
    need = lib.dsa_sparse_attn_workspace_bytes(tokens, HEADS, topk)
    ws = workspace.get(dev, "attention", need)
    with workspace.device_guard(dev):
        fn = (lib.dsa_sparse_attn, lib.dsa_sparse_attn_cuda_core, lib.dsa_sparse_attn_tcgen05)[variant]
        rc = fn(
            q_nope.data_ptr(), q_pe.data_ptr(), ckv_cache.data_ptr(), kpe_cache.data_ptr(),
            sparse_indices.data_ptr(), sparse_indices.stride(0), float(sm_scale),
            output.data_ptr(), lse.data_ptr(), tokens, HEADS, topk, slots, ws.data_ptr(),
            ws.numel(), workspace.status_word(dev).data_ptr(),
            workspace.stream_handle(dev))
    _lib.check(rc, "dsa_sparse_attn")
    return None


def run(q_nope, q_pe, ckv_cache, kpe_cache, sparse_indices, sm_scale, output=None, lse=None,
        variant=0):
    """Value-returning form: allocates the outputs that are not passed; returns (output, lse)."""
    tokens = q_nope.shape[0]
    if output is None:
        output = torch.empty(tokens, HEADS, CKV, dtype=torch.bfloat16, device=q_nope.device)
    if lse is None:
        lse = torch.empty(tokens, HEADS, dtype=torch.float32, device=q_nope.device)
    kernel(q_nope, q_pe, ckv_cache, kpe_cache, sparse_indices, sm_scale, output, lse, variant)
    return output, lse
