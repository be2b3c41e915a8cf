"""FP8 top-k indexer operator: same entry signature and tensor layouts as the reference's
`kernel(q_index_fp8, k_index_cache_fp8, weights, seq_lens, block_table, topk_indices)`
(archive/dsa_topk_indexer_fp8_h64_d128_topk2048_ps64/solution/triton/indexer_baseline.py:39-51),
destination-passing style as flashinfer-bench calls it.  `run(...)` is the value-returning form.

All tensors must be CUDA tensors on one device; there is no CPU path.
"""
from __future__ import annotations

import torch

from . import _lib, workspace

TOPK = 2048
HEADS = 64
DIM = 128
PAGE = 64


def _check(q, cache, weights, seq_lens, block_table):
    if not q.is_cuda:
        raise RuntimeError("dsa indexer: CUDA tensors required (this operator has no CPU path)")
    dev = q.device
    for name, t in (("k_index_cache_fp8", cache), ("weights", weights), ("seq_lens", seq_lens),
                    ("block_table", block_table)):
        if t.device != dev:
            raise RuntimeError(f"dsa indexer: {name} is on {t.device}, q_index_fp8 on {dev}")
    batch = q.shape[0]
    if q.shape[1:] != (HEADS, DIM) or q.element_size() != 1:
        raise ValueError(f"q_index_fp8 must be [B,{HEADS},{DIM}] fp8, got {tuple(q.shape)} {q.dtype}")
    if cache.dim() != 4 or cache.shape[1:] != (PAGE, 1, DIM + 4) or cache.element_size() != 1:
        raise ValueError(f"k_index_cache_fp8 must be [P,{PAGE},1,{DIM + 4}] int8, got {tuple(cache.shape)}")
    if weights.shape != (batch, HEADS) or weights.dtype != torch.float32:
        raise ValueError("weights must be [B,64] float32")
    if seq_lens.shape != (batch,) or seq_lens.dtype != torch.int32:
        raise ValueError("seq_lens must be [B] int32")
    if block_table.dim() != 2 or block_table.shape[0] != batch or block_table.dtype != torch.int32:
        raise ValueError("block_table must be [B,max_pages] int32")
    if not (q.is_contiguous() and cache.is_contiguous() and weights.is_contiguous()
            and seq_lens.is_contiguous()):
        raise ValueError("q_index_fp8, k_index_cache_fp8, weights and seq_lens must be contiguous")
    if block_table.shape[1] > 1 and block_table.stride(1) != 1:
        raise ValueError("block_table rows must be dense (stride(1) == 1)")


def kernel(q_index_fp8, k_index_cache_fp8, weights, seq_lens, block_table, topk_indices, send=None):
    """Write the top-2048 global slot ids of every request into `topk_indices` ([B,2048] int32,
    -1 padded).  Enqueued on the current stream; returns None without synchronising.

    `send` (head-sharded layers only, see `dist.PeerPushPlan`): (address of the host array of the
    peers' staging buffers, world, rank, row_offset, epoch) -- every finished row is then also
    stored into the peers' memory (`dsa_indexer_topk_send`)."""
    _check(q_index_fp8, k_index_cache_fp8, weights, seq_lens, block_table)
    batch = q_index_fp8.shape[0]
    if topk_indices.shape != (batch, TOPK) or topk_indices.dtype != torch.int32 \
            or topk_indices.stride(1) != 1 or topk_indices.device != q_index_fp8.device:
        raise ValueError("topk_indices must be a [B,2048] int32 tensor with dense rows on the same device")
    if batch == 0:
        return None
    lib = _lib.load()
    dev = q_index_fp8.device
    max_pages = block_table.shape[1]
    if max_pages == 0:
        topk_indices.fill_(-1)
        return None
    need = lib.dsa_indexer_workspace_bytes(batch, max_pages)
    ws = workspace.get(dev, "indexer", need)
    status = workspace.status_word(dev)
    with workspace.device_guard(dev):
        if send is None:
            rc = lib.dsa_indexer_topk(
                q_index_fp8.data_ptr(), k_index_cache_fp8.data_ptr(), weights.data_ptr(),
                seq_lens.data_ptr(), block_table.data_ptr(), block_table.stride(0),
                topk_indices.data_ptr(), topk_indices.stride(0), batch, k_index_cache_fp8.shape[0],
                max_pages, ws.data_ptr(), ws.numel(), status.data_ptr(),
                workspace.stream_handle(dev))
        else:
            stage_array, world, rank, row_offset, epoch = send
            rc = lib.dsa_indexer_topk_send(
                q_index_fp8.data_ptr(), k_index_cache_fp8.data_ptr(), weights.data_ptr(),
                seq_lens.data_ptr(), block_table.data_ptr(), block_table.stride(0),
                topk_indices.data_ptr(), topk_indices.stride(0), batch, k_index_cache_fp8.shape[0],
                max_pages, ws.data_ptr(), ws.numel(), stage_array, world, rank, row_offset, epoch,
                status.data_ptr(), workspace.stream_handle(dev))
    _lib.check(rc, "dsa_indexer_topk" if send is None else "dsa_indexer_topk_send")
    return None


def run(q_index_fp8, k_index_cache_fp8, weights, seq_lens, block_table, topk_indices=None):
    """Value-returning form: allocates the output when it is not passed."""
    if topk_indices is None:
        topk_indices = torch.empty(q_index_fp8.shape[0], TOPK, dtype=torch.int32,
                                   device=q_index_fp8.device)
    kernel(q_index_fp8, k_index_cache_fp8, weights, seq_lens, block_table, topk_indices)
    return topk_indices


def scores(q_index_fp8, k_index_cache_fp8, weights, seq_lens, block_table, variant=0, out=None):
    """Stage 1 alone: fp32 score rows [B, max_pages*64]; entries at or beyond seq_len are left as
    they were (NaN-filled when `out` is allocated here).  variant 0 = tcgen05, 1 = CUDA-core."""
    _check(q_index_fp8, k_index_cache_fp8, weights, seq_lens, block_table)
    batch, max_pages = q_index_fp8.shape[0], block_table.shape[1]
    width = (max_pages * PAGE + 127) // 128 * 128
    if out is None:
        out = torch.full((batch, width), float("nan"), dtype=torch.float32, device=q_index_fp8.device)
    lib = _lib.load()
    dev = q_index_fp8.device
    with workspace.device_guard(dev):
        rc = lib.dsa_indexer_scores(
            q_index_fp8.data_ptr(), k_index_cache_fp8.data_ptr(), weights.data_ptr(),
            seq_lens.data_ptr(), block_table.data_ptr(), block_table.stride(0), out.data_ptr(),
            out.stride(0), batch, k_index_cache_fp8.shape[0], max_pages, variant,
            workspace.status_word(dev).data_ptr(), workspace.stream_handle(dev))
    _lib.check(rc, "dsa_indexer_scores")
    return out


def select(score_rows, seq_lens, block_table, topk_indices=None):
    """Stage 2 alone: top-2048 + page remap over given fp32 score rows."""
    batch = score_rows.shape[0]
    if topk_indices is None:
        topk_indices = torch.empty(batch, TOPK, dtype=torch.int32, device=score_rows.device)
    lib = _lib.load()
    dev = score_rows.device
    with workspace.device_guard(dev):
        rc = lib.dsa_topk_select(
            score_rows.data_ptr(), score_rows.stride(0), seq_lens.data_ptr(), block_table.data_ptr(),
            block_table.stride(0), topk_indices.data_ptr(), topk_indices.stride(0), batch,
            block_table.shape[1], workspace.status_word(dev).data_ptr(),
            workspace.stream_handle(dev))
    _lib.check(rc, "dsa_topk_select")
    return topk_indices
