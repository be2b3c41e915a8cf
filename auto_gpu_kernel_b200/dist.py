"""Multi-GPU layouts of the DSA decode block (one process per GPU, torch.distributed).

The reference has no multi-GPU path; its attention definition only notes that 16 heads are one
tensor-parallel rank of a 128-head model (sparse_baseline.py:4-5).  Two layouts follow from the
data dependencies of the two definitions:

* request-sharded (`shard_range`, `decode_block_local`): requests are independent in both stages
  (indexer_baseline.py:62 loops over them), so every rank runs indexer -> attention on its own
  requests and its own cache pages.  No collective at all.
* head-sharded attention (`decode_block_head_sharded`): the indexer stays request-sharded, the
  attention of ALL tokens runs on every rank for that rank's 16 of the 128 heads, with the ckv/kpe
  caches replicated.  Every rank then needs every request's indices: one all-gather of the int32
  [B, 2048] index tensor (1 MiB at B = 128) is the only exchange step of the path.

The stage functions are parameters so that the orchestration can be exercised on CPU ranks (gloo)
with stand-ins; by default they are the CUDA operators of this package.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

TOPK = 2048
HEADS_PER_RANK = 16


def shard_range(total: int, rank: int, world: int) -> range:
    """Contiguous, balanced shard of `total` items: the first `total % world` ranks get one more."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world {rank}/{world}")
    base, extra = divmod(total, world)
    lo = rank * base + min(rank, extra)
    return range(lo, lo + base + (1 if rank < extra else 0))


def _default_ops():
    from . import indexer, sparse_attention
    return indexer.kernel, sparse_attention.kernel


def decode_block_local(idx_args, q_nope, q_pe, ckv_cache, kpe_cache, sm_scale, topk_indices, output,
                       lse, indexer_fn=None, attention_fn=None):
    """Request-sharded layout: the rank's own requests, no communication."""
    if indexer_fn is None or attention_fn is None:
        indexer_fn, attention_fn = _default_ops()
    indexer_fn(*idx_args, topk_indices)
    attention_fn(q_nope, q_pe, ckv_cache, kpe_cache, topk_indices, sm_scale, output, lse)
    return output, lse


def gather_indices(local_indices: torch.Tensor, counts, group=None) -> torch.Tensor:
    """All-gather of the per-rank index rows into the full [B, 2048] tensor (rank order).

    `counts[r]` is the number of requests of rank r.  Equal counts use one
    all_gather_into_tensor; ragged counts pad to the largest shard first."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return local_indices
    width = local_indices.shape[1]
    most = max(counts)
    if local_indices.shape[0] != most:
        pad = torch.full((most - local_indices.shape[0], width), -1, dtype=local_indices.dtype,
                         device=local_indices.device)
        local_indices = torch.cat([local_indices, pad], dim=0)
    gathered = torch.empty(world * most, width, dtype=local_indices.dtype, device=local_indices.device)
    dist.all_gather_into_tensor(gathered, local_indices.contiguous(), group=group)
    if all(c == most for c in counts):
        return gathered
    rows = [gathered[r * most: r * most + counts[r]] for r in range(world)]
    return torch.cat(rows, dim=0)


def decode_block_head_sharded(idx_args_local, counts, q_nope_heads, q_pe_heads, ckv_cache, kpe_cache,
                              sm_scale, output, lse, local_indices=None, group=None, indexer_fn=None,
                              attention_fn=None):
    """Head-sharded layout of the full 128-head block (128 heads = 8 ranks x 16).

    idx_args_local : indexer inputs of this rank's request shard (q, cache, weights, seq_lens,
                     block_table); the cache holds (at least) this shard's pages
    counts         : requests per rank, in rank order (sum = B)
    q_nope_heads   : [B, 16, 512] bf16, this rank's heads of ALL tokens; q_pe_heads likewise
    ckv/kpe caches : replicated, identical page numbering on every rank
    output, lse    : [B, 16, 512] bf16 / [B, 16] fp32 for this rank's heads
    Returns the gathered [B, 2048] index tensor.
    """
    if indexer_fn is None or attention_fn is None:
        indexer_fn, attention_fn = _default_ops()
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    if local_indices is None:
        local_indices = torch.empty(counts[rank], TOPK, dtype=torch.int32,
                                    device=q_nope_heads.device)
    indexer_fn(*idx_args_local, local_indices)
    all_indices = gather_indices(local_indices, counts, group)
    attention_fn(q_nope_heads, q_pe_heads, ckv_cache, kpe_cache, all_indices, sm_scale, output, lse)
    return all_indices
