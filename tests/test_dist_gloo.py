"""The multi-GPU orchestration on two CPU ranks (gloo): request sharding, the all-gather of the index
rows (equal and ragged shards) and the head-sharded attention call sequence.  The two stage
functions are replaced by the CPU oracle here; the CUDA operators are covered by the gpu tests."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
for p in (ROOT, ROOT / "oracle"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))

from auto_gpu_kernel_b200 import dist as dsa_dist  # noqa: E402
from auto_gpu_kernel_b200 import inputs as wl  # noqa: E402


def test_shard_range_is_balanced_and_complete():
    for total in (0, 1, 5, 64, 127, 128):
        for world in (1, 2, 3, 8):
            parts = [dsa_dist.shard_range(total, r, world) for r in range(world)]
            assert [i for p in parts for i in p] == list(range(total))
            assert max(len(p) for p in parts) - min(len(p) for p in parts) <= 1
    with pytest.raises(ValueError):
        dsa_dist.shard_range(4, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, lens, result_path):
    import dsa_oracle as oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(2)
        batch = len(lens)
        block = wl.make_decode_block_inputs(lens, seed=5, heads=16 * world)   # same on every rank
        idx = block.indexer
        mine = dsa_dist.shard_range(batch, rank, world)
        counts = [len(dsa_dist.shard_range(batch, r, world)) for r in range(world)]
        sel = slice(mine.start, mine.stop)
        local_args = (idx.q_index_fp8[sel], idx.k_index_cache_fp8, idx.weights[sel], idx.seq_lens[sel],
                      idx.block_table[sel])
        heads = slice(16 * rank, 16 * rank + 16)
        out = torch.empty(batch, 16, 512, dtype=torch.bfloat16)
        lse = torch.empty(batch, 16, dtype=torch.float32)

        def indexer_fn(q, cache, w, sl, bt, topk):
            oracle.indexer_topk(q, cache, w, sl, bt, topk_indices=topk)

        def attention_fn(qn, qp, ckv, kpe, ind, scale, o, l):
            oracle.sparse_attention(qn, qp, ckv, kpe, ind, scale, output=o, lse=l)

        gathered = dsa_dist.decode_block_head_sharded(
            local_args, counts, block.q_nope[:, heads].contiguous(), block.q_pe[:, heads].contiguous(),
            block.ckv_cache, block.kpe_cache, block.sm_scale, out, lse,
            indexer_fn=indexer_fn, attention_fn=attention_fn)
        # single-process answer for the whole batch and this rank's heads
        want_idx = oracle.indexer_topk(*idx.args())
        want_out, want_lse = oracle.sparse_attention(block.q_nope[:, heads], block.q_pe[:, heads],
                                                     block.ckv_cache, block.kpe_cache, want_idx,
                                                     block.sm_scale)
        ok = bool(torch.equal(gathered, want_idx) and torch.equal(lse, want_lse)
                  and torch.equal(out.view(torch.int16), want_out.view(torch.int16)))
        flags = [None] * world
        dist.all_gather_object(flags, ok)
        if rank == 0:
            Path(result_path).write_text("ok" if all(flags) else f"mismatch {flags}")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("lens", [[300, 2100, 64, 2500], [100, 2300, 70, 2049, 1]],
                         ids=["equal_shards", "ragged_shards"])
def test_head_sharded_block_on_two_gloo_ranks(tmp_path, lens):
    result = tmp_path / "result.txt"
    mp.spawn(_worker, args=(2, _free_port(), lens, str(result)), nprocs=2, join=True)
    assert result.read_text() == "ok"


def _prefill_worker(rank, world, port, result_path):
    import dsa_oracle as oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(2)
        chunk = 7                                                     # not divisible by the world size
        inp = wl.make_shared_prefix_indexer_inputs(prefix_len=2300, chunk_len=chunk, seed=9)
        att = wl.make_attention_inputs([2400] * chunk, seed=9)       # queries and caches only
        pages = inp.k_index_cache_fp8.shape[0]
        ckv, kpe = att.ckv_cache[:pages], att.kpe_cache[:pages]
        calls = []

        def indexer_fn(q, cache, w, sl, bt, topk):
            calls.append(bt.stride(0))
            oracle.indexer_topk(q, cache, w, sl, bt.contiguous(), topk_indices=topk)

        def attention_fn(qn, qp, c, k, ind, scale, o, l):
            oracle.sparse_attention(qn, qp, c, k, ind, scale, output=o, lse=l)

        mine, topk, out, lse = dsa_dist.prefill_block_token_sharded(
            inp.args(), att.q_nope, att.q_pe, ckv, kpe, att.sm_scale, rank, world,
            indexer_fn=indexer_fn, attention_fn=attention_fn)
        want_idx = oracle.indexer_topk(*inp.args())
        want_out, want_lse = oracle.sparse_attention(att.q_nope, att.q_pe, ckv, kpe, want_idx, att.sm_scale)
        sel = slice(mine.start, mine.stop)
        ok = bool(calls == [0] and torch.equal(topk, want_idx[sel]) and torch.equal(lse, want_lse[sel])
                  and torch.equal(out.view(torch.int16), want_out[sel].view(torch.int16)))
        # the shards of all ranks tile the chunk
        spans = [None] * world
        dist.all_gather_object(spans, (mine.start, mine.stop, ok))
        if rank == 0:
            tiled = [i for a, b, _ in spans for i in range(a, b)] == list(range(chunk))
            Path(result_path).write_text("ok" if tiled and all(s[2] for s in spans) else f"mismatch {spans}")
    finally:
        dist.destroy_process_group()


def test_token_sharded_prefill_on_two_gloo_ranks(tmp_path):
    result = tmp_path / "result.txt"
    mp.spawn(_prefill_worker, args=(2, _free_port(), str(result)), nprocs=2, join=True)
    assert result.read_text() == "ok"


def _plan_worker(rank, world, port, result_path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ok = True
        for counts in ([3, 3], [3, 2]):
            plan = dsa_dist.HeadShardedPlan(counts, rank, torch.device("cpu"), width=8)
            ptr = plan.all_rows.data_ptr()
            for step in range(2):                                   # the same buffers every step
                plan.local_rows.copy_(torch.full((counts[rank], 8), 10 * step + rank, dtype=torch.int32))
                rows = plan.gather()
                want = torch.cat([torch.full((c, 8), 10 * step + r, dtype=torch.int32)
                                  for r, c in enumerate(counts)])
                ok = ok and torch.equal(rows, want) and rows.data_ptr() == ptr
        flags = [None] * world
        dist.all_gather_object(flags, bool(ok))
        if rank == 0:
            Path(result_path).write_text("ok" if all(flags) else f"mismatch {flags}")
    finally:
        dist.destroy_process_group()


def test_head_sharded_plan_reuses_its_buffers(tmp_path):
    result = tmp_path / "result.txt"
    mp.spawn(_plan_worker, args=(2, _free_port(), str(result)), nprocs=2, join=True)
    assert result.read_text() == "ok"


def test_peer_push_plan_refuses_cpu_ranks():
    """The pushed exchange is a CUDA kernel over NVLink: on CPU ranks the plan says so instead of
    falling back to anything (the all-gather plan is the one for other process groups)."""
    import pytest
    from auto_gpu_kernel_b200 import dist as dsa_dist
    with pytest.raises(RuntimeError, match="CUDA"):
        dsa_dist.PeerPushPlan([2, 2], 0, "cpu")
