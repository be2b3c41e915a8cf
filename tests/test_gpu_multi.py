"""Two-GPU run of the head-sharded block with the CUDA operators and NCCL (skipped on one GPU)."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_path):
    for p in (ROOT, ROOT / "oracle"):
        if str(p) not in sys.path:
            sys.path.insert(0, str(p))
    import torch.distributed as dist
    from auto_gpu_kernel_b200 import dist as dsa_dist, indexer, inputs as wl, sparse_attention, workspace
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        lens = [3000, 2100, 70, 5000, 2500, 4097, 9000]
        batch = len(lens)
        block = wl.make_decode_block_inputs(lens, seed=9, device=dev, heads=16 * world)
        idx = block.indexer
        mine = dsa_dist.shard_range(batch, rank, world)
        counts = [len(dsa_dist.shard_range(batch, r, world)) for r in range(world)]
        sel = slice(mine.start, mine.stop)
        local_args = (idx.q_index_fp8[sel].contiguous(), idx.k_index_cache_fp8,
                      idx.weights[sel].contiguous(), idx.seq_lens[sel].contiguous(),
                      idx.block_table[sel].contiguous())
        heads = slice(16 * rank, 16 * rank + 16)
        qn, qp = block.q_nope[:, heads].contiguous(), block.q_pe[:, heads].contiguous()
        out = torch.empty(batch, 16, 512, dtype=torch.bfloat16, device=dev)
        lse = torch.empty(batch, 16, dtype=torch.float32, device=dev)
        gathered = dsa_dist.decode_block_head_sharded(local_args, counts, qn, qp, block.ckv_cache,
                                                      block.kpe_cache, block.sm_scale, out, lse)
        workspace.check_status(dev)
        # the same on one GPU, all requests at once
        want_idx = indexer.run(*idx.args())
        want_out, want_lse = sparse_attention.run(qn, qp, block.ckv_cache, block.kpe_cache, gathered,
                                                  block.sm_scale)
        same_sets = torch.equal(torch.sort(gathered, 1).values, torch.sort(want_idx, 1).values)
        ok = bool(same_sets and torch.equal(out.view(torch.int16), want_out.view(torch.int16))
                  and torch.equal(lse, want_lse))
        flags = [None] * world
        dist.all_gather_object(flags, ok)
        if rank == 0:
            Path(result_path).write_text("ok" if all(flags) else f"mismatch {flags}")
    finally:
        dist.destroy_process_group()


def test_head_sharded_block_on_two_gpus(tmp_path):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    result = tmp_path / "result.txt"
    mp.spawn(_worker, args=(2, _free_port(), str(result)), nprocs=2, join=True)
    assert result.read_text() == "ok"
