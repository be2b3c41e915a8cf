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


def _push_worker(rank, world, port, result_path):
    """Head-sharded block with the index rows pushed by the library's own exchange kernel, three steps
    with changing inputs (both row buffers and growing epochs), ragged shards."""
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
        counts = [len(dsa_dist.shard_range(batch, r, world)) for r in range(world)]
        mine = dsa_dist.shard_range(batch, rank, world)
        sel = slice(mine.start, mine.stop)
        plan = dsa_dist.PeerPushPlan(counts, rank, dev)
        heads = slice(16 * rank, 16 * rank + 16)
        ok = True
        for step in range(3):
            block = wl.make_decode_block_inputs(lens, seed=20 + step, device=dev, heads=16 * world)
            idx = block.indexer
            local_args = (idx.q_index_fp8[sel].contiguous(), idx.k_index_cache_fp8,
                          idx.weights[sel].contiguous(), idx.seq_lens[sel].contiguous(),
                          idx.block_table[sel].contiguous())
            qn, qp = block.q_nope[:, heads].contiguous(), block.q_pe[:, heads].contiguous()
            out = torch.empty(batch, 16, 512, dtype=torch.bfloat16, device=dev)
            lse = torch.empty(batch, 16, dtype=torch.float32, device=dev)
            gathered = dsa_dist.decode_block_head_sharded(local_args, counts, qn, qp, block.ckv_cache,
                                                          block.kpe_cache, block.sm_scale, out, lse, plan=plan)
            workspace.check_status(dev)
            want_idx = indexer.run(*idx.args())
            want_out, want_lse = sparse_attention.run(qn, qp, block.ckv_cache, block.kpe_cache, gathered,
                                                      block.sm_scale)
            ok = ok and torch.equal(torch.sort(gathered, 1).values, torch.sort(want_idx, 1).values)
            ok = ok and torch.equal(out.view(torch.int16), want_out.view(torch.int16)) and torch.equal(lse, want_lse)
            ok = ok and plan.epoch == step + 1
        plan.close()
        flags = [None] * world
        dist.all_gather_object(flags, bool(ok))
        if rank == 0:
            Path(result_path).write_text("ok" if all(flags) else f"mismatch {flags}")
    finally:
        dist.destroy_process_group()


def _silent_peer_worker(rank, world, port, result_path):
    """Rank 1 takes part in step 1 and then stays silent (alive, its buffers mapped, but it neither
    selects nor sends); rank 0 runs step 2 alone with a poll limit of 50 ms.  Rank 0 must come back with
    DSA_STATUS_WAIT_TIMEOUT, its own rows intact, and a usable context; nothing hangs or faults."""
    for p in (ROOT, ROOT / "oracle"):
        if str(p) not in sys.path:
            sys.path.insert(0, str(p))
    import time
    import torch.distributed as dist
    from auto_gpu_kernel_b200 import dist as dsa_dist, indexer, inputs as wl, workspace
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        lens = [3000, 2100, 5000, 2500]
        counts = [2, 2]
        sel = slice(2 * rank, 2 * rank + 2)
        inp = wl.make_indexer_inputs(lens, seed=40, device=dev)
        args = (inp.q_index_fp8[sel].contiguous(), inp.k_index_cache_fp8, inp.weights[sel].contiguous(),
                inp.seq_lens[sel].contiguous(), inp.block_table[sel].contiguous())
        plan = dsa_dist.PeerPushPlan(counts, rank, dev, wait_limit_ns=50_000_000)
        want = indexer.run(*inp.args())
        plan.run_indexer(*args)
        rows = plan.gather().clone()
        workspace.check_status(dev)
        ok = torch.equal(torch.sort(rows, 1).values, torch.sort(want, 1).values)
        dist.barrier()
        outcome = "skipped"
        if rank == 0:
            t0 = time.perf_counter()
            plan.run_indexer(*args)
            plan.gather()
            torch.cuda.synchronize(dev)
            waited = time.perf_counter() - t0
            try:
                workspace.check_status(dev)
                outcome = "no timeout was reported"
            except RuntimeError as exc:
                outcome = "ok" if "0x1" in str(exc) and 0.04 < waited < 5.0 else f"unexpected: {exc} after {waited:.3f} s"
            mine = plan.all_rows[:2]
            if not torch.equal(torch.sort(mine, 1).values, torch.sort(want[:2], 1).values):
                outcome = "own rows damaged"
            # the context is still good for ordinary work
            again = indexer.run(*inp.args())
            workspace.check_status(dev)
            if not torch.equal(torch.sort(again, 1).values, torch.sort(want, 1).values):
                outcome = "context unusable after the timeout"
        dist.barrier()            # rank 1 has stayed alive (its buffers mapped) until rank 0 is done
        plan.close()
        if rank == 0:
            Path(result_path).write_text(outcome if ok else "step 1 mismatch")
    finally:
        dist.destroy_process_group()


def test_silent_peer_ends_in_a_timeout_status(tmp_path):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    result = tmp_path / "result.txt"
    mp.spawn(_silent_peer_worker, args=(2, _free_port(), str(result)), nprocs=2, join=True)
    assert result.read_text() == "ok"


def test_head_sharded_block_with_pushed_rows_on_two_gpus(tmp_path):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    result = tmp_path / "result.txt"
    mp.spawn(_push_worker, args=(2, _free_port(), str(result)), nprocs=2, join=True)
    assert result.read_text() == "ok"


def test_row_exchange_two_ranks_in_turn_on_one_gpu(cuda):
    """The exchange kernel with both ranks' buffers on one GPU, the ranks called one after the other
    (never at the same time): rank 1 pushes and, with rank 0 silent, its poll runs out after the
    2 ms it was given and reports DSA_STATUS_WAIT_TIMEOUT, leaving rank 0's rows as they were;
    rank 0 then pushes and finds rank 1's rows already there; rank 1, called again, now finds
    rank 0's.  A second epoch through the same staging buffers must not be satisfied by the first."""
    import ctypes
    for p in (ROOT, ROOT / "oracle"):
        if str(p) not in sys.path:
            sys.path.insert(0, str(p))
    from auto_gpu_kernel_b200 import _lib, workspace
    lib = _lib.load()
    counts, width = [5, 3], 2048
    total = sum(counts)
    gen = torch.Generator(device=cuda).manual_seed(5)
    status = workspace.status_word(cuda)
    stage = [torch.zeros(total, width, 2, dtype=torch.int32, device=cuda) for _ in range(2)]
    stage_ptrs = (ctypes.c_void_p * 2)(stage[0].data_ptr(), stage[1].data_ptr())
    rows = [torch.full((total, width), -7, dtype=torch.int32, device=cuda) for _ in range(2)]

    def call(rank, epoch, limit_ns=2_000_000):
        offset = sum(counts[:rank])
        rc = lib.dsa_index_rows_exchange(rows[rank].data_ptr(), ctypes.addressof(stage_ptrs), 2, rank,
                                         counts[rank], offset, total, width, width, epoch, 3, limit_ns,
                                         status.data_ptr(), workspace.stream_handle(cuda))
        _lib.check(rc, "dsa_index_rows_exchange")

    for epoch in (1, 2):
        truth = torch.randint(-1, 1 << 20, (total, width), dtype=torch.int32, device=cuda, generator=gen)
        before = rows[1][:5].clone()
        rows[0][:5] = truth[:5]
        rows[1][5:] = truth[5:]
        call(1, epoch)
        with pytest.raises(RuntimeError, match="0x1"):
            workspace.check_status(cuda)
        assert torch.equal(rows[1][:5], before)            # nothing taken: rank 0 has not sent this epoch
        assert torch.equal(stage[0][5:, :, 0], truth[5:]) and (stage[0][5:, :, 1] == epoch).all()
        call(0, epoch)
        assert workspace.check_status(cuda) == 0
        assert torch.equal(rows[0], truth)
        call(1, epoch)
        assert workspace.check_status(cuda) == 0
        assert torch.equal(rows[1], truth)
    # argument checks
    bad = lib.dsa_index_rows_exchange(rows[0].data_ptr(), ctypes.addressof(stage_ptrs), 9, 0, 1, 0, 8, width, width,
                                      1, 3, 1000, status.data_ptr(), None)
    assert bad < 0
    bad = lib.dsa_index_rows_exchange(rows[0].data_ptr(), ctypes.addressof(stage_ptrs), 2, 0, 5, 0, 8, width, width,
                                      0, 3, 1000, status.data_ptr(), None)
    assert bad < 0
    bad = lib.dsa_index_rows_exchange(rows[0].data_ptr(), ctypes.addressof(stage_ptrs), 2, 0, 5, 0, 8, width, width,
                                      1, 0, 1000, status.data_ptr(), None)
    assert bad < 0


@pytest.mark.parametrize("path", ["hist", "minmax"])
def test_selection_sends_its_rows(cuda, monkeypatch, path):
    """dsa_indexer_topk_send with the "peer" buffer on the same GPU: after the call the peer's staging
    rows [offset, offset + B) hold (id, epoch) pairs of exactly the rows the indexer returned --
    sent by the selection kernel itself on the histogram path (long and short rows, a row longer
    than one CTA's slice), by the push-only pass on the other -- and nothing else was touched; the
    take-only exchange on the "peer" then finds them."""
    import ctypes
    for p in (ROOT, ROOT / "oracle"):
        if str(p) not in sys.path:
            sys.path.insert(0, str(p))
    from auto_gpu_kernel_b200 import _lib, indexer, inputs as wl, workspace
    from helpers import assert_topk_matches
    monkeypatch.setenv("DSA_INDEXER_PATH", path)
    lens = [3000, 70, 2049, 50000, 2048, 9000]
    inp = wl.make_indexer_inputs(lens, seed=31, device=cuda)
    batch, offset, total, epoch = len(lens), 3, 12, 7
    stage = [torch.zeros(total, 2048, 2, dtype=torch.int32, device=cuda) for _ in range(2)]
    stage_ptrs = (ctypes.c_void_p * 2)(stage[0].data_ptr(), stage[1].data_ptr())
    rows = torch.full((total, 2048), -9, dtype=torch.int32, device=cuda)     # rank 0's index tensor
    indexer.kernel(*inp.args(), rows[offset:offset + batch],
                   send=(ctypes.addressof(stage_ptrs), 2, 0, offset, epoch))
    workspace.check_status(cuda)
    assert_topk_matches(inp, rows[offset:offset + batch], label=f"{path}: local rows")
    assert torch.equal(stage[1][offset:offset + batch, :, 0], rows[offset:offset + batch])
    assert (stage[1][offset:offset + batch, :, 1] == epoch).all()
    assert int(stage[1][:offset].abs().sum()) == 0 and int(stage[1][offset + batch:].abs().sum()) == 0
    assert int(stage[0].abs().sum()) == 0                                   # nothing is sent to oneself
    # the peer (rank 1, no rows of its own in this test) takes them
    peer_rows = torch.full((total, 2048), -9, dtype=torch.int32, device=cuda)
    lib = _lib.load()
    rc = lib.dsa_index_rows_exchange(peer_rows.data_ptr(), ctypes.addressof(stage_ptrs), 2, 1, 0, total, total,
                                     2048, 2048, epoch, 2, 2_000_000, workspace.status_word(cuda).data_ptr(),
                                     workspace.stream_handle(cuda))
    _lib.check(rc, "dsa_index_rows_exchange")
    with pytest.raises(RuntimeError, match="0x1"):       # rows outside [offset, offset + B) never arrive
        workspace.check_status(cuda)
    assert torch.equal(peer_rows[offset:offset + batch], rows[offset:offset + batch])
    assert (peer_rows[:offset] == -9).all() and (peer_rows[offset + batch:] == -9).all()


def test_head_sharded_block_on_two_gpus(tmp_path):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    result = tmp_path / "result.txt"
    mp.spawn(_worker, args=(2, _free_port(), str(result)), nprocs=2, join=True)
    assert result.read_text() == "ok"


def test_one_process_drives_two_gpus(cuda):
    """The C ABI may be called for several devices from one process: kernel attributes (the
    opt-in to large dynamic shared memory) and the SM count are kept per device, so the first
    launch on cuda:1 after calls on cuda:0 works like the first launch on cuda:0."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    for p in (ROOT, ROOT / "oracle"):
        if str(p) not in sys.path:
            sys.path.insert(0, str(p))
    import dsa_oracle as oracle
    from auto_gpu_kernel_b200 import indexer, inputs as wl, sparse_attention, workspace
    from helpers import assert_attention_close, assert_topk_matches
    lens = [3000, 2100, 70, 5000]
    results = []
    for index in (0, 1, 0):
        dev = torch.device("cuda", index)
        block = wl.make_decode_block_inputs(lens, seed=12, device=dev)
        idx = block.indexer
        topk = indexer.run(*idx.args())
        scores = indexer.scores(*idx.args(), variant=0)
        out, lse = sparse_attention.run(block.q_nope, block.q_pe, block.ckv_cache, block.kpe_cache,
                                        topk, block.sm_scale)
        out_tc, lse_tc = sparse_attention.run(block.q_nope, block.q_pe, block.ckv_cache, block.kpe_cache,
                                              topk, block.sm_scale, variant=2)
        workspace.check_status(dev)
        assert topk.device == dev and out.device == dev and scores.device == dev
        assert_topk_matches(idx, topk, label=f"cuda:{index}")
        ref_out, ref_lse = oracle.sparse_attention(block.q_nope.cpu(), block.q_pe.cpu(), block.ckv_cache.cpu(),
                                                   block.kpe_cache.cpu(), topk.cpu(), block.sm_scale)
        assert_attention_close(out, lse, ref_out, ref_lse, label=f"cuda:{index}")
        assert_attention_close(out_tc, lse_tc, ref_out, ref_lse, label=f"cuda:{index} tcgen05")
        results.append(torch.sort(topk.cpu(), dim=1).values)
    assert torch.equal(results[0], results[1]) and torch.equal(results[0], results[2])


def _prefill_worker(rank, world, port, result_path):
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
        chunk = 150
        inp = wl.make_shared_prefix_indexer_inputs(prefix_len=4000, chunk_len=chunk, seed=14, device=dev)
        pages = inp.k_index_cache_fp8.shape[0]
        gen = torch.Generator(device=dev).manual_seed(15)
        ckv = torch.randn(pages, 64, 512, generator=gen, device=dev).to(torch.bfloat16)
        kpe = torch.randn(pages, 64, 64, generator=gen, device=dev).to(torch.bfloat16)
        qn = (torch.randn(chunk, 16, 512, generator=gen, device=dev) * 0.1).to(torch.bfloat16)
        qp = (torch.randn(chunk, 16, 64, generator=gen, device=dev) * 0.1).to(torch.bfloat16)
        mine, topk, out, lse = dsa_dist.prefill_block_token_sharded(inp.args(), qn, qp, ckv, kpe, 192 ** -0.5,
                                                                    rank, world)
        workspace.check_status(dev)
        # the whole chunk on this GPU alone
        shared = inp.block_table[:1].expand(chunk, -1)
        want_idx = indexer.run(inp.q_index_fp8, inp.k_index_cache_fp8, inp.weights, inp.seq_lens, shared)
        sel = slice(mine.start, mine.stop)
        want_out, want_lse = sparse_attention.run(qn[sel].contiguous(), qp[sel].contiguous(), ckv, kpe, topk,
                                                  192 ** -0.5)
        ok = bool(torch.equal(torch.sort(topk, 1).values, torch.sort(want_idx[sel], 1).values)
                  and torch.equal(out.view(torch.int16), want_out.view(torch.int16))
                  and torch.equal(lse, want_lse))
        flags = [None] * world
        dist.all_gather_object(flags, ok)
        if rank == 0:
            Path(result_path).write_text("ok" if all(flags) else f"mismatch {flags}")
    finally:
        dist.destroy_process_group()


def test_token_sharded_prefill_on_two_gpus(tmp_path):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    result = tmp_path / "result.txt"
    mp.spawn(_prefill_worker, args=(2, _free_port(), str(result)), nprocs=2, join=True)
    assert result.read_text() == "ok"
