"""Host-buffer decode step: slab layout on CPU, results against the plain operators on a GPU."""
import pytest
import torch

from auto_gpu_kernel_b200 import host_step


def test_slab_layout_is_aligned_and_disjoint():
    (a, na), (b, nb), (r, nr) = host_step.step_layout(batch=3, max_pages=5)
    for fields, total in ((a, na), (b, nb), (r, nr)):
        end = 0
        for f in fields:
            assert f.offset % host_step.ALIGN == 0
            assert f.offset >= end
            end = f.offset + f.nbytes
        assert total >= end and total % host_step.ALIGN == 0
    names = [f.name for f in a + b]
    assert names == ["q_index_fp8", "weights", "seq_lens", "block_table", "q_nope", "q_pe"]
    sizes = {f.name: f.nbytes for f in a + b + r}
    assert sizes["q_index_fp8"] == 3 * 64 * 128
    assert sizes["block_table"] == 3 * 5 * 4
    assert sizes["q_nope"] == 3 * 16 * 512 * 2
    assert sizes["topk_indices"] == 3 * 2048 * 4
    # output and lse precede the indices so that they leave in one copy
    assert [f.name for f in r] == ["output", "lse", "topk_indices"]


@pytest.mark.gpu
def test_host_step_matches_operators():
    from auto_gpu_kernel_b200 import indexer, sparse_attention, workspace, inputs as wl
    dev = torch.device("cuda", 0)
    lens = [5000, 64, 2049, 9000, 1, 3333]
    blk = wl.make_decode_block_inputs(lens, seed=11, device=dev)
    idx = blk.indexer
    step = host_step.HostDecodeStep(idx.k_index_cache_fp8, blk.ckv_cache, blk.kpe_cache,
                                    batch=len(lens), max_pages=idx.block_table.shape[1],
                                    sm_scale=blk.sm_scale)
    want_topk = indexer.run(*idx.args())
    want_out, want_lse = sparse_attention.run(blk.q_nope, blk.q_pe, blk.ckv_cache, blk.kpe_cache,
                                              want_topk, blk.sm_scale)
    torch.cuda.synchronize()
    for _ in range(2):   # the second call reuses the slabs
        topk, out, lse = step.run(idx.q_index_fp8.cpu(), idx.weights.cpu(), idx.seq_lens.cpu(),
                                  idx.block_table.cpu(), blk.q_nope.cpu(), blk.q_pe.cpu())
        assert not topk.is_cuda and topk.is_pinned()
        assert torch.equal(topk.sort(dim=1).values, want_topk.cpu().sort(dim=1).values)
        # the order of ids within a row may differ between two selections, and with it the
        # summation order: bit-exact against the operators run on the step's own ids, within the
        # attention tolerance against the first selection
        own_out, own_lse = sparse_attention.run(blk.q_nope, blk.q_pe, blk.ckv_cache, blk.kpe_cache,
                                                topk.to(dev), blk.sm_scale)
        assert torch.equal(out.view(torch.int16), own_out.cpu().view(torch.int16))
        assert torch.equal(lse, own_lse.cpu())
        torch.testing.assert_close(out.float(), want_out.cpu().float(), atol=1e-2, rtol=1e-2)
        torch.testing.assert_close(lse, want_lse.cpu(), atol=1e-3, rtol=1e-3)
        out.zero_()
    assert workspace.check_status(dev) == 0
    assert step.h2d_bytes == sum(t.numel() * t.element_size() for t in
                                 (idx.q_index_fp8, idx.weights, idx.seq_lens, idx.block_table,
                                  blk.q_nope, blk.q_pe))
