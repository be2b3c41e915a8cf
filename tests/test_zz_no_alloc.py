"""dsa_indexer_topk_noalloc: the indexer entry point for callers that cannot allocate device memory
(a serving loop whose memory pool is frozen, a plugin that may only touch the tensors it was handed,
a process whose allocator belongs to another runtime).  Its score scratch is a fixed array inside the
library, so the checks here are: same selection as the workspace-taking entry point, on two calls in
a row (the second call sees the first call's leftovers in the scratch), and a clean refusal beyond
the built-in capacity.  Collected last on purpose: a run that stops at the first failure has then
already run every other test."""
import pytest
import torch

import dsa_oracle as oracle
from auto_gpu_kernel_b200 import _lib, indexer, inputs as wl, workspace
from helpers import assert_topk_matches

pytestmark = pytest.mark.gpu

MAX_SCORES = 2 * 1024 * 1024          # DSA_NOALLOC_MAX_SCORES of include/dsa_b200.h
ERR_SCRATCH_TOO_SMALL = -6


def _call_noalloc(lib, inp, out):
    dev = inp.q_index_fp8.device
    status = workspace.status_word(dev)
    with torch.cuda.device(dev):
        return lib.dsa_indexer_topk_noalloc(
            inp.q_index_fp8.data_ptr(), inp.k_index_cache_fp8.data_ptr(), inp.weights.data_ptr(),
            inp.seq_lens.data_ptr(), inp.block_table.data_ptr(), inp.block_table.stride(0),
            out.data_ptr(), out.stride(0), inp.q_index_fp8.shape[0], inp.k_index_cache_fp8.shape[0],
            inp.block_table.shape[1], status.data_ptr(), torch.cuda.current_stream(dev).cuda_stream)


def test_noalloc_matches_workspace_entry_point_twice(cuda):
    lib = _lib.load()
    # two different batches back to back: the second runs over the first one's leftover scores
    for seed, lens in ((21, [5000, 2048, 0, 9000, 3000, 70]), (22, [2500, 12000, 4097])):
        inp = wl.make_indexer_inputs(lens, seed=seed, device=cuda)
        want = indexer.run(*inp.args())                      # entry point with caller workspace
        got = torch.full_like(want, 777)
        assert _call_noalloc(lib, inp, got) == 0
        workspace.check_status(cuda)
        # the selected SET is deterministic (bit-exact integer output up to order within a row)
        assert torch.equal(torch.sort(got, dim=1).values, torch.sort(want, dim=1).values)
        # and it stands on its own against the oracle (acceptance rule of the definition)
        rows = [r.cpu() for r in oracle.indexer_scores(*inp.args())]
        assert_topk_matches(inp, got, rows, label=f"noalloc seed {seed}")


def test_noalloc_rejects_sizes_beyond_its_scratch(cuda):
    lib = _lib.load()
    inp = wl.make_indexer_inputs([300, 200], seed=3, device=cuda)
    out = torch.empty(2, 2048, dtype=torch.int32, device=cuda)
    dev = inp.q_index_fp8.device
    # pretend a block table wide enough that batch x padded context exceeds the capacity
    too_wide = MAX_SCORES // (2 * 64) + 2
    with torch.cuda.device(dev):
        rc = lib.dsa_indexer_topk_noalloc(
            inp.q_index_fp8.data_ptr(), inp.k_index_cache_fp8.data_ptr(), inp.weights.data_ptr(),
            inp.seq_lens.data_ptr(), inp.block_table.data_ptr(), inp.block_table.stride(0),
            out.data_ptr(), out.stride(0), 2, inp.k_index_cache_fp8.shape[0], too_wide, None,
            torch.cuda.current_stream(dev).cuda_stream)
    assert rc == ERR_SCRATCH_TOO_SMALL
    assert b"scratch" in lib.dsa_b200_error_string(rc)
