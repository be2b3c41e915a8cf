"""The benchmark configurations at their full sizes, checked through size-independent properties
and against the oracle on a sample of rows (the oracle runs on the GPU in fp32 where the CPU would
take minutes)."""
import pytest
import torch

import dsa_oracle as oracle
from auto_gpu_kernel_b200 import indexer, inputs as wl, sparse_attention, workspace
from helpers import assert_attention_close

pytestmark = pytest.mark.gpu


def _check_rows_against_oracle(inp, out, rows):
    """Acceptance rule on selected requests; scores recomputed by the oracle on the GPU."""
    for b in rows:
        sub = wl.IndexerInputs(inp.q_index_fp8[b:b + 1], inp.k_index_cache_fp8, inp.weights[b:b + 1],
                               inp.seq_lens[b:b + 1], inp.block_table[b:b + 1])
        ref = oracle.indexer_scores(*sub.args())[0].cpu()
        info = oracle.check_topk_row(ref, inp.block_table[b].cpu(), int(inp.seq_lens[b]), out[b].cpu())
        assert info["ok"], f"request {b}: {info}"


def _check_structure(inp, out):
    """Every row: exactly min(2048, L) distinct ids that belong to the request's pages, then -1."""
    out = out.cpu()
    lens = inp.seq_lens.cpu()
    table = inp.block_table.cpu()
    for b in range(out.shape[0]):
        k = min(2048, int(lens[b]))
        row = out[b]
        valid = row[row >= 0]
        assert valid.numel() == k and torch.unique(valid).numel() == k, f"row {b}"
        pages = set(table[b, : (int(lens[b]) + 63) // 64].tolist())
        assert set((valid // 64).tolist()) <= pages, f"row {b}: slot outside the request"


def test_cfg1_attention_decode_t64_ctx8k_32k(cuda):
    lens = wl.uniform_lengths(64, 8192, 32768, seed=1)
    inp = wl.make_attention_inputs(lens, seed=1, device=cuda)
    out, lse = sparse_attention.run(*inp.args())
    workspace.check_status(cuda)
    ref_out, ref_lse = oracle.sparse_attention(*inp.args(), output=torch.empty_like(out),
                                               lse=torch.empty_like(lse))
    assert_attention_close(out, lse, ref_out.cpu(), ref_lse.cpu(), label="cfg1")
    # linearity property of the definition: the output does not depend on the order of the indices
    perm = torch.randperm(2048, device=cuda)
    out2, lse2 = sparse_attention.run(inp.q_nope, inp.q_pe, inp.ckv_cache, inp.kpe_cache,
                                      inp.sparse_indices[:, perm].contiguous(), inp.sm_scale)
    assert torch.allclose(lse2, lse, atol=1e-4, rtol=1e-4)
    assert torch.allclose(out2.float(), out.float(), atol=1e-2, rtol=1e-2)


def test_headline_indexer_b64_ctx32k(cuda):
    inp = wl.make_indexer_inputs([32768] * 64, seed=3, device=cuda)
    out = indexer.run(*inp.args())
    workspace.check_status(cuda)
    _check_structure(inp, out)
    _check_rows_against_oracle(inp, out, [0, 31, 63])


def test_cfg2_indexer_long_context_b256(cuda):
    lens = wl.uniform_lengths(256, 32768, 131072, seed=2)
    inp = wl.make_indexer_inputs(lens, seed=2, device=cuda)          # ~2.8 GB of key pages
    out = indexer.run(*inp.args())
    workspace.check_status(cuda)
    _check_structure(inp, out)
    longest = max(range(256), key=lambda b: lens[b])
    _check_rows_against_oracle(inp, out, [0, longest, 255])


def test_cfg3_chunked_prefill_indexer_and_attention(cuda):
    """One request: 16K prefix + 4096-token chunk; query row i sees the first 16384 + i + 1 tokens.
    All rows share one block_table row (stride 0)."""
    inp = wl.make_shared_prefix_indexer_inputs(prefix_len=16384, chunk_len=4096, seed=4, device=cuda)
    shared = inp.block_table[:1].expand(4096, -1)
    out = indexer.run(inp.q_index_fp8, inp.k_index_cache_fp8, inp.weights, inp.seq_lens, shared)
    workspace.check_status(cuda)
    # causality: row i only selects positions < 16384 + i + 1 (checked through the page remap)
    table = inp.block_table[0].cpu()
    inv = {int(p): n for n, p in enumerate(table.tolist())}
    for i in (0, 1, 2047, 4095):
        row = out[i].cpu()
        assert (row >= 0).all()
        local = torch.tensor([inv[int(s) // 64] * 64 + int(s) % 64 for s in row.tolist()])
        assert int(local.max()) < 16384 + i + 1 and torch.unique(local).numel() == 2048
    _check_rows_against_oracle(inp, out, [0, 2048, 4095])
    # sparse attention for the chunk's 4096 query tokens over the indices just produced
    pages = inp.k_index_cache_fp8.shape[0]
    gen = torch.Generator(device=cuda).manual_seed(8)
    ckv = torch.randn(pages, 64, 512, generator=gen, device=cuda).to(torch.bfloat16)
    kpe = torch.randn(pages, 64, 64, generator=gen, device=cuda).to(torch.bfloat16)
    qn = (torch.randn(4096, 16, 512, generator=gen, device=cuda) * 0.1).to(torch.bfloat16)
    qp = (torch.randn(4096, 16, 64, generator=gen, device=cuda) * 0.1).to(torch.bfloat16)
    o, l = sparse_attention.run(qn, qp, ckv, kpe, out, 192 ** -0.5)
    workspace.check_status(cuda)
    rows = torch.tensor([0, 1000, 4095], device=cuda)
    ro, rl = oracle.sparse_attention(qn[rows], qp[rows], ckv, kpe, out[rows], 192 ** -0.5)
    assert_attention_close(o[rows], l[rows], ro.cpu(), rl.cpu(), label="cfg3 attention")
