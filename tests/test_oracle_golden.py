"""The CPU oracle against the fixtures produced by the reference's own PyTorch definitions
(tests/golden/make_golden.py).  Runs without a GPU."""
import numpy as np
import pytest
import torch

import dsa_oracle as oracle
from helpers import (assert_attention_close, assert_topk_matches, load_attention_golden,
                     load_indexer_golden)


def test_e4m3_table_matches_torch_cast():
    codes = torch.arange(256, dtype=torch.uint8)
    ref = codes.view(torch.float8_e4m3fn).to(torch.float32).numpy()
    mine = oracle.e4m3fn_table()
    nan = np.isnan(ref)
    assert np.array_equal(np.isnan(mine), nan)
    assert np.array_equal(mine[~nan], ref[~nan])


@pytest.mark.parametrize("name", ["indexer_cfg0", "indexer_edges"])
def test_page_unpack_matches_reference_dequant(name):
    inp, _, z = load_indexer_golden(name)
    dense = oracle.dequant_index_pages(inp.k_index_cache_fp8)
    assert torch.equal(dense[0], torch.from_numpy(z["dequant_page0"]))
    assert torch.equal(dense[-1], torch.from_numpy(z["dequant_last"]))
    # table decode == torch decode on the raw bytes
    raw = inp.k_index_cache_fp8.view(torch.uint8).reshape(-1, oracle.PAGE_BYTES)[:, :oracle.PAGE_DATA_BYTES]
    data, _ = oracle.unpack_index_pages(inp.k_index_cache_fp8)
    assert np.array_equal(oracle.e4m3fn_table()[raw.numpy()].reshape(data.shape), data.numpy())


@pytest.mark.parametrize("name", ["indexer_cfg0", "indexer_edges"])
def test_indexer_oracle_reproduces_reference_indices(name):
    inp, golden_idx, _ = load_indexer_golden(name)
    mine, rows = oracle.indexer_topk(*inp.args(), return_scores=True)
    # structure is exact: same number of valid ids per row, -1 tail
    assert torch.equal((mine >= 0).sum(1), (golden_idx >= 0).sum(1))
    expect = torch.minimum(inp.seq_lens, torch.tensor(oracle.TOPK)).to(torch.int64)
    assert torch.equal((golden_idx >= 0).sum(1), expect)
    # the golden (reference) output satisfies the acceptance rule against oracle scores and vice versa
    assert_topk_matches(inp, golden_idx, rows, label=f"{name}/reference")
    assert_topk_matches(inp, mine, rows, label=f"{name}/oracle")
    for b in range(mine.shape[0]):
        assert set(mine[b].tolist()) == set(golden_idx[b].tolist())


@pytest.mark.parametrize("name", ["attention_small", "attention_padded"])
def test_attention_oracle_reproduces_reference(name):
    inp, ref_out, ref_lse = load_attention_golden(name)
    out, lse = oracle.sparse_attention(*inp.args())
    blank = torch.isinf(ref_lse)
    assert torch.equal(torch.isinf(lse), blank)
    assert torch.allclose(lse[~blank], ref_lse[~blank], atol=1e-5, rtol=1e-5)
    assert torch.equal(torch.isnan(out.float()), torch.isnan(ref_out.float()))
    keep = ~torch.isnan(ref_out.float())
    assert torch.allclose(out.float()[keep], ref_out.float()[keep], atol=1e-2, rtol=1e-2)
    # bf16 outputs should agree to the last bit almost everywhere (same ops, same order)
    same = (out.view(torch.int16)[keep] == ref_out.view(torch.int16)[keep]).float().mean()
    assert same > 0.99


def test_check_topk_row_classifier():
    scores = torch.arange(4000, dtype=torch.float32)            # wide gaps: exact mode
    table = torch.arange(64, dtype=torch.int32)
    want = torch.arange(4000 - 2048, 4000, dtype=torch.int32)
    assert oracle.check_topk_row(scores, table, 4000, want)["ok"]
    bad = want.clone(); bad[0] = 0
    assert not oracle.check_topk_row(scores, table, 4000, bad)["ok"]
    dup = want.clone(); dup[0] = dup[1]
    assert not oracle.check_topk_row(scores, table, 4000, dup)["ok"]
    # flat boundary: any of the tied elements is acceptable
    flat = torch.ones(4000)
    flat[:1000] = 2.0
    pick = torch.cat([torch.arange(1000), torch.arange(2500, 3548)]).to(torch.int32)
    info = oracle.check_topk_row(flat, table, 4000, pick)
    assert info["ok"] and info["mode"] == "tolerant"
    short = torch.full((2048,), -1, dtype=torch.int32); short[:100] = torch.arange(100, dtype=torch.int32)
    assert oracle.check_topk_row(torch.rand(100), table, 100, short)["ok"]
    short[99] = -1
    assert not oracle.check_topk_row(torch.rand(100), table, 100, short)["ok"]
