"""GPU parity of the FP8 top-k indexer against the CPU oracle / golden fixtures.  Every call goes
through the C ABI of libdsa_b200.so (via the ctypes host layer)."""
import pytest
import torch

import dsa_oracle as oracle
from auto_gpu_kernel_b200 import indexer, inputs as wl, workspace
from helpers import assert_topk_matches, load_indexer_golden

pytestmark = pytest.mark.gpu

# Score tolerance: e4m3 x e4m3 products are exact in fp32, so the only differences against the
# oracle are fp32 summation order and where the per-token scale is applied (~1e-6 relative).
SCORE_RTOL = 2e-5


def _score_err(got_rows, ref_rows, seq_lens):
    worst = 0.0
    for b, ref in enumerate(ref_rows):
        n = int(seq_lens[b])
        if n == 0:
            continue
        got = got_rows[b, :n].float().cpu()
        ref = ref.float().cpu()
        assert torch.isfinite(got).all(), f"row {b}: non-finite scores"
        worst = max(worst, float((got - ref).abs().max() / ref.abs().max().clamp_min(1e-20)))
    return worst


@pytest.mark.parametrize("variant", [1, 0], ids=["cuda_core", "tcgen05"])
@pytest.mark.parametrize("name", ["indexer_cfg0", "indexer_edges"])
def test_scores_match_oracle(cuda, name, variant):
    inp, _, _ = load_indexer_golden(name)
    ref = oracle.indexer_scores(*inp.args())
    got = indexer.scores(*inp.to(cuda).args(), variant=variant)
    workspace.check_status(cuda)
    assert _score_err(got, ref, inp.seq_lens) < SCORE_RTOL


@pytest.mark.parametrize("name", ["indexer_cfg0", "indexer_edges"])
def test_topk_matches_golden(cuda, name):
    inp, golden_idx, _ = load_indexer_golden(name)
    dev = inp.to(cuda)
    out = torch.full((len(inp.seq_lens), wl.TOPK), 12345, dtype=torch.int32, device=cuda)
    assert indexer.kernel(*dev.args(), out) is None
    workspace.check_status(cuda)
    modes = assert_topk_matches(inp, out, label=name)
    out2 = indexer.run(*dev.args())
    for b in range(out.shape[0]):  # the selected SET is deterministic
        assert set(out[b].tolist()) == set(out2[b].tolist())
        if modes[b] in ("exact", "all"):
            assert set(out[b].tolist()) == set(golden_idx[b].tolist())


def _check_selection(row, n, table_row, got_row):
    """Selected ids are distinct, belong to the row, and carry exactly the top-2048 score multiset
    (torch.topk breaks exact ties arbitrarily, so sets are compared through their scores)."""
    got = got_row.tolist()
    assert len(set(got)) == 2048 and min(got) >= 0
    inv = {int(p): i for i, p in enumerate(table_row.tolist())}
    local = torch.tensor([inv[g // 64] * 64 + g % 64 for g in got])
    assert int(local.max()) < n
    want = torch.topk(row[:n], 2048).values
    assert torch.equal(torch.sort(row[local], descending=True).values, want)


@pytest.mark.parametrize("length", [2049, 5000, 5003, 45056, 45057, 49153, 131072])
def test_select_against_torch_topk(cuda, length):
    """Selection alone on synthetic rows: positive, negative and mixed scores; staged and streamed
    row paths (the boundary is 45056 scores), lengths that are not multiples of four."""
    gen = torch.Generator(device="cpu").manual_seed(length)
    pages = (length + 63) // 64
    table = torch.randperm(pages, generator=gen).to(torch.int32).unsqueeze(0).repeat(3, 1)
    rows = torch.randn(3, pages * 64, generator=gen)
    rows[1] = -rows[1].abs() - 1.0           # all negative
    rows[2] = rows[2] * 1e-3 + 5.0           # one binade, many exact ties: coarse first digit
    lens = torch.tensor([length, length, length - 1], dtype=torch.int32)
    got = indexer.select(rows.to(cuda), lens.to(cuda), table.to(cuda)).cpu()
    workspace.check_status(cuda)
    for b in range(3):
        _check_selection(rows[b], int(lens[b]), table[b], got[b])


def test_select_ties_take_lowest_positions(cuda):
    length = 6000
    rows = torch.zeros(2, 6016)
    rows[0, 100:200] = 1.0                      # 100 above, 5900 tied at zero -> lowest 1948 zeros
    rows[1] = -0.0
    rows[1, ::2] = 0.0                          # +0 > -0 in key order, still all "equal" as floats
    table = torch.arange(94, dtype=torch.int32).unsqueeze(0).repeat(2, 1).to(cuda)
    lens = torch.tensor([length, length], dtype=torch.int32, device=cuda)
    got = indexer.select(rows.to(cuda), lens, table).cpu()
    workspace.check_status(cuda)
    zeros = [i for i in range(length) if not 100 <= i < 200][:1948]
    assert set(got[0].tolist()) == set(range(100, 200)) | set(zeros)
    assert len(set(got[1].tolist())) == 2048 and min(got[1].tolist()) >= 0 and max(got[1].tolist()) < length


def test_long_ragged_batch_against_gpu_oracle(cuda):
    """Lengths beyond the staged-row limit, ragged, one empty and one short request; the oracle runs
    on the GPU in fp32 for speed (same code as on CPU)."""
    lens = [70001, 0, 33000, 1500, 131072, 2048, 2049]
    inp = wl.make_indexer_inputs(lens, seed=11, device=cuda)
    out = indexer.run(*inp.args())
    workspace.check_status(cuda)
    rows = [r.cpu() for r in oracle.indexer_scores(*inp.args())]
    assert_topk_matches(inp, out, rows, label="ragged")
    got_tc = indexer.scores(*inp.args(), variant=0)
    got_cc = indexer.scores(*inp.args(), variant=1)
    assert _score_err(got_tc, rows, lens) < SCORE_RTOL
    assert _score_err(got_cc, rows, lens) < SCORE_RTOL


def test_shared_block_table_rows_prefill(cuda):
    """Chunked prefill: many query rows over one request's pages, block_table passed with row
    stride 0 (expand) and causal per-row lengths."""
    inp = wl.make_shared_prefix_indexer_inputs(prefix_len=3000, chunk_len=96, seed=5, device=cuda)
    shared = inp.block_table[:1].expand(96, -1)
    assert shared.stride(0) == 0
    out_a = indexer.run(inp.q_index_fp8, inp.k_index_cache_fp8, inp.weights, inp.seq_lens, shared)
    out_b = indexer.run(*inp.args())
    workspace.check_status(cuda)
    assert_topk_matches(inp, out_a, label="prefill")
    for r in range(96):
        assert set(out_a[r].tolist()) == set(out_b[r].tolist())


@pytest.mark.parametrize("prefix_len,chunk_len", [(3000, 96), (5000, 37), (200, 300), (0, 17)])
def test_prefill_scorer_matches_oracle_and_streaming_kernel(cuda, prefix_len, chunk_len):
    """The shared-pages scorer (eight rows per key tile, N = 256 products) against the oracle and
    against the streaming tcgen05 kernel: chunk sizes that are not multiples of 8, rows shorter
    than one tile, a prefix of zero."""
    inp = wl.make_shared_prefix_indexer_inputs(prefix_len=prefix_len, chunk_len=chunk_len, seed=6,
                                               device=cuda)
    shared = inp.block_table[:1].expand(chunk_len, -1)
    lens = inp.seq_lens.tolist()
    rows = [r.cpu() for r in oracle.indexer_scores(*inp.args())]
    got_pf = indexer.scores(inp.q_index_fp8, inp.k_index_cache_fp8, inp.weights, inp.seq_lens,
                            shared, variant=0)
    got_st = indexer.scores(inp.q_index_fp8, inp.k_index_cache_fp8, inp.weights, inp.seq_lens,
                            shared, variant=2)
    workspace.check_status(cuda)
    assert _score_err(got_pf, rows, lens) < SCORE_RTOL
    assert _score_err(got_st, rows, lens) < SCORE_RTOL
    for b, n in enumerate(lens):   # untouched beyond each row's length
        assert torch.isnan(got_pf[b, n:]).all()


def test_prefill_scorer_ragged_lengths(cuda):
    """Rows of one launch need not be causal: arbitrary lengths over the shared pages, including
    empty rows and rows at the top-k boundary."""
    inp = wl.make_shared_prefix_indexer_inputs(prefix_len=6000, chunk_len=40, seed=8, device=cuda)
    lens = [6040, 0, 1, 2048, 2049, 127, 128, 129, 6000, 64] * 4
    seq = torch.tensor(lens, dtype=torch.int32, device=cuda)
    shared = inp.block_table[:1].expand(40, -1)
    args = (inp.q_index_fp8, inp.k_index_cache_fp8, inp.weights, seq)
    rows = [r.cpu() for r in oracle.indexer_scores(*args, inp.block_table)]
    got = indexer.scores(*args, shared, variant=0)
    assert _score_err(got, rows, lens) < SCORE_RTOL
    out = indexer.run(*args, shared)
    workspace.check_status(cuda)
    ragged = wl.IndexerInputs(inp.q_index_fp8, inp.k_index_cache_fp8, inp.weights, seq, inp.block_table)
    assert_topk_matches(ragged, out, rows, label="prefill ragged")


@pytest.mark.parametrize("junk", ["random", "ones", "nan", "tiny_range"])
def test_foreign_minmax_words_cost_speed_not_correctness(cuda, junk, monkeypatch):
    """Two-kernel path (DSA_INDEXER_PATH=minmax; also taken by batches beyond 1024 requests): the scorer leaves
    each row's min / max in the workspace for the selection.  Whatever those words hold when a
    call starts (an aborted call, a caller that did not zero the workspace), the selected set
    stays exact: the bins are clamped and monotone for any [lo, hi]."""
    monkeypatch.setenv("DSA_INDEXER_PATH", "minmax")
    lens = [3000, 2049, 40000, 9000]
    inp = wl.make_indexer_inputs(lens, seed=17, device=cuda)
    rows = [r.cpu() for r in oracle.indexer_scores(*inp.args())]
    first = indexer.run(*inp.args())                       # creates the shared workspace
    assert_topk_matches(inp, first, rows, label="clean")
    lib_need = 512 * 1024
    ws = workspace.get(cuda, "indexer", lib_need)
    words = ws[:lib_need].view(torch.int32)
    if junk == "random":
        words.random_(-2**31, 2**31 - 1)
    elif junk == "ones":
        words.fill_(-1)
    elif junk == "nan":
        words.copy_(torch.full_like(words, 0x7FC00000 | (1 << 31) - (1 << 31)))   # key of a NaN
    else:   # a [lo, hi] far above every score: everything falls into the lowest bin
        key = torch.tensor([1.0e30], dtype=torch.float32).view(torch.int32).item() | -2**31
        words[0::2] = key
        words[1::2] = ~key
    for attempt in range(2):    # the call that meets the junk, then the one after it
        out = indexer.run(*inp.args())
        workspace.check_status(cuda)
        assert_topk_matches(inp, out, rows, label=f"{junk} attempt {attempt}")
    torch.cuda.synchronize()
    assert int(words[: 2 * len(lens)].abs().sum()) == 0     # put back to zero for the next call


def test_foreign_histogram_is_flagged_then_healed(cuda, monkeypatch):
    """Default path (the scorer counts each request's scores into a histogram in the workspace, which
    must be zero between calls).  Counts that are not this call's -- an aborted call, a workspace
    that was never zeroed -- cannot be told from real ones, so the call that meets them reports
    DSA_STATUS_TOPK_COUNT (the selection's own totals disagree with the histogram); it also puts the
    histograms back to zero, so the next call is exact again."""
    monkeypatch.setenv("DSA_INDEXER_PATH", "hist")
    lens = [3000, 2049, 40000, 9000]
    inp = wl.make_indexer_inputs(lens, seed=23, device=cuda)
    rows = [r.cpu() for r in oracle.indexer_scores(*inp.args())]
    first = indexer.run(*inp.args())                       # creates the shared workspace
    workspace.check_status(cuda)
    assert_topk_matches(inp, first, rows, label="clean")
    ws = workspace.get(cuda, "indexer", 1)
    hist = ws[512 * 1024: 512 * 1024 + len(lens) * 4096 * 4].view(torch.int32)
    hist.random_(0, 5)
    indexer.run(*inp.args())
    with pytest.raises(RuntimeError, match="0x8"):
        workspace.check_status(cuda)
    torch.cuda.synchronize()
    assert int(hist.abs().max()) == 0
    out = indexer.run(*inp.args())
    workspace.check_status(cuda)
    assert_topk_matches(inp, out, rows, label="after the flagged call")


def test_strided_block_table_and_output_rows(cuda):
    """block_table and topk_indices may be column slices of wider tensors (row stride larger than
    the row length): the reference's kernels take the strides as arguments too."""
    lens = [2500, 7000, 64, 3000, 2049]
    inp = wl.make_indexer_inputs(lens, seed=23, device=cuda)
    pages = inp.block_table.shape[1]
    wide_table = torch.full((len(lens), pages + 37), -5, dtype=torch.int32, device=cuda)
    wide_table[:, :pages] = inp.block_table
    wide_out = torch.full((len(lens), 2048 + 64), -9, dtype=torch.int32, device=cuda)
    table_view, out_view = wide_table[:, :pages], wide_out[:, :2048]
    assert table_view.stride(0) == pages + 37 and out_view.stride(0) == 2048 + 64
    indexer.kernel(inp.q_index_fp8, inp.k_index_cache_fp8, inp.weights, inp.seq_lens, table_view, out_view)
    workspace.check_status(cuda)
    rows = [r.cpu() for r in oracle.indexer_scores(*inp.args())]
    assert_topk_matches(inp, out_view.contiguous(), rows, label="strided")
    assert (wide_out[:, 2048:] == -9).all()          # nothing written past a row


def test_rows_within_topk_need_no_scores(cuda):
    """When no request can exceed 2048 tokens (max_pages <= 32) every cached token is selected and
    the scorer is not launched: the result is the request's slots, whatever the keys are."""
    lens = [0, 1, 63, 64, 700, 2047, 2048]
    inp = wl.make_indexer_inputs(lens, seed=13, device=cuda)
    assert inp.block_table.shape[1] == 32
    inp.k_index_cache_fp8.view(torch.uint8).fill_(0xFF)      # NaN keys and scales: must not matter
    out = indexer.run(*inp.args())
    workspace.check_status(cuda)
    for b, n in enumerate(lens):
        want = (inp.block_table[b, torch.arange(n, device=cuda) // 64].long() * 64
                + torch.arange(n, device=cuda) % 64)
        assert torch.equal(out[b, :n].long().sort().values, want.sort().values)
        assert (out[b, n:] == -1).all()


def test_cpu_tensors_are_rejected():
    inp = wl.make_indexer_inputs([100], seed=0)
    with pytest.raises(RuntimeError, match="no CPU path"):
        indexer.run(*inp.args())


def test_short_rows_chained_with_attention_on_one_index_buffer(cuda):
    """Contexts within top-k: no scorer is launched, so the selection is the programmatic dependent
    of whatever ran before it -- here the previous step's attention, which reads the very index
    buffer the selection rewrites.  Many steps back to back on one stream with changing lengths:
    every step's attention must have seen that step's indices, none of the next step's."""
    from auto_gpu_kernel_b200 import sparse_attention
    batch, steps = 8, 24
    block = wl.make_decode_block_inputs([2048] * batch, seed=19, device=cuda)
    idx = block.indexer
    assert idx.block_table.shape[1] == 32
    gen = torch.Generator().manual_seed(20)
    lens = [torch.randint(1, 2049, (batch,), generator=gen).to(torch.int32) for _ in range(steps)]
    lens_dev = [x.to(cuda) for x in lens]
    topk = torch.empty(batch, 2048, dtype=torch.int32, device=cuda)
    outs = [torch.empty_like(block.q_nope) for _ in range(steps)]
    lses = [torch.empty(batch, 16, dtype=torch.float32, device=cuda) for _ in range(steps)]
    torch.cuda.synchronize()
    for s in range(steps):
        indexer.kernel(idx.q_index_fp8, idx.k_index_cache_fp8, idx.weights, lens_dev[s], idx.block_table, topk)
        sparse_attention.kernel(block.q_nope, block.q_pe, block.ckv_cache, block.kpe_cache, topk,
                                block.sm_scale, outs[s], lses[s])
    workspace.check_status(cuda)
    table = idx.block_table.cpu().long()
    pos = torch.arange(2048)
    for s in range(steps):
        want = torch.full((batch, 2048), -1, dtype=torch.int32)
        for b in range(batch):
            n = int(lens[s][b])
            want[b, :n] = (table[b, pos[:n] // 64] * 64 + pos[:n] % 64).to(torch.int32)
        ref_out, ref_lse = oracle.sparse_attention(block.q_nope, block.q_pe, block.ckv_cache, block.kpe_cache,
                                                   want.to(cuda), block.sm_scale,
                                                   output=torch.empty_like(outs[s]), lse=torch.empty_like(lses[s]))
        assert torch.allclose(lses[s], ref_lse, atol=1e-3, rtol=1e-3), f"step {s}"
        assert torch.allclose(outs[s].float(), ref_out.float(), atol=1e-2, rtol=1e-2), f"step {s}"
