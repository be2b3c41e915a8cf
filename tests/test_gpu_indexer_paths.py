"""The two selection paths of dsa_indexer_topk -- "hist" (default: the scorer builds each request's
score histogram, the selection kernel starts from it) and "minmax" (the scorer hands over the
row's min / max, the selection builds a histogram of its own) -- driven through the C ABI with
score rows chosen by the test: `indexer_inputs_from_scores` builds a key cache whose scores are exactly a given fp32
row, so the selection logic (boundary bin, candidate ranking, the radix descent for over-full
bins, tie order, short rows, many requests) is checked against torch.topk on known rows."""
import pytest
import torch

import dsa_oracle as oracle
from auto_gpu_kernel_b200 import indexer, inputs as wl, workspace
from helpers import assert_topk_matches, indexer_inputs_from_scores

pytestmark = pytest.mark.gpu


@pytest.fixture(params=["hist", "minmax"], autouse=True)
def indexer_path(request, monkeypatch):
    """Every test of this file runs once per path (DSA_INDEXER_PATH is read on every call)."""
    monkeypatch.setenv("DSA_INDEXER_PATH", request.param)
    return request.param


def _local_positions(got_row, table_row, n):
    """Positions inside the request of the given global slots (only the request's own pages count:
    the unused tail of a block_table row holds zeros)."""
    inv = {int(p): i for i, p in enumerate(table_row[: (n + 63) // 64].tolist())}
    return torch.tensor([inv[g // 64] * 64 + g % 64 for g in got_row.tolist()])


def _check_row(row, n, table_row, got_row, label=""):
    """Distinct ids of the request carrying exactly the top-2048 score multiset, or all of the row
    plus -1 padding when it is not longer than 2048."""
    k = min(2048, n)
    valid = got_row[got_row >= 0]
    assert valid.numel() == k and torch.unique(valid).numel() == k, f"{label}: {valid.numel()} ids"
    assert (got_row[k:] == -1).all() or n > 2048, label
    if k == 0:
        return
    local = _local_positions(valid, table_row, n)
    assert int(local.max()) < n, label
    want = torch.topk(row[:n].float().nan_to_num(nan=-3.0e38, neginf=-3.0e38), k).values
    have = torch.sort(row[local].float().nan_to_num(nan=-3.0e38, neginf=-3.0e38), descending=True).values
    assert torch.equal(have, want), label


def _run(rows, lens, cuda, seed=0):
    inp = indexer_inputs_from_scores(rows, lens, seed=seed, device=cuda)
    out = torch.full((len(lens), 2048), 777, dtype=torch.int32, device=cuda)
    indexer.kernel(*inp.args(), out)
    workspace.check_status(cuda)
    return inp, out.cpu()


@pytest.mark.parametrize("length", [2049, 5000, 5003, 45057, 131072, 200001])
def test_selection_against_torch_topk(cuda, length):
    """Positive, negative, mixed and one-binade rows (the last puts the whole row into one bin of
    the first histogram, so it takes the radix descent), lengths that are not multiples of 4 or 128,
    and one beyond what four CTAs can stage in shared memory (the slices are then swept from L2)."""
    gen = torch.Generator().manual_seed(length)
    width = (length + 63) // 64 * 64
    rows = torch.randn(4, width, generator=gen)
    rows[1] = -rows[1].abs() - 1.0
    rows[2] = rows[2] * 1e-3 + 5.0
    rows[3] = rows[3].abs() * 1e-4        # many tiny values and a long tail of bins
    lens = [length, length, length - 1, length]
    inp, got = _run(rows, lens, cuda, seed=length)
    for b in range(4):
        _check_row(rows[b], lens[b], inp.block_table[b].cpu(), got[b], label=f"len {length} row {b}")


def test_ties_take_lowest_positions(cuda):
    length = 6000
    rows = torch.zeros(3, 6016)
    rows[0, 100:200] = 1.0                 # 100 above, 5900 tied at zero -> the lowest 1948 zeros
    rows[1, 4000:4010] = -1.0              # ten below, everything else tied
    rows[2] = 0.25
    rows[2, 5:3000:2] = 0.25000003         # 1498 just above (next fp32), 550 of the ties wanted
    inp, got = _run(rows, [length] * 3, cuda, seed=3)
    table = inp.block_table.cpu()
    sel = [set(_local_positions(got[b], table[b], length).tolist()) for b in range(3)]
    zeros = [i for i in range(length) if not 100 <= i < 200][:1948]
    assert sel[0] == set(range(100, 200)) | set(zeros)
    assert sel[1] == set(range(2048))
    high = set(range(5, 3000, 2))
    rest = [i for i in range(length) if i not in high][: 2048 - len(high)]
    assert sel[2] == high | set(rest)


@pytest.mark.parametrize("step", [0.125, 0.01])
def test_quantised_scores_tie_across_the_boundary(cuda, step):
    """Scores on a coarse grid: hundreds to thousands of equal values straddle the 2048th place, in
    the boundary bin and at the exact threshold.  Equal bit patterns are taken lowest position
    first; -0.0 ranks below +0.0 (torch.topk calls them equal, so either order is a valid top-k)."""
    gen = torch.Generator().manual_seed(int(1 / step))
    lens = [33000, 9000, 2049, 20000, 12345, 70000]
    width = (max(lens) + 63) // 64 * 64
    rows = (torch.randn(len(lens), width, generator=gen) / step).round() * step
    inp, got = _run(rows, lens, cuda, seed=11)
    table = inp.block_table.cpu()
    for b, n in enumerate(lens):
        _check_row(rows[b], n, table[b], got[b], label=f"row {b}")
        local = _local_positions(got[b], table[b], n)
        thr = rows[b][local].min()
        same = (rows[b][:n].view(torch.int32) == thr.view(torch.int32)).nonzero().flatten().tolist()
        chosen = set(local.tolist())
        taken = [p for p in same if p in chosen]
        assert taken == same[: len(taken)], f"row {b}: ties at the threshold are not the lowest positions"


def test_nan_and_inf_rank_lowest(cuda):
    length = 5000
    gen = torch.Generator().manual_seed(9)
    rows = torch.randn(2, 5056, generator=gen)
    rows[0, ::3] = float("nan")
    rows[0, 1::7] = float("-inf")
    rows[1, :4000] = float("nan")          # fewer than 2048 ordinary scores: 1048 NaNs must be taken
    inp, got = _run(rows, [length] * 2, cuda, seed=4)
    table = inp.block_table.cpu()
    for b in range(2):
        _check_row(rows[b], length, table[b], got[b], label=f"row {b}")
    taken = _local_positions(got[1], table[1], length)
    assert set(range(4000, 5000)) <= set(taken.tolist())
    assert sorted(i for i in taken.tolist() if i < 4000) == list(range(1048))   # lowest positions first


def test_many_requests_complete_in_any_order(cuda, indexer_path):
    """More requests than SMs, ragged lengths with short and empty rows in between; and a second
    call over the same workspace: whatever a call leaves behind must not disturb the next."""
    gen = torch.Generator().manual_seed(77)
    lens = [int(x) for x in torch.randint(2049, 9000, (150,), generator=gen)]
    for i in range(0, 150, 11):
        lens[i] = [0, 1, 2047, 2048, 700][(i // 11) % 5]
    lens[7] = 70000
    width = (max(lens) + 63) // 64 * 64
    rows = torch.randn(len(lens), width, generator=gen)
    inp, got = _run(rows, lens, cuda, seed=5)
    table = inp.block_table.cpu()
    for b, n in enumerate(lens):
        _check_row(rows[b], n, table[b], got[b], label=f"request {b} len {n}")
    # and a second call over the same workspace: every control word and histogram was put back
    inp2, got2 = _run(rows, lens, cuda, seed=5)
    for b, n in enumerate(lens):
        _check_row(rows[b], n, table[b], got2[b], label=f"second call, request {b}")
    ws = workspace.get(cuda, "indexer", 1)
    torch.cuda.synchronize()
    histograms = ws[512 * 1024: 512 * 1024 + 1024 * 4096 * 4].view(torch.int32)    # all 1024 histograms
    assert int(histograms.abs().max()) == 0
    if indexer_path == "minmax":     # the words of this batch's requests (the other path never touches them)
        assert int(ws[: 2 * 4 * len(lens)].view(torch.int32).abs().max()) == 0


def test_hundreds_of_medium_rows(cuda):
    """More than two rows per SM, each small enough for half an SM's shared memory: on the min / max
    path this is the shape that runs two narrow selection CTAs per SM (chunked prefill).  Rows with
    600 and with 5000 tied scores at the boundary take the candidate ranking's overflow route."""
    gen = torch.Generator().manual_seed(321)
    lens = [int(x) for x in torch.randint(2049, 12000, (320,), generator=gen)]
    lens[3], lens[200] = 11999, 2049
    width = (max(lens) + 63) // 64 * 64
    rows = torch.randn(len(lens), width, generator=gen)
    rows[5, 1000:1600] = 0.5          # 600 ties inside the top 2048 of a ~N(0,1) row
    rows[6, :5000] = 10.0             # 5000 ties above everything else: the lowest 2048 positions
    rows[7] = rows[7] * 1e-6 + 3.0    # one binade
    lens[5], lens[6], lens[7] = 9000, 9000, 9000
    inp, got = _run(rows, lens, cuda, seed=6)
    table = inp.block_table.cpu()
    for b, n in enumerate(lens):
        _check_row(rows[b], n, table[b], got[b], label=f"request {b} len {n}")
    assert set(_local_positions(got[6], table[6], lens[6]).tolist()) == set(range(2048))


def test_more_requests_than_histograms(cuda, indexer_path):
    """1100 requests: beyond the 1024 histograms of the workspace, so the call takes the min / max
    selection whatever DSA_INDEXER_PATH says, and leaves the histogram region untouched."""
    if indexer_path == "minmax":
        pytest.skip("one run is enough: the path is chosen from the batch size")
    gen = torch.Generator().manual_seed(1100)
    lens = [int(x) for x in torch.randint(2049, 4000, (1100,), generator=gen)]
    lens[0], lens[1099], lens[500] = 3999, 2049, 17
    width = (max(lens) + 63) // 64 * 64
    rows = torch.randn(len(lens), width, generator=gen)
    inp, got = _run(rows, lens, cuda, seed=8)
    table = inp.block_table.cpu()
    for b in list(range(0, 1100, 37)) + [1023, 1024, 1099]:
        _check_row(rows[b], lens[b], table[b], got[b], label=f"request {b} len {lens[b]}")
    valid = (got >= 0).sum(dim=1)
    assert torch.equal(valid, torch.tensor([min(2048, n) for n in lens]))
    ws = workspace.get(cuda, "indexer", 1)
    torch.cuda.synchronize()
    assert int(ws[512 * 1024: 512 * 1024 + 1024 * 4096 * 4].view(torch.int32).abs().max()) == 0


def test_paths_select_the_same_set(cuda, monkeypatch, indexer_path):
    if indexer_path == "minmax":
        pytest.skip("compared from the other side")
    lens = [3000, 2049, 40000, 9000, 100, 0, 33000]
    inp = wl.make_indexer_inputs(lens, seed=31, device=cuda)
    rows = [r.cpu() for r in oracle.indexer_scores(*inp.args())]
    got = indexer.run(*inp.args())
    workspace.check_status(cuda)
    assert_topk_matches(inp, got, rows, label=indexer_path)
    monkeypatch.setenv("DSA_INDEXER_PATH", "minmax")
    split = indexer.run(*inp.args())
    workspace.check_status(cuda)
    assert_topk_matches(inp, split, rows, label="minmax")
    assert torch.equal(torch.sort(got, dim=1).values, torch.sort(split, dim=1).values)


def test_bad_page_ids_are_flagged_not_followed(cuda):
    """A block_table entry outside [0, num_pages) -- first or second page of a tile, negative or too
    large -- sets DSA_STATUS_BAD_PAGE and is replaced by page 0; nothing faults."""
    lens = [4096, 4096, 4096]
    inp = wl.make_indexer_inputs(lens, seed=41, device=cuda)
    workspace.check_status(cuda)
    for col, value in ((0, -7), (1, -7), (3, 10**6), (2, inp.k_index_cache_fp8.shape[0])):
        table = inp.block_table.clone()
        table[1, col] = value
        out = indexer.run(inp.q_index_fp8, inp.k_index_cache_fp8, inp.weights, inp.seq_lens, table)
        with pytest.raises(RuntimeError, match="block_table entry outside"):
            workspace.check_status(cuda)
        got = indexer.scores(inp.q_index_fp8, inp.k_index_cache_fp8, inp.weights, inp.seq_lens, table)
        with pytest.raises(RuntimeError, match="block_table entry outside"):
            workspace.check_status(cuda)
        assert out.shape == (3, 2048) and torch.isfinite(got[0, :4096]).all()
