"""GPU parity of sparse MLA attention against the CPU oracle / golden fixtures, through the C ABI."""
import pytest
import torch

import dsa_oracle as oracle
from auto_gpu_kernel_b200 import inputs as wl, sparse_attention, workspace
from helpers import assert_attention_close, load_attention_golden

pytestmark = pytest.mark.gpu


VARIANTS = pytest.mark.parametrize("variant", [1, 0, 2], ids=["cuda_core", "mma_sync", "tcgen05"])


@VARIANTS
@pytest.mark.parametrize("name", ["attention_small", "attention_padded"])
def test_matches_golden(cuda, name, variant):
    inp, ref_out, ref_lse = load_attention_golden(name)
    dev = inp.to(cuda)
    out = torch.full_like(ref_out, 7.0, device=cuda)
    lse = torch.full_like(ref_lse, 7.0, device=cuda)
    assert sparse_attention.kernel(*dev.args(), out, lse, variant) is None
    workspace.check_status(cuda)
    assert_attention_close(out, lse, ref_out, ref_lse, label=name)
    out2, lse2 = sparse_attention.run(*dev.args(), variant=variant)  # workspace counters reused
    assert_attention_close(out2, lse2, ref_out, ref_lse, label=name + "/again")


@VARIANTS
@pytest.mark.parametrize("tokens", [1, 2, 8, 64, 300, 700])
def test_token_counts_against_gpu_oracle(cuda, tokens, variant):
    """Different token counts exercise different splits of the selected rows across CTAs: many
    segments per token (1, 2, 8), a few (64, 300), whole tokens per CTA (700)."""
    lens = wl.uniform_lengths(tokens, 2100, 6000, seed=tokens)
    inp = wl.make_attention_inputs(lens, seed=tokens, device=cuda)
    out, lse = sparse_attention.run(*inp.args(), variant=variant)
    workspace.check_status(cuda)
    ref_out, ref_lse = oracle.sparse_attention(
        *[a if not torch.is_tensor(a) else a for a in inp.args()],
        output=torch.empty_like(out), lse=torch.empty_like(lse))
    assert_attention_close(out, lse, ref_out.cpu(), ref_lse.cpu(), label=f"T={tokens}")


@pytest.mark.parametrize("tokens", [16, 18, 33, 37, 63, 70, 74, 130, 148])
def test_cluster_split_token_counts(cuda, tokens):
    """Token counts at which the default kernel runs one cluster of 8 / 4 / 2 / 1 CTAs per token
    and merges through distributed shared memory; rows with few valid ids leave some ranks of a
    cluster without any live tile, and one row is fully masked."""
    lens = wl.uniform_lengths(tokens, 40, 6000, seed=100 + tokens)
    inp = wl.make_attention_inputs(lens, seed=100 + tokens, device=cuda)
    idx = inp.sparse_indices.clone()
    idx[1, 70:] = -1            # two tiles live, the rest masked
    idx[2] = -1                 # nothing valid: output 0, lse -inf
    idx[3, :1500] = -1          # only the last ranks see valid rows
    inp.sparse_indices = idx
    out, lse = sparse_attention.run(*inp.args(), variant=0)
    workspace.check_status(cuda)
    ref_out, ref_lse = oracle.sparse_attention(*inp.args(), output=torch.empty_like(out),
                                               lse=torch.empty_like(lse))
    assert_attention_close(out, lse, ref_out.cpu(), ref_lse.cpu(), label=f"cluster T={tokens}")
    out_cc, lse_cc = sparse_attention.run(*inp.args(), variant=1)
    assert_attention_close(out, lse, out_cc.cpu(), lse_cc.cpu(), label=f"cluster vs cuda-core T={tokens}")


@VARIANTS
@pytest.mark.parametrize("topk", [1, 64, 100, 512, 1000, 2047])
def test_other_index_widths(cuda, topk, variant):
    """The C ABI takes the width of the index rows as an argument: widths that are not the
    definition's 2048, including ones that are not multiples of the 64-row tile."""
    for tokens in (3, 20, 70, 140):
        inp = wl.make_attention_inputs([6000] * tokens, seed=31 * tokens + topk, device=cuda)
        inp.sparse_indices = inp.sparse_indices[:, :topk].contiguous()
        out, lse = sparse_attention.run(*inp.args(), variant=variant)
        workspace.check_status(cuda)
        ref_out, ref_lse = oracle.sparse_attention(*inp.args(), output=torch.empty_like(out),
                                                   lse=torch.empty_like(lse))
        assert_attention_close(out, lse, ref_out.cpu(), ref_lse.cpu(), label=f"topk={topk} T={tokens}")


@VARIANTS
def test_token_count_changes_between_calls(cuda, variant):
    """One workspace serves calls of different token counts: the arrival counters of one call must
    never sit where an earlier call with another token count left partial results."""
    for tokens in (8, 70, 3, 130, 40, 9):
        lens = wl.uniform_lengths(tokens, 2100, 5000, seed=7 * tokens)
        inp = wl.make_attention_inputs(lens, seed=7 * tokens, device=cuda)
        out, lse = sparse_attention.run(*inp.args(), variant=variant)
        workspace.check_status(cuda)
        ref_out, ref_lse = oracle.sparse_attention(*inp.args(), output=torch.empty_like(out),
                                                   lse=torch.empty_like(lse))
        assert_attention_close(out, lse, ref_out.cpu(), ref_lse.cpu(), label=f"sequence T={tokens}")


@VARIANTS
def test_interior_and_leading_padding(cuda, variant):
    """-1 entries anywhere in a row (not only the tail) are masked."""
    inp = wl.make_attention_inputs([4000, 4000, 4000], seed=9, device=cuda)
    idx = inp.sparse_indices.clone()
    idx[0, ::3] = -1
    idx[1, :1000] = -1
    idx[2, 5:] = -1
    inp.sparse_indices = idx
    out, lse = sparse_attention.run(*inp.args(), variant=variant)
    workspace.check_status(cuda)
    ref_out, ref_lse = oracle.sparse_attention(*inp.to("cpu").args())
    assert_attention_close(out, lse, ref_out, ref_lse, label="interior padding")


@VARIANTS
def test_large_logits_are_stable(cuda, variant):
    """Scaled-up queries give logits far outside exp range: the online softmax must not overflow."""
    inp = wl.make_attention_inputs([3000, 2500], seed=4, device=cuda)
    inp.q_nope = (inp.q_nope.float() * 40).to(torch.bfloat16)
    out, lse = sparse_attention.run(*inp.args(), variant=variant)
    workspace.check_status(cuda)
    ref_out, ref_lse = oracle.sparse_attention(*inp.to("cpu").args())
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()
    assert_attention_close(out, lse, ref_out, ref_lse, label="large logits")


@VARIANTS
def test_out_of_range_slot_is_masked_and_reported(cuda, variant):
    inp = wl.make_attention_inputs([2500], seed=6, device=cuda)
    slots = inp.ckv_cache.shape[0] * 64
    inp.sparse_indices[0, 7] = slots + 5
    out, lse = sparse_attention.run(*inp.args(), variant=variant)
    with pytest.raises(RuntimeError, match="sparse index outside"):
        workspace.check_status(cuda)
    cpu = inp.to("cpu")
    cpu.sparse_indices[0, 7] = -1
    ref_out, ref_lse = oracle.sparse_attention(*cpu.args())
    assert_attention_close(out, lse, ref_out, ref_lse, label="bad slot")


def test_ascending_logits_force_rescales(cuda):
    """Rows ordered so that logits grow tile after tile: the running max is refreshed repeatedly
    and the accumulated output is rescaled in place many times."""
    inp = wl.make_attention_inputs([4096], seed=12, device=cuda)
    cpu = inp.to("cpu")
    logits = (cpu.q_nope[0, 0].float() @ cpu.ckv_cache.reshape(-1, 512)[cpu.sparse_indices[0].long()].float().T)
    order = torch.argsort(logits)                       # ascending for head 0
    inp.sparse_indices[0] = inp.sparse_indices[0][order.to(cuda)]
    inp.q_nope = (inp.q_nope.float() * 30).to(torch.bfloat16)
    out, lse = sparse_attention.run(*inp.args())
    workspace.check_status(cuda)
    ref_out, ref_lse = oracle.sparse_attention(*inp.to("cpu").args())
    assert_attention_close(out, lse, ref_out, ref_lse, label="ascending")


def test_cpu_tensors_are_rejected():
    inp = wl.make_attention_inputs([100], seed=0)
    with pytest.raises(RuntimeError, match="no CPU path"):
        sparse_attention.run(*inp.args())
