"""Shared helpers of the test-suite: golden fixture loading and acceptance checks."""
from pathlib import Path

import numpy as np
import torch

import dsa_oracle as oracle
from auto_gpu_kernel_b200 import inputs as wl

GOLDEN = Path(__file__).resolve().parent / "golden"

# Tolerances of the acceptance rule: attention output atol = rtol = 1e-2
# (bf16), LSE 1e-3; indexer: exact set where the boundary gap > 1e-3 relative, else recall >= 0.999
# and selected scores within 1e-3.
ATT_ATOL = 1e-2
ATT_RTOL = 1e-2
LSE_TOL = 1e-3


def load_indexer_golden(name):
    z = np.load(GOLDEN / f"{name}.npz")
    inp = wl.IndexerInputs(
        torch.from_numpy(z["q_u8"]).view(torch.float8_e4m3fn),
        torch.from_numpy(z["cache_i8"]),
        torch.from_numpy(z["weights"]),
        torch.from_numpy(z["seq_lens"]),
        torch.from_numpy(z["block_table"]))
    return inp, torch.from_numpy(z["topk_indices"]), z


def load_attention_golden(name):
    z = np.load(GOLDEN / f"{name}.npz")
    bf = lambda k: torch.from_numpy(z[k]).view(torch.bfloat16)
    inp = wl.AttentionInputs(bf("q_nope_u16"), bf("q_pe_u16"), bf("ckv_u16"), bf("kpe_u16"),
                             torch.from_numpy(z["sparse_indices"]), float(z["sm_scale"]))
    return inp, bf("output_u16"), torch.from_numpy(z["lse"])


def assert_topk_matches(inp, got_indices, ref_rows=None, label=""):
    """Apply the indexer acceptance rule row by row against oracle score rows."""
    got = got_indices.cpu()
    cpu = inp.to("cpu")
    if ref_rows is None:
        ref_rows = oracle.indexer_scores(*cpu.args())
    modes = []
    for b, row in enumerate(ref_rows):
        info = oracle.check_topk_row(row, cpu.block_table[b], int(cpu.seq_lens[b]), got[b])
        assert info["ok"], f"{label} request {b}: {info}"
        modes.append(info.get("mode"))
    return modes


def assert_attention_close(out, lse, ref_out, ref_lse, label=""):
    out = out.float().cpu()
    lse = lse.float().cpu()
    ref_out = ref_out.float()
    ref_lse = ref_lse.float()
    blank = torch.isinf(ref_lse) & (ref_lse < 0)          # rows with no valid index
    assert torch.equal(torch.isinf(lse) & (lse < 0), blank), f"{label}: -inf LSE pattern differs"
    keep = ~blank
    assert torch.allclose(lse[keep], ref_lse[keep], atol=LSE_TOL, rtol=LSE_TOL), \
        f"{label}: lse max err {(lse[keep] - ref_lse[keep]).abs().max()}"
    # fully masked rows: the reference's softmax yields NaN, the kernels define 0
    assert (out[blank] == 0).all(), f"{label}: masked rows must be zero"
    err = (out[keep] - ref_out[keep]).abs()
    bound = ATT_ATOL + ATT_RTOL * ref_out[keep].abs()
    assert (err <= bound).all(), f"{label}: output max err {err.max()}"


def indexer_inputs_from_scores(rows, lens, seed=0, device="cpu"):
    """Indexer inputs whose score rows are EXACTLY the given fp32 rows (any sign, +-0, inf, NaN).

    Two heads carry everything: q[0] = +e0, q[1] = -e0, w[0] = +1, w[1] = -1, all else zero; token t
    holds the key sign(x_t) * e0 with the per-token scale |x_t|.  Then (reference order, scale
    inside the key: indexer_baseline.py:36,75-80) relu(x)*1 + relu(-x)*(-1) = x, and (kernel order,
    scale after the head sum) |x| * (+1 or -1) = x, both without rounding."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    lens = [int(n) for n in lens]
    batch = len(lens)
    need = [(n + 63) // 64 for n in lens]
    total = max(sum(need), 1)
    max_pages = max(1, max(need))
    perm = torch.randperm(total, generator=gen).to(torch.int32)
    table = torch.zeros(batch, max_pages, dtype=torch.int32)
    raw = torch.zeros(total, wl.PAGE_BYTES, dtype=torch.uint8)
    data = raw[:, : 64 * 128].view(total, 64, 128)
    scales = torch.zeros(total, 64, dtype=torch.float32)
    plus_one = int(torch.tensor([1.0]).to(torch.float8_e4m3fn).view(torch.uint8))
    minus_one = int(torch.tensor([-1.0]).to(torch.float8_e4m3fn).view(torch.uint8))
    at = 0
    for b, n in enumerate(need):
        pages = perm[at:at + n].long()
        table[b, :n] = perm[at:at + n]
        at += n
        x = torch.zeros(n * 64, dtype=torch.float32)
        x[: lens[b]] = rows[b][: lens[b]].float()
        negative = torch.signbit(x)
        data[pages, :, 0] = torch.where(negative, minus_one, plus_one).to(torch.uint8).view(n, 64)
        scales[pages] = x.abs().view(n, 64)
    raw[:, 64 * 128:] = scales.view(torch.uint8).reshape(total, -1)
    cache = raw.view(torch.int8).reshape(total, 64, 1, 132)
    q = torch.zeros(batch, 64, 128)
    q[:, 0, 0] = 1.0
    q[:, 1, 0] = -1.0
    w = torch.zeros(batch, 64)
    w[:, 0] = 1.0
    w[:, 1] = -1.0
    inp = wl.IndexerInputs(q.to(torch.float8_e4m3fn), cache, w, torch.tensor(lens, dtype=torch.int32), table)
    return inp.to(device)
