"""Randomised shapes through the C ABI against the oracle, one shared workspace across all calls:
batch sizes, context lengths and valid-index counts change from call to call the way they do in a
serving loop, which is what exposes state that leaks from one call into the next."""
import os
import random

import pytest
import torch

import dsa_oracle as oracle
from auto_gpu_kernel_b200 import indexer, sparse_attention, inputs as wl, workspace
from helpers import assert_attention_close, assert_topk_matches

pytestmark = pytest.mark.gpu

# DSA_TEST_SEEDS=<n> widens the sweep (soak runs); the default keeps the suite short.
SEEDS = range(int(os.environ.get("DSA_TEST_SEEDS", "10")))

SPECIAL_LENGTHS = [0, 1, 63, 64, 65, 127, 128, 129, 2047, 2048, 2049, 2111, 4096, 45056, 45057]


def _random_lengths(rng, batch, longest):
    lens = []
    for _ in range(batch):
        if rng.random() < 0.35:
            lens.append(min(rng.choice(SPECIAL_LENGTHS), longest))
        else:
            lens.append(rng.randint(0, longest))
    return lens


@pytest.mark.parametrize("seed", SEEDS)
def test_indexer_random_batches(cuda, seed):
    rng = random.Random(1000 + seed)
    for call in range(5):
        batch = rng.choice([1, 2, 3, 5, 8, 17, 33, 40, 75])
        longest = rng.choice([300, 2048, 5000, 20000, 70000 if batch <= 8 else 9000])
        lens = _random_lengths(rng, batch, longest)
        inp = wl.make_indexer_inputs(lens, seed=rng.randrange(1 << 30), device=cuda)
        out = indexer.run(*inp.args())
        workspace.check_status(cuda)
        rows = [r.cpu() for r in oracle.indexer_scores(*inp.args())]
        assert_topk_matches(inp, out, rows, label=f"seed {seed} call {call} B={batch} lens={lens[:6]}")


@pytest.mark.parametrize("seed", SEEDS)
def test_attention_random_token_counts(cuda, seed):
    rng = random.Random(2000 + seed)
    for call in range(5):
        tokens = rng.choice([1, 2, 3, 7, 15, 16, 31, 40, 64, 74, 75, 100, 128, 148, 149, 200])
        lens = [rng.choice([5, 64, 100, 2048, 2049, 3000, 6000]) for _ in range(tokens)]
        inp = wl.make_attention_inputs(lens, seed=rng.randrange(1 << 30), device=cuda,
                                       pad_tail=rng.choice([0, 0, 7, 1000, 2040]))
        idx = inp.sparse_indices.clone()
        for t in range(tokens):                       # holes anywhere, sometimes a blank row
            r = rng.random()
            if r < 0.15:
                idx[t, rng.randrange(2048)::rng.choice([2, 3, 64])] = -1
            elif r < 0.2:
                idx[t] = -1
        inp.sparse_indices = idx
        out, lse = sparse_attention.run(*inp.args())
        workspace.check_status(cuda)
        ref_out, ref_lse = oracle.sparse_attention(*inp.args(), output=torch.empty_like(out),
                                                   lse=torch.empty_like(lse))
        assert_attention_close(out, lse, ref_out.cpu(), ref_lse.cpu(),
                               label=f"seed {seed} call {call} T={tokens}")
