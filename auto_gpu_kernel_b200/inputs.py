"""Seeded synthetic workloads for the two DSA definitions.

The contest trace set the reference is evaluated on is not redistributable with this repository,
so the tests and the benchmark build inputs with the same shapes, dtypes, layouts and value
distributions instead:

  * index-key cache: keys ~ N(0,1), per-token absmax / 448 scale, e4m3 data, packed into
    [num_pages, 64, 1, 132] int8 pages of 8192 data bytes followed by 64 fp32 scales (the layout
    unpacked by indexer_baseline.py:16-36 of the reference);
  * q ~ N(0,1) cast to e4m3, weights ~ N(0,1) * (64*128)^-0.5;
  * block_table = a random permutation of the pages each request needs, unused tail 0;
  * attention: q_nope/q_pe ~ N(0,1)*0.1 bf16, ckv/kpe ~ N(0,1) bf16, sparse_indices = distinct
    random global slots inside the request's pages, -1 padded when the request is shorter.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

PAGE_SIZE = 64
INDEX_HEADS = 64
INDEX_DIM = 128
PAGE_BYTES = PAGE_SIZE * (INDEX_DIM + 4)
TOPK = 2048
ATTN_HEADS = 16
CKV_DIM = 512
KPE_DIM = 64
FP8_MAX = 448.0


def pack_index_pages(keys_fp32: torch.Tensor) -> torch.Tensor:
    """Quantise fp32 keys [P,64,128] per token (absmax/448) and pack to [P,64,1,132] int8."""
    pages = keys_fp32.shape[0]
    amax = keys_fp32.abs().amax(dim=-1).clamp_min(1e-12)
    scale = (amax / FP8_MAX).to(torch.float32)                       # [P,64]
    data = (keys_fp32 / scale.unsqueeze(-1)).to(torch.float8_e4m3fn)  # [P,64,128]
    raw = torch.empty(pages, PAGE_BYTES, dtype=torch.uint8, device=keys_fp32.device)
    raw[:, : PAGE_SIZE * INDEX_DIM] = data.view(torch.uint8).reshape(pages, -1)
    raw[:, PAGE_SIZE * INDEX_DIM:] = scale.contiguous().view(torch.uint8).reshape(pages, -1)
    return raw.view(torch.int8).reshape(pages, PAGE_SIZE, 1, INDEX_DIM + 4)


@dataclass
class IndexerInputs:
    q_index_fp8: torch.Tensor        # [B,64,128] float8_e4m3fn
    k_index_cache_fp8: torch.Tensor  # [P,64,1,132] int8
    weights: torch.Tensor            # [B,64] float32
    seq_lens: torch.Tensor           # [B] int32
    block_table: torch.Tensor        # [B,max_pages] int32

    def args(self):
        return (self.q_index_fp8, self.k_index_cache_fp8, self.weights, self.seq_lens,
                self.block_table)

    def to(self, device):
        return IndexerInputs(*[t.to(device) for t in self.args()])


def make_indexer_inputs(seq_lens, seed=0, device="cpu", extra_pages=0, chunk_pages=4096):
    """One request per entry of `seq_lens`; pages are private to a request and shuffled."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    lens = [int(x) for x in seq_lens]
    batch = len(lens)
    need = [(n + PAGE_SIZE - 1) // PAGE_SIZE for n in lens]
    total = sum(need) + extra_pages
    max_pages = max(1, max(need) if need else 1)
    perm = torch.randperm(max(total, 1), generator=gen).to(torch.int32)
    table = torch.zeros(batch, max_pages, dtype=torch.int32)
    at = 0
    for b, n in enumerate(need):
        table[b, :n] = perm[at:at + n]
        at += n
    dev = torch.device(device)
    dgen = torch.Generator(device=dev).manual_seed(seed + 1)
    cache = torch.empty(max(total, 1), PAGE_SIZE, 1, INDEX_DIM + 4, dtype=torch.int8, device=dev)
    for lo in range(0, max(total, 1), chunk_pages):
        hi = min(lo + chunk_pages, max(total, 1))
        keys = torch.randn(hi - lo, PAGE_SIZE, INDEX_DIM, generator=dgen, device=dev)
        cache[lo:hi] = pack_index_pages(keys)
    q = torch.randn(batch, INDEX_HEADS, INDEX_DIM, generator=dgen, device=dev).to(torch.float8_e4m3fn)
    w = torch.randn(batch, INDEX_HEADS, generator=dgen, device=dev) * (INDEX_HEADS * INDEX_DIM) ** -0.5
    return IndexerInputs(q, cache, w.to(torch.float32),
                         torch.tensor(lens, dtype=torch.int32, device=dev), table.to(dev))


def make_shared_prefix_indexer_inputs(prefix_len, chunk_len, seed=0, device="cpu"):
    """Chunked prefill: `chunk_len` query rows over one request's pages; row i sees the first
    prefix_len + i + 1 tokens.  All rows carry the same block_table row."""
    total_len = prefix_len + chunk_len
    base = make_indexer_inputs([total_len], seed=seed, device=device)
    dev = torch.device(device)
    dgen = torch.Generator(device=dev).manual_seed(seed + 7)
    q = torch.randn(chunk_len, INDEX_HEADS, INDEX_DIM, generator=dgen, device=dev).to(torch.float8_e4m3fn)
    w = torch.randn(chunk_len, INDEX_HEADS, generator=dgen, device=dev) * (INDEX_HEADS * INDEX_DIM) ** -0.5
    lens = torch.arange(prefix_len + 1, total_len + 1, dtype=torch.int32, device=dev)
    table = base.block_table.expand(chunk_len, -1).contiguous()
    return IndexerInputs(q, base.k_index_cache_fp8, w.to(torch.float32), lens, table)


@dataclass
class AttentionInputs:
    q_nope: torch.Tensor          # [T,16,512] bf16
    q_pe: torch.Tensor            # [T,16,64] bf16
    ckv_cache: torch.Tensor       # [P,64,512] bf16
    kpe_cache: torch.Tensor       # [P,64,64] bf16
    sparse_indices: torch.Tensor  # [T,2048] int32
    sm_scale: float

    def args(self):
        return (self.q_nope, self.q_pe, self.ckv_cache, self.kpe_cache, self.sparse_indices,
                self.sm_scale)

    def to(self, device):
        t = [x.to(device) for x in self.args()[:5]]
        return AttentionInputs(*t, self.sm_scale)


def make_attention_inputs(seq_lens, seed=0, device="cpu", heads=ATTN_HEADS, pad_tail=0,
                          chunk_pages=2048):
    """One query token per entry of `seq_lens`.  Each token owns ceil(L/64) shuffled pages and
    selects min(2048, L) distinct slots among its first L tokens; `pad_tail` forces that many
    extra -1 entries at the end of every row."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    lens = [int(x) for x in seq_lens]
    tokens = len(lens)
    need = [(n + PAGE_SIZE - 1) // PAGE_SIZE for n in lens]
    total = max(sum(need), 1)
    perm = torch.randperm(total, generator=gen)
    idx = torch.full((tokens, TOPK), -1, dtype=torch.int32)
    at = 0
    for t, (n_tok, n_pg) in enumerate(zip(lens, need)):
        pages = perm[at:at + n_pg]
        at += n_pg
        k = max(0, min(TOPK - pad_tail, n_tok))
        local = torch.randperm(n_tok, generator=gen)[:k]
        idx[t, :k] = (pages[local // PAGE_SIZE] * PAGE_SIZE + local % PAGE_SIZE).to(torch.int32)
    dev = torch.device(device)
    dgen = torch.Generator(device=dev).manual_seed(seed + 1)
    ckv = torch.empty(total, PAGE_SIZE, CKV_DIM, dtype=torch.bfloat16, device=dev)
    kpe = torch.empty(total, PAGE_SIZE, KPE_DIM, dtype=torch.bfloat16, device=dev)
    for lo in range(0, total, chunk_pages):
        hi = min(lo + chunk_pages, total)
        ckv[lo:hi] = torch.randn(hi - lo, PAGE_SIZE, CKV_DIM, generator=dgen, device=dev).to(torch.bfloat16)
        kpe[lo:hi] = torch.randn(hi - lo, PAGE_SIZE, KPE_DIM, generator=dgen, device=dev).to(torch.bfloat16)
    qn = (torch.randn(tokens, heads, CKV_DIM, generator=dgen, device=dev) * 0.1).to(torch.bfloat16)
    qp = (torch.randn(tokens, heads, KPE_DIM, generator=dgen, device=dev) * 0.1).to(torch.bfloat16)
    return AttentionInputs(qn, qp, ckv, kpe, idx.to(dev), 1.0 / math.sqrt(192.0))


def uniform_lengths(count, lo, hi, seed=0):
    """`count` sequence lengths uniform in [lo, hi], seeded."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randint(lo, hi + 1, (count,), generator=gen).tolist()


@dataclass
class DecodeBlockInputs:
    """One decode step of the DSA block: the indexer picks 2048 slots per request, attention reads
    them from ckv/kpe caches that share the index-key cache's page numbering."""
    indexer: IndexerInputs
    q_nope: torch.Tensor
    q_pe: torch.Tensor
    ckv_cache: torch.Tensor
    kpe_cache: torch.Tensor
    sm_scale: float


def make_decode_block_inputs(seq_lens, seed=0, device="cpu", heads=ATTN_HEADS, chunk_pages=2048):
    idx = make_indexer_inputs(seq_lens, seed=seed, device=device)
    pages = idx.k_index_cache_fp8.shape[0]
    dev = torch.device(device)
    dgen = torch.Generator(device=dev).manual_seed(seed + 3)
    ckv = torch.empty(pages, PAGE_SIZE, CKV_DIM, dtype=torch.bfloat16, device=dev)
    kpe = torch.empty(pages, PAGE_SIZE, KPE_DIM, dtype=torch.bfloat16, device=dev)
    for lo in range(0, pages, chunk_pages):
        hi = min(lo + chunk_pages, pages)
        ckv[lo:hi] = torch.randn(hi - lo, PAGE_SIZE, CKV_DIM, generator=dgen, device=dev).to(torch.bfloat16)
        kpe[lo:hi] = torch.randn(hi - lo, PAGE_SIZE, KPE_DIM, generator=dgen, device=dev).to(torch.bfloat16)
    tokens = len(seq_lens)
    qn = (torch.randn(tokens, heads, CKV_DIM, generator=dgen, device=dev) * 0.1).to(torch.bfloat16)
    qp = (torch.randn(tokens, heads, KPE_DIM, generator=dgen, device=dev) * 0.1).to(torch.bfloat16)
    return DecodeBlockInputs(idx, qn, qp, ckv, kpe, 1.0 / math.sqrt(192.0))
