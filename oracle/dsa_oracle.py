"""CPU oracle for the DeepSeek Sparse Attention hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, on CPU tensors, the arithmetic of the reference repository's two PyTorch
definitions:

  * the FP8 top-k indexer  -- archive/dsa_topk_indexer_fp8_h64_d128_topk2048_ps64/solution/triton/
                              indexer_baseline.py:16-36 (page unpack + dequantise) and :39-90 (score,
                              top-k, page -> global slot remap, -1 padding);
  * sparse MLA attention   -- archive/dsa_sparse_attention_h16_ckv512_kpe64_topk2048_ps64/solution/
                              triton/sparse_baseline.py:12-45 (gather, fp32 logits, -inf mask,
                              base-2 LSE, softmax @ V -> bf16).

It is the checker for the CUDA kernels and the timed CPU baseline of the benchmark.  Nothing in the
shipped package imports it: only the tests, the smoke check and the benchmark's CPU legs do.

Parity pin: the reference holds no golden vectors for this path, so the oracle is pinned against
outputs of the reference's own two files, imported and executed on CPU by
tests/golden/make_golden.py; the resulting fixtures live in tests/golden/*.npz and
tests/test_oracle_golden.py checks this module against them.
"""
from __future__ import annotations

import math

import numpy as np
import torch

PAGE_SIZE = 64          # tokens per page (both caches)
INDEX_HEADS = 64        # indexer heads
INDEX_DIM = 128         # indexer head dim (fp8 bytes per cached token)
PAGE_DATA_BYTES = PAGE_SIZE * INDEX_DIM            # 8192 fp8 bytes, token-major
PAGE_BYTES = PAGE_SIZE * (INDEX_DIM + 4)           # 8448: data then 64 fp32 scales
TOPK = 2048


# ----------------------------------------------------------------------------------------------
# FP8 e4m3fn decode, written out so the byte format is stated here and not only inside torch.
# ----------------------------------------------------------------------------------------------
def e4m3fn_table() -> np.ndarray:
    """256-entry float32 table of the e4m3fn code points (bias 7, no inf, 0x7f/0xff = NaN)."""
    out = np.empty(256, dtype=np.float32)
    for code in range(256):
        sign = -1.0 if code & 0x80 else 1.0
        exp = (code >> 3) & 0xF
        man = code & 0x7
        if exp == 0xF and man == 0x7:
            val = float("nan")
        elif exp == 0:
            val = sign * (man / 8.0) * 2.0 ** (-6)
        else:
            val = sign * (1.0 + man / 8.0) * 2.0 ** (exp - 7)
        out[code] = val
    return out


def unpack_index_pages(k_index_cache_fp8: torch.Tensor, pages: torch.Tensor | None = None):
    """Split packed index-key pages into (fp8 data as float32 [n,64,128], scale float32 [n,64]).

    Page layout (indexer_baseline.py:16-36): each page is 8448 bytes; bytes [0,8192) hold the
    64x128 e4m3 keys token-major, bytes [8192,8448) hold the 64 per-token fp32 scales.
    `pages` optionally selects a subset of pages (int64 indices) before decoding.
    """
    raw = k_index_cache_fp8.view(torch.uint8).reshape(k_index_cache_fp8.shape[0], PAGE_BYTES)
    if pages is not None:
        raw = raw[pages]
    n = raw.shape[0]
    data = raw[:, :PAGE_DATA_BYTES].contiguous().view(torch.float8_e4m3fn)
    data = data.reshape(n, PAGE_SIZE, INDEX_DIM).to(torch.float32)
    scale = raw[:, PAGE_DATA_BYTES:].contiguous().view(torch.float32).reshape(n, PAGE_SIZE)
    return data, scale


def dequant_index_pages(k_index_cache_fp8: torch.Tensor, pages: torch.Tensor | None = None):
    """fp32 keys [n,64,128] = e4m3 value * per-token scale (indexer_baseline.py:36)."""
    data, scale = unpack_index_pages(k_index_cache_fp8, pages)
    return data * scale.unsqueeze(-1)


# ----------------------------------------------------------------------------------------------
# Cache writers (the producers of the inputs above).  The reference ships no writer; this restates
# the layout its reader (indexer_baseline.py:16-36) unpacks, with the e4m3 rounding written out.
# ----------------------------------------------------------------------------------------------
def quantize_e4m3fn(values: np.ndarray) -> np.ndarray:
    """float32 -> e4m3fn code (uint8): round to nearest, ties to the even code, saturating at 448."""
    table = e4m3fn_table()
    pos = table[:0x7F].astype(np.float64)                 # codes 0x00..0x7e: 0 .. 448, ascending
    mag = np.minimum(np.abs(values.astype(np.float64)), 448.0)
    hi = np.clip(np.searchsorted(pos, mag, side="left"), 1, len(pos) - 1)
    lo = hi - 1
    d_lo, d_hi = mag - pos[lo], pos[hi] - mag
    pick_hi = (d_hi < d_lo) | ((d_hi == d_lo) & (hi % 2 == 0))
    code = np.where(pick_hi, hi, lo).astype(np.uint8)
    code = np.where(mag == 0.0, 0, code).astype(np.uint8)
    sign = (np.signbit(values).astype(np.uint8) << 7)
    return code | sign


def write_index_keys(keys: torch.Tensor, slots: torch.Tensor, k_index_cache_fp8: torch.Tensor):
    """Quantise keys [n,128] per token (scale = max(absmax, 1e-12) / 448, data = e4m3(key / scale))
    and store token t at global slot slots[t] (-1 skips) of the packed pages, in place."""
    raw = k_index_cache_fp8.view(torch.uint8).reshape(k_index_cache_fp8.shape[0], PAGE_BYTES)
    k = keys.to(torch.float32).numpy()
    amax = np.maximum(np.abs(k).max(axis=1), np.float32(1e-12)).astype(np.float32)
    scale = (amax / np.float32(448.0)).astype(np.float32)
    codes = quantize_e4m3fn((k / scale[:, None]).astype(np.float32))
    for t, slot in enumerate(slots.tolist()):
        if slot < 0:
            continue
        page, pos = divmod(slot, PAGE_SIZE)
        raw[page, pos * INDEX_DIM:(pos + 1) * INDEX_DIM] = torch.from_numpy(codes[t])
        at = PAGE_DATA_BYTES + 4 * pos
        raw[page, at:at + 4] = torch.from_numpy(scale[t:t + 1].view(np.uint8))
    return k_index_cache_fp8


def append_kv(ckv, kpe, slots, ckv_cache, kpe_cache):
    """ckv_cache.flat[slot] = ckv[t], kpe_cache.flat[slot] = kpe[t] for slot = slots[t] >= 0 (the
    flat views of sparse_baseline.py:18-19), in place."""
    flat_c = ckv_cache.view(-1, ckv_cache.shape[-1])
    flat_p = kpe_cache.view(-1, kpe_cache.shape[-1])
    keep = slots >= 0
    flat_c[slots[keep].long()] = ckv[keep]
    flat_p[slots[keep].long()] = kpe[keep]
    return ckv_cache, kpe_cache


@torch.no_grad()
def indexer_scores(q_index_fp8, k_index_cache_fp8, weights, seq_lens, block_table):
    """Per-request fp32 score rows, list of 1-D tensors of length seq_len[b].

    score[t] = sum_h w[b,h] * relu(q[b,h] . K[t]) with K dequantised first, the order of operations
    of indexer_baseline.py:75-80 (fp32 matmul, relu, scale by w, sum over heads).
    """
    q = q_index_fp8.to(torch.float32)
    rows = []
    for b in range(q.shape[0]):
        length = int(seq_lens[b])
        if length == 0:
            rows.append(torch.empty(0, dtype=torch.float32))
            continue
        n_pages = (length + PAGE_SIZE - 1) // PAGE_SIZE
        pages = block_table[b, :n_pages].to(torch.long)
        keys = dequant_index_pages(k_index_cache_fp8, pages).reshape(-1, INDEX_DIM)[:length]
        s = q[b] @ keys.T                                     # [64, L]
        s = torch.relu(s) * weights[b].to(torch.float32)[:, None]
        rows.append(s.sum(dim=0))
    return rows


@torch.no_grad()
def indexer_topk(q_index_fp8, k_index_cache_fp8, weights, seq_lens, block_table,
                 topk_indices=None, return_scores=False):
    """Top-2048 global slot ids per request, -1 padded (indexer_baseline.py:60, :82-90).

    The slot id of local token i of request b is block_table[b, i // 64] * 64 + i % 64.
    Order inside a row follows torch.topk (descending score); only the set is contractual.
    """
    batch = q_index_fp8.shape[0]
    if topk_indices is None:
        topk_indices = torch.empty(batch, TOPK, dtype=torch.int32)
    topk_indices.fill_(-1)
    rows = indexer_scores(q_index_fp8, k_index_cache_fp8, weights, seq_lens, block_table)
    for b, s in enumerate(rows):
        length = s.numel()
        if length == 0:
            continue
        k = min(TOPK, length)
        _, local = torch.topk(s, k)
        page = block_table[b].to(torch.long)[local // PAGE_SIZE]
        topk_indices[b, :k] = (page * PAGE_SIZE + local % PAGE_SIZE).to(torch.int32)
    if return_scores:
        return topk_indices, rows
    return topk_indices


def slots_to_local(block_table_row: torch.Tensor, seq_len: int, slots: torch.Tensor) -> torch.Tensor:
    """Invert the page remap for one request: global slot id -> local token position, or -1 when
    the slot does not belong to the request's first ceil(seq_len/64) pages / first seq_len tokens."""
    n_pages = (seq_len + PAGE_SIZE - 1) // PAGE_SIZE
    pages = block_table_row[:n_pages].to(torch.long)
    lut = {int(p): i for i, p in enumerate(pages.tolist())}
    out = []
    for s in slots.tolist():
        if s < 0:
            out.append(-1)
            continue
        i = lut.get(s // PAGE_SIZE, -1)
        pos = i * PAGE_SIZE + s % PAGE_SIZE if i >= 0 else -1
        out.append(pos if 0 <= pos < seq_len else -1)
    return torch.tensor(out, dtype=torch.long)


def check_topk_row(ref_scores: torch.Tensor, block_table_row: torch.Tensor, seq_len: int,
                   got_slots: torch.Tensor, gap_rel: float = 1e-3, recall_min: float = 0.999,
                   score_tol: float = 1e-3) -> dict:
    """Acceptance rule for one indexer output row against the oracle's score row.

    * structure: exactly min(2048, seq_len) non-negative entries, all distinct, all belonging to
      the request, every other entry -1;
    * if the oracle's k-th and (k+1)-th largest scores differ by more than `gap_rel` relative,
      the selected set must equal the oracle's set exactly;
    * otherwise recall >= `recall_min` and the sorted selected scores must match the oracle's
      sorted top-k scores within `score_tol` (relative to the largest magnitude in the row);
      recall counts a selected element as a hit when it is in the oracle's set or its oracle
      score lies within `score_tol` (relative) of the k-th score, so that elements tied with the
      boundary are interchangeable.
    Returns a dict with ok flag and diagnostics.
    """
    k = min(TOPK, seq_len)
    got = got_slots.to(torch.long)
    valid = got[got >= 0]
    info = {"ok": False, "k": k, "n_valid": int(valid.numel())}
    if valid.numel() != k or (got < 0).sum() != got.numel() - k:
        info["why"] = "wrong number of valid entries"
        return info
    local = slots_to_local(block_table_row, seq_len, valid)
    if (local < 0).any():
        info["why"] = "slot outside the request"
        return info
    if torch.unique(local).numel() != k:
        info["why"] = "duplicate slots"
        return info
    if k == seq_len:
        info["ok"] = True
        info["mode"] = "all"
        return info
    order = torch.argsort(ref_scores, descending=True, stable=True)
    ref_set = set(order[:k].tolist())
    got_set = set(local.tolist())
    s_sorted = ref_scores[order]
    kth, nxt = float(s_sorted[k - 1]), float(s_sorted[k])
    gap = (kth - nxt) / max(abs(kth), 1e-30)
    near = ref_scores[local] >= kth - score_tol * max(abs(kth), 1e-30)
    hits = sum(1 for pos, ok in zip(local.tolist(), near.tolist()) if ok or pos in ref_set)
    recall = hits / k
    info.update(gap=gap, recall=recall, strict_recall=len(ref_set & got_set) / k)
    if gap > gap_rel:
        info["mode"] = "exact"
        info["ok"] = ref_set == got_set
        if not info["ok"]:
            info["why"] = "set differs although the boundary gap is wide"
        return info
    info["mode"] = "tolerant"
    got_scores = torch.sort(ref_scores[local], descending=True).values
    ref_top = s_sorted[:k]
    denom = max(float(ref_top.abs().max()), 1e-30)
    err = float((got_scores - ref_top).abs().max()) / denom
    info["score_err"] = err
    info["ok"] = recall >= recall_min and err <= score_tol
    if not info["ok"]:
        info["why"] = "recall or selected-score tolerance"
    return info


@torch.no_grad()
def sparse_attention(q_nope, q_pe, ckv_cache, kpe_cache, sparse_indices, sm_scale,
                     output=None, lse=None):
    """Sparse MLA attention over the selected rows (sparse_baseline.py:12-45).

    logits[t,h,k] = (q_nope[t,h].ckv[idx[t,k]] + q_pe[t,h].kpe[idx[t,k]]) * sm_scale, idx == -1
    masked to -inf; lse = logsumexp(logits) / ln 2; out = softmax(logits) @ ckv rows -> bf16.
    A row whose indices are all -1 gives lse = -inf and NaN output, exactly as the reference's
    softmax of all -inf does.
    """
    tokens, heads, d_ckv = q_nope.shape
    d_kpe = q_pe.shape[-1]
    topk = sparse_indices.shape[-1]
    if output is None:
        output = torch.empty(tokens, heads, d_ckv, dtype=torch.bfloat16)
    if lse is None:
        lse = torch.empty(tokens, heads, dtype=torch.float32)
    flat_c = ckv_cache.reshape(-1, d_ckv)
    flat_p = kpe_cache.reshape(-1, d_kpe)
    keep = sparse_indices != -1
    rows = sparse_indices.clamp(min=0).to(torch.long).reshape(-1)
    kc = flat_c[rows].reshape(tokens, topk, d_ckv).to(torch.float32)
    kp = flat_p[rows].reshape(tokens, topk, d_kpe).to(torch.float32)
    logits = torch.bmm(q_nope.to(torch.float32), kc.transpose(1, 2))
    logits = logits + torch.bmm(q_pe.to(torch.float32), kp.transpose(1, 2))
    logits = logits * sm_scale
    logits.masked_fill_(~keep.unsqueeze(1), float("-inf"))
    lse.copy_(torch.logsumexp(logits, dim=-1) / math.log(2.0))
    probs = torch.softmax(logits, dim=-1)
    output.copy_(torch.bmm(probs, kc).to(torch.bfloat16))
    return output, lse
