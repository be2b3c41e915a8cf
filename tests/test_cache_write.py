"""Cache writers: oracle against the golden fixture (CPU), CUDA writers against the oracle (GPU),
and the written caches read back by the path's own kernels."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import dsa_oracle as oracle

GOLDEN = Path(__file__).resolve().parent / "golden"


def _golden():
    z = np.load(GOLDEN / "cache_write.npz")
    return (torch.from_numpy(z["keys"]), torch.from_numpy(z["slots"]),
            torch.from_numpy(z["cache_i8"]), torch.from_numpy(z["dequant"]))


def test_e4m3_rounding_matches_torch_cast():
    gen = torch.Generator().manual_seed(0)
    x = torch.cat([torch.randn(20000, generator=gen) * 100, torch.randn(20000, generator=gen) * 0.01,
                   torch.linspace(-448, 448, 4097), torch.tensor([0.0, -0.0, 447.9, 448.0, 1e-9])])
    x = x.clamp(-448, 448)
    want = x.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    got = oracle.quantize_e4m3fn(x.numpy())
    assert np.array_equal(got, want)
    # every finite code point is a fixed point of the rounding
    table = oracle.e4m3fn_table()
    finite = np.array([c for c in range(256) if not np.isnan(table[c])], dtype=np.uint8)
    back = oracle.quantize_e4m3fn(table[finite])
    assert np.array_equal(back & 0x7F, finite & 0x7F)


def test_oracle_writer_against_golden_bytes_and_reference_reader():
    keys, slots, want_cache, want_dense = _golden()
    cache = torch.zeros_like(want_cache)
    oracle.write_index_keys(keys, slots, cache)
    assert torch.equal(cache, want_cache)
    dense = oracle.dequant_index_pages(cache)
    assert torch.equal(dense, want_dense)
    # what was written reads back as the key within e4m3 resolution (3 mantissa bits) of its scale
    for t in (0, 1, 2, 3, 4, 50, 202):
        page, pos = divmod(int(slots[t]), 64)
        amax = keys[t].abs().max().clamp_min(1e-12)
        assert (dense[page, pos] - keys[t]).abs().max() <= amax / 16 + 1e-30
    assert int(slots[7]) == -1


def test_oracle_append_kv():
    gen = torch.Generator().manual_seed(1)
    ckv = torch.randn(10, 512, generator=gen).to(torch.bfloat16)
    kpe = torch.randn(10, 64, generator=gen).to(torch.bfloat16)
    slots = torch.tensor([5, 64, -1, 0, 127, 3, 70, 71, 72, 1], dtype=torch.int32)
    cc, pc = torch.zeros(2, 64, 512, dtype=torch.bfloat16), torch.zeros(2, 64, 64, dtype=torch.bfloat16)
    oracle.append_kv(ckv, kpe, slots, cc, pc)
    assert torch.equal(cc.view(-1, 512)[64], ckv[1]) and torch.equal(pc.view(-1, 64)[127], kpe[4])
    assert cc.view(-1, 512)[2].abs().sum() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gpu_index_cache_write_bit_exact(dtype):
    from auto_gpu_kernel_b200 import cache_write, workspace
    dev = torch.device("cuda", 0)
    keys, slots, want_cache, _ = _golden()
    if dtype == torch.bfloat16:
        keys = keys.to(torch.bfloat16)
        want_cache = oracle.write_index_keys(keys, slots, torch.zeros_like(want_cache))
    cache = torch.zeros_like(want_cache, device=dev)
    cache_write.write_index_keys(keys.to(dev), slots.to(dev), cache)
    torch.cuda.synchronize()
    assert torch.equal(cache.cpu(), want_cache)
    assert workspace.check_status(dev) == 0


@pytest.mark.gpu
def test_gpu_writers_large_and_strided():
    from auto_gpu_kernel_b200 import cache_write, workspace
    dev = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(3)
    pages, n = 300, 9000
    wide = torch.randn(n, 160, generator=gen)                  # strided rows: 128 of 160 columns
    keys = wide[:, 16:144]
    slots = torch.randperm(pages * 64, generator=gen)[:n].to(torch.int32)
    slots[::97] = -1
    want = oracle.write_index_keys(keys, slots, torch.zeros(pages, 64, 1, 132, dtype=torch.int8))
    cache = torch.zeros(pages, 64, 1, 132, dtype=torch.int8, device=dev)
    cache_write.write_index_keys(wide.to(dev)[:, 16:144], slots.to(dev), cache)
    assert torch.equal(cache.cpu(), want)

    ckv = torch.randn(n, 512, generator=gen).to(torch.bfloat16)
    kpe = torch.randn(n, 64, generator=gen).to(torch.bfloat16)
    wc, wp = oracle.append_kv(ckv, kpe, slots, torch.zeros(pages, 64, 512, dtype=torch.bfloat16),
                              torch.zeros(pages, 64, 64, dtype=torch.bfloat16))
    cc = torch.zeros(pages, 64, 512, dtype=torch.bfloat16, device=dev)
    pc = torch.zeros(pages, 64, 64, dtype=torch.bfloat16, device=dev)
    cache_write.append_kv(ckv.to(dev), kpe.to(dev), slots.to(dev), cc, pc)
    assert torch.equal(cc.cpu().view(torch.int16), wc.view(torch.int16))
    assert torch.equal(pc.cpu().view(torch.int16), wp.view(torch.int16))
    assert workspace.check_status(dev) == 0


@pytest.mark.gpu
def test_gpu_bad_slot_is_skipped_and_reported():
    from auto_gpu_kernel_b200 import cache_write, workspace
    dev = torch.device("cuda", 0)
    keys = torch.ones(3, 128, device=dev)
    slots = torch.tensor([0, 64 * 2, 1], dtype=torch.int32, device=dev)   # slot 128 is past 2 pages
    cache = torch.zeros(2, 64, 1, 132, dtype=torch.int8, device=dev)
    cache_write.write_index_keys(keys, slots, cache)
    with pytest.raises(RuntimeError, match="outside"):
        workspace.check_status(dev)
    assert workspace.check_status(dev) == 0
    data, scale = oracle.unpack_index_pages(cache.cpu())
    assert scale[0, 0] == pytest.approx(1 / 448) and scale[0, 1] == pytest.approx(1 / 448)
    assert scale[1].abs().sum() == 0


@pytest.mark.gpu
def test_gpu_block_from_raw_activations():
    """Writers feed the path: caches written by the CUDA writers give the same indexer and
    attention results as caches packed on the host."""
    from auto_gpu_kernel_b200 import cache_write, indexer, sparse_attention, workspace, inputs as wl
    dev = torch.device("cuda", 0)
    lens = [3000, 2500, 4100]
    blk = wl.make_decode_block_inputs(lens, seed=21, device=dev)
    idx = blk.indexer
    pages = idx.k_index_cache_fp8.shape[0]
    gen = torch.Generator(device=dev).manual_seed(5)
    keys = torch.randn(pages * 64, 128, generator=gen, device=dev)
    slots = torch.randperm(pages * 64, generator=gen, device=dev).to(torch.int32)
    cache_a = torch.zeros_like(idx.k_index_cache_fp8)
    cache_write.write_index_keys(keys, slots, cache_a)
    ordered = torch.empty_like(keys)
    ordered[slots.long()] = keys
    # packed on the host: torch's CUDA division by a Python scalar multiplies by the reciprocal,
    # which is not the IEEE division the layout is defined with
    cache_b = wl.pack_index_pages(ordered.cpu().view(pages, 64, 128)).to(dev)
    assert torch.equal(cache_a, cache_b)
    top_a = indexer.run(idx.q_index_fp8, cache_a, idx.weights, idx.seq_lens, idx.block_table)
    top_b = indexer.run(idx.q_index_fp8, cache_b, idx.weights, idx.seq_lens, idx.block_table)
    assert torch.equal(top_a.sort(dim=1).values, top_b.sort(dim=1).values)

    ckv_rows = blk.ckv_cache.view(-1, 512)[slots.long()]
    kpe_rows = blk.kpe_cache.view(-1, 64)[slots.long()]
    cc, pc = torch.zeros_like(blk.ckv_cache), torch.zeros_like(blk.kpe_cache)
    cache_write.append_kv(ckv_rows, kpe_rows, slots, cc, pc)
    assert torch.equal(cc.view(torch.int16), blk.ckv_cache.view(torch.int16))
    out_a, lse_a = sparse_attention.run(blk.q_nope, blk.q_pe, cc, pc, top_a, blk.sm_scale)
    out_b, lse_b = sparse_attention.run(blk.q_nope, blk.q_pe, blk.ckv_cache, blk.kpe_cache, top_a,
                                        blk.sm_scale)
    assert torch.equal(out_a.view(torch.int16), out_b.view(torch.int16)) and torch.equal(lse_a, lse_b)
    assert workspace.check_status(dev) == 0
