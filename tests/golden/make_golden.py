"""Generate the golden fixtures in this directory by running the REFERENCE repository's own two
PyTorch definitions on CPU.  Run once, in a container where the reference checkout is mounted:

    python tests/golden/make_golden.py /path/to/reference [--only=cache_write]

It imports (read-only, by file path)
  archive/dsa_topk_indexer_fp8_h64_d128_topk2048_ps64/solution/triton/indexer_baseline.py::kernel
  archive/dsa_sparse_attention_h16_ckv512_kpe64_topk2048_ps64/solution/triton/sparse_baseline.py::kernel
feeds them seeded inputs from auto_gpu_kernel_b200.inputs and stores inputs + outputs as .npz.
The fixtures travel with the repository; the reference checkout does not.
"""
import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

from auto_gpu_kernel_b200 import inputs as wl  # noqa: E402

IDX_REL = "archive/dsa_topk_indexer_fp8_h64_d128_topk2048_ps64/solution/triton/indexer_baseline.py"
ATT_REL = "archive/dsa_sparse_attention_h16_ckv512_kpe64_topk2048_ps64/solution/triton/sparse_baseline.py"


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _u8(t):
    return t.contiguous().view(torch.uint8).numpy()


def indexer_case(ref, name, seq_lens, seed):
    inp = wl.make_indexer_inputs(seq_lens, seed=seed)
    out = torch.empty(len(seq_lens), wl.TOPK, dtype=torch.int32)
    ref.kernel(*inp.args(), out)
    dense = ref.dequant_fp8_kv_cache(inp.k_index_cache_fp8)
    np.savez_compressed(
        HERE / f"{name}.npz",
        q_u8=_u8(inp.q_index_fp8), cache_i8=inp.k_index_cache_fp8.numpy(),
        weights=inp.weights.numpy(), seq_lens=inp.seq_lens.numpy(),
        block_table=inp.block_table.numpy(), topk_indices=out.numpy(),
        # a few dequantised rows pin the page unpacking independently of the top-k
        dequant_page0=dense[0].numpy(), dequant_last=dense[-1].numpy())
    print(name, "pages", inp.k_index_cache_fp8.shape[0], "->", (out >= 0).sum(dim=1).tolist())


def attention_case(ref, name, seq_lens, seed, pad_tail=0, blank_row=None):
    inp = wl.make_attention_inputs(seq_lens, seed=seed, pad_tail=pad_tail)
    if blank_row is not None:
        inp.sparse_indices[blank_row] = -1
    tokens = len(seq_lens)
    out = torch.empty(tokens, wl.ATTN_HEADS, wl.CKV_DIM, dtype=torch.bfloat16)
    lse = torch.empty(tokens, wl.ATTN_HEADS, dtype=torch.float32)
    ref.kernel(*inp.args(), out, lse)
    np.savez_compressed(
        HERE / f"{name}.npz",
        q_nope_u16=inp.q_nope.view(torch.int16).numpy(), q_pe_u16=inp.q_pe.view(torch.int16).numpy(),
        ckv_u16=inp.ckv_cache.view(torch.int16).numpy(), kpe_u16=inp.kpe_cache.view(torch.int16).numpy(),
        sparse_indices=inp.sparse_indices.numpy(), sm_scale=np.float64(inp.sm_scale),
        output_u16=out.view(torch.int16).numpy(), lse=lse.numpy())
    print(name, "valid per token", (inp.sparse_indices >= 0).sum(dim=1).tolist())


def cache_write_case(ref, name, seed):
    """Keys -> packed pages.  The reference has no writer, so the expected bytes come from the
    plain torch formulation of the layout its reader unpacks (absmax / 448 scale, torch's e4m3
    cast), and the reference's own dequant_fp8_kv_cache of those bytes pins the reader's view."""
    gen = torch.Generator().manual_seed(seed)
    pages, n = 5, 203
    keys = torch.randn(n, wl.INDEX_DIM, generator=gen)
    keys[0] = 0.0                                            # all-zero token: scale from the clamp
    keys[1] *= torch.logspace(-8, 2, wl.INDEX_DIM)           # wide range: e4m3 subnormals and zeros
    keys[2] = -keys[2].abs()                                 # maximum is negative
    keys[3] = 448.0 * torch.linspace(-1, 1, wl.INDEX_DIM)    # exact code points and ties
    keys[4, 1:] = keys[4, 0] * 1e-3
    slots = torch.randperm(pages * wl.PAGE_SIZE, generator=gen)[:n].to(torch.int32)
    slots[7] = -1                                            # not cached
    cache = torch.zeros(pages, wl.PAGE_BYTES, dtype=torch.uint8)
    amax = keys.abs().amax(dim=-1).clamp_min(1e-12)
    scale = (amax / wl.FP8_MAX).to(torch.float32)
    data = (keys / scale.unsqueeze(-1)).to(torch.float8_e4m3fn).view(torch.uint8)
    for t in range(n):
        s = int(slots[t])
        if s < 0:
            continue
        pg, pos = divmod(s, wl.PAGE_SIZE)
        cache[pg, pos * wl.INDEX_DIM:(pos + 1) * wl.INDEX_DIM] = data[t]
        cache[pg, wl.PAGE_SIZE * wl.INDEX_DIM + 4 * pos: wl.PAGE_SIZE * wl.INDEX_DIM + 4 * pos + 4] = \
            scale[t:t + 1].view(torch.uint8)
    packed = cache.view(torch.int8).reshape(pages, wl.PAGE_SIZE, 1, wl.INDEX_DIM + 4)
    dense = ref.dequant_fp8_kv_cache(packed)                 # [pages,64,128] fp32
    np.savez_compressed(HERE / f"{name}.npz", keys=keys.numpy(), slots=slots.numpy(),
                        cache_i8=packed.numpy(), dequant=dense.numpy())
    print(name, "tokens", n, "pages", pages)


def main():
    args = [a for a in sys.argv[1:] if not a.startswith("--only=")]
    only = [a.split("=", 1)[1] for a in sys.argv[1:] if a.startswith("--only=")]
    if not args:
        sys.exit(__doc__)
    root = Path(args[0])
    if only == ["cache_write"]:
        idx_ref = _load(root / IDX_REL, "ref_indexer_baseline")
        cache_write_case(idx_ref, "cache_write", seed=5)
        return
    torch.manual_seed(0)
    idx_ref = _load(root / IDX_REL, "ref_indexer_baseline")
    att_ref = _load(root / ATT_REL, "ref_sparse_baseline")
    # The reference's own CPU-runnable case: 4 requests of 1024..4096 tokens.
    indexer_case(idx_ref, "indexer_cfg0", [1024, 2048, 3000, 4096], seed=0)
    # Ragged/edge lengths: empty request, single token, page boundary +-1, just over top-k.
    indexer_case(idx_ref, "indexer_edges", [0, 1, 63, 64, 65, 2047, 2049, 2500], seed=1)
    # Attention: three tokens over few pages, last token shorter than top-k (tail -1 padding).
    attention_case(att_ref, "attention_small", [700, 640, 130], seed=2)
    # Attention with forced tail padding and one fully masked row (lse=-inf, NaN output in the
    # reference; recorded as produced).
    attention_case(att_ref, "attention_padded", [300, 256, 64], seed=3, pad_tail=1900, blank_row=2)
    # Cache writer: keys -> packed pages, read back by the reference's dequantiser.
    cache_write_case(idx_ref, "cache_write", seed=5)


if __name__ == "__main__":
    main()
