"""One decode step of the DSA block for callers whose per-step tensors live in HOST memory.

The reference's callers hand CUDA tensors to `kernel(...)`; a serving loop that builds the query,
the weights and the block table on the host pays for the copies itself.  `HostDecodeStep` is that
loop's entry: it owns one pinned input slab and one pinned result slab (named views below), a
device mirror of each and a side stream, and runs

    main stream : H2D [q_index | weights | seq_lens | block_table]  ->  indexer  ->  (wait q)  ->
                  attention  ->  D2H [output | lse]
    side stream : H2D [q_nope | q_pe]  (under the indexer)   ...   D2H indices (under the attention)

so that a step costs two copies on the critical path instead of nine.  The whole sequence is one
call of the C ABI (`dsa_decode_step_host`): the Python side only fills a struct once.  The paged
caches are device-resident state, as for the reference's callers.  The caller fills `inputs.*` in
place (or passes tensors to `run`, which copies them into the slab first) and reads `outputs.*`
after `run` returns; `run` synchronises.
"""
from __future__ import annotations

from dataclasses import dataclass
from types import SimpleNamespace

import torch

import ctypes

from . import _lib, indexer, workspace

ALIGN = 256


@dataclass(frozen=True)
class Field:
    name: str
    shape: tuple
    dtype: torch.dtype
    offset: int
    nbytes: int


def slab_layout(fields):
    """Offsets of (name, shape, dtype) fields packed into one slab, each 256-byte aligned.
    Returns ([Field...], total_bytes)."""
    out, at = [], 0
    for name, shape, dtype in fields:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        out.append(Field(name, tuple(int(s) for s in shape), dtype, at, nbytes))
        at += (nbytes + ALIGN - 1) // ALIGN * ALIGN
    return out, at


def step_layout(batch: int, max_pages: int, heads: int = 16):
    """The three slabs of a step: indexer inputs, attention inputs, results (indices last so that
    output + lse are one contiguous copy)."""
    a, a_bytes = slab_layout([
        ("q_index_fp8", (batch, indexer.HEADS, indexer.DIM), torch.uint8),
        ("weights", (batch, indexer.HEADS), torch.float32),
        ("seq_lens", (batch,), torch.int32),
        ("block_table", (batch, max_pages), torch.int32),
    ])
    b, b_bytes = slab_layout([
        ("q_nope", (batch, heads, 512), torch.bfloat16),
        ("q_pe", (batch, heads, 64), torch.bfloat16),
    ])
    r, r_bytes = slab_layout([
        ("output", (batch, heads, 512), torch.bfloat16),
        ("lse", (batch, heads), torch.float32),
        ("topk_indices", (batch, indexer.TOPK), torch.int32),
    ])
    return (a, a_bytes), (b, b_bytes), (r, r_bytes)


def _views(slab: torch.Tensor, fields, base: int = 0):
    ns = SimpleNamespace()
    for f in fields:
        raw = slab[base + f.offset: base + f.offset + f.nbytes]
        setattr(ns, f.name, raw.view(f.dtype).view(f.shape))
    return ns


class HostDecodeStep:
    def __init__(self, k_index_cache_fp8, ckv_cache, kpe_cache, batch: int, max_pages: int,
                 sm_scale: float, heads: int = 16):
        if not k_index_cache_fp8.is_cuda:
            raise RuntimeError("HostDecodeStep: the paged caches must be CUDA tensors")
        self.device = k_index_cache_fp8.device
        self.k_index_cache_fp8, self.ckv_cache, self.kpe_cache = k_index_cache_fp8, ckv_cache, kpe_cache
        self.batch, self.max_pages, self.sm_scale = batch, max_pages, sm_scale
        (fa, na), (fb, nb), (fr, nr) = step_layout(batch, max_pages, heads)
        self._na, self._nb = na, nb
        self._host_in = torch.empty(na + nb, dtype=torch.uint8).pin_memory()
        self._dev_in = torch.empty(na + nb, dtype=torch.uint8, device=self.device)
        self._host_out = torch.empty(nr, dtype=torch.uint8).pin_memory()
        self._dev_out = torch.empty(nr, dtype=torch.uint8, device=self.device)
        self._split = next(f.offset for f in fr if f.name == "topk_indices")
        self.inputs = _views(self._host_in, fa)
        for k, v in vars(_views(self._host_in, fb, na)).items():
            setattr(self.inputs, k, v)
        self.outputs = _views(self._host_out, fr)
        self._d = _views(self._dev_in, fa)
        for k, v in vars(_views(self._dev_in, fb, na)).items():
            setattr(self._d, k, v)
        self._r = _views(self._dev_out, fr)
        self._side = torch.cuda.Stream(self.device)
        self.h2d_bytes = sum(f.nbytes for f in fa) + sum(f.nbytes for f in fb)
        self.d2h_bytes = sum(f.nbytes for f in fr)
        # workspaces of its own: the shared grow-only ones may move when another call grows them
        lib = _lib.load()
        with torch.cuda.device(self.device):
            iws = lib.dsa_indexer_workspace_bytes(batch, max_pages)
            aws = lib.dsa_sparse_attn_workspace_bytes(batch, heads, indexer.TOPK)
            self._iws = torch.zeros(iws, dtype=torch.uint8, device=self.device)
            self._aws = torch.zeros(aws, dtype=torch.uint8, device=self.device)
            self._events = [torch.cuda.Event() for _ in range(3)]
            for ev in self._events:      # an event gets its handle when it is first recorded
                ev.record(self._side)
            self._side.synchronize()
        d, r = self._d, self._r
        self._args = _lib.HostStepArgs(
            host_in=self._host_in.data_ptr(), dev_in=self._dev_in.data_ptr(),
            in_indexer_bytes=na, in_attention_bytes=nb,
            host_out=self._host_out.data_ptr(), dev_out=self._dev_out.data_ptr(),
            out_attention_bytes=self._split, out_indices_bytes=nr - self._split,
            q_index_fp8=d.q_index_fp8.data_ptr(), weights=d.weights.data_ptr(),
            seq_lens=d.seq_lens.data_ptr(), block_table=d.block_table.data_ptr(),
            block_table_stride=max_pages, q_nope=d.q_nope.data_ptr(), q_pe=d.q_pe.data_ptr(),
            output=r.output.data_ptr(), lse=r.lse.data_ptr(), topk_indices=r.topk_indices.data_ptr(),
            k_index_cache=k_index_cache_fp8.data_ptr(), ckv_cache=ckv_cache.data_ptr(),
            kpe_cache=kpe_cache.data_ptr(), batch=batch, num_pages=k_index_cache_fp8.shape[0],
            max_pages=max_pages, num_slots=ckv_cache.numel() // 512, sm_scale=sm_scale,
            indexer_workspace=self._iws.data_ptr(), indexer_workspace_bytes=iws,
            attention_workspace=self._aws.data_ptr(), attention_workspace_bytes=aws,
            status_dev=workspace.status_word(self.device).data_ptr(),
            stream=0, side_stream=self._side.cuda_stream,
            ev_first_copy=self._events[0].cuda_event, ev_q_ready=self._events[1].cuda_event,
            ev_indices_ready=self._events[2].cuda_event)
        self._args_ref = ctypes.byref(self._args)
        self._lib = lib

    def run(self, q_index_fp8=None, weights=None, seq_lens=None, block_table=None, q_nope=None,
            q_pe=None):
        """Run one step over `inputs.*` (after copying any tensors given here into them) and return
        (topk_indices, output, lse) as views of the pinned result slab."""
        given = dict(q_index_fp8=q_index_fp8, weights=weights, seq_lens=seq_lens,
                     block_table=block_table, q_nope=q_nope, q_pe=q_pe)
        for name, t in given.items():
            if t is not None:
                dst = getattr(self.inputs, name)
                dst.copy_(t.view(torch.uint8) if name == "q_index_fp8" and t.element_size() == 1
                          and t.dtype != torch.uint8 else t)
        self._args.stream = workspace.stream_handle(self.device)
        with workspace.device_guard(self.device):
            rc = self._lib.dsa_decode_step_host(self._args_ref)
        _lib.check(rc, "dsa_decode_step_host")
        return self.outputs.topk_indices, self.outputs.output, self.outputs.lse
