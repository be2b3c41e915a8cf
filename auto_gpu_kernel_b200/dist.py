"""Multi-GPU layouts of the DSA decode block (one process per GPU, torch.distributed).

The reference has no multi-GPU path; its attention definition only notes that 16 heads are one
tensor-parallel rank of a 128-head model (sparse_baseline.py:4-5).  Two layouts follow from the
data dependencies of the two definitions:

* request-sharded (`shard_range`, `decode_block_local`): requests are independent in both stages
  (indexer_baseline.py:62 loops over them), so every rank runs indexer -> attention on its own
  requests and its own cache pages.  No collective at all.
* head-sharded attention (`decode_block_head_sharded`): the indexer stays request-sharded, the
  attention of ALL tokens runs on every rank for that rank's 16 of the 128 heads, with the ckv/kpe
  caches replicated.  Every rank then needs every request's indices: one all-gather of the int32
  [B, 2048] index tensor (1 MiB at B = 128) is the only exchange step of the path
  (`HeadShardedPlan`: NCCL), or the same exchange as pushes into the peers' buffers by a kernel
  of this library (`PeerPushPlan`).

The stage functions are parameters so that the orchestration can be exercised on CPU ranks (gloo)
with stand-ins; by default they are the CUDA operators of this package.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

TOPK = 2048
HEADS_PER_RANK = 16


def shard_range(total: int, rank: int, world: int) -> range:
    """Contiguous, balanced shard of `total` items: the first `total % world` ranks get one more."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world {rank}/{world}")
    base, extra = divmod(total, world)
    lo = rank * base + min(rank, extra)
    return range(lo, lo + base + (1 if rank < extra else 0))


def _default_ops():
    from . import indexer, sparse_attention
    return indexer.kernel, sparse_attention.kernel


def decode_block_local(idx_args, q_nope, q_pe, ckv_cache, kpe_cache, sm_scale, topk_indices, output,
                       lse, indexer_fn=None, attention_fn=None):
    """Request-sharded layout: the rank's own requests, no communication."""
    if indexer_fn is None or attention_fn is None:
        indexer_fn, attention_fn = _default_ops()
    indexer_fn(*idx_args, topk_indices)
    attention_fn(q_nope, q_pe, ckv_cache, kpe_cache, topk_indices, sm_scale, output, lse)
    return output, lse


class HeadShardedPlan:
    """Buffers of the head-sharded layout, allocated once: the rank's own index rows are written by
    the indexer straight into its slot of the gathered tensor's source buffer, and every step's
    all-gather lands in the same pre-allocated [world * most, 2048] tensor -- no allocation, copy
    or concatenation per step.

    counts[r] = requests of rank r.  With equal counts (the usual case: B divisible by the world
    size) `all_rows` is the gathered tensor itself; with ragged counts every shard is padded to
    the largest one with rows of -1 and `all_rows` is a compacted copy made after the gather."""

    def __init__(self, counts, rank, device, group=None, width=TOPK):
        self.counts = [int(c) for c in counts]
        self.rank, self.group, self.world = rank, group, len(self.counts)
        self.most = max(self.counts)
        self.equal = all(c == self.most for c in self.counts)
        self.padded = torch.full((self.most, width), -1, dtype=torch.int32, device=device)
        self.local_rows = self.padded[: self.counts[rank]]
        if self.world == 1:
            self.gathered = self.padded
            self.all_rows = self.local_rows
        else:
            self.gathered = torch.empty(self.world * self.most, width, dtype=torch.int32, device=device)
            self.all_rows = self.gathered if self.equal else torch.empty(sum(self.counts), width,
                                                                        dtype=torch.int32, device=device)

    def gather(self):
        """All-gather of the index rows (the one collective of the path); returns `all_rows`."""
        if self.world == 1:
            return self.all_rows
        dist.all_gather_into_tensor(self.gathered, self.padded, group=self.group)
        if not self.equal:
            at = 0
            for r, c in enumerate(self.counts):
                self.all_rows[at:at + c].copy_(self.gathered[r * self.most: r * self.most + c])
                at += c
        return self.all_rows


class _DeviceBytes:
    """A raw device allocation as an object torch can wrap without copying."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 3, "strides": None}


class _PeerSlabs:
    """One zeroed device allocation per rank that every other rank of the host can address:
    created by the library (`dsa_peer_slab_create`), its CUDA IPC handle exchanged through the
    process group, the peers' allocations opened with this rank's device current (which also
    enables peer access to their GPUs).  `ptrs[r]` = rank r's slab as seen from this GPU."""

    def __init__(self, nbytes: int, device, group):
        import ctypes
        from . import _lib, workspace
        self._lib, self._guard, self.device = _lib, workspace.device_guard, torch.device(device)
        lib = _lib.load()
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        own, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
        with self._guard(self.device):
            rc = lib.dsa_peer_slab_create(nbytes, ctypes.addressof(own), ctypes.addressof(handle))
        error = None if rc == 0 else f"dsa_peer_slab_create returned {rc}"
        self.own, self.nbytes = (own.value if rc == 0 else None), nbytes
        handles = [None] * world
        dist.all_gather_object(handles, handle.raw if rc == 0 else None, group=group)
        self.ptrs, self._opened = [], []
        for r, raw in enumerate(handles):
            if error is not None:
                break
            if raw is None:
                error = f"rank {r} has no buffer"
                break
            if r == rank:
                self.ptrs.append(self.own)
                continue
            buf, got = ctypes.create_string_buffer(raw, 64), ctypes.c_void_p()
            with self._guard(self.device):
                rc = lib.dsa_peer_slab_open(ctypes.addressof(buf), ctypes.addressof(got))
            if rc != 0:
                error = f"dsa_peer_slab_open(rank {r}) returned {rc}"
                break
            self.ptrs.append(got.value)
            self._opened.append(got.value)
        self._group = group
        # every slab is mapped everywhere before anyone writes -- or nobody goes on: the outcome is
        # agreed on by all ranks, so a failure on one of them cannot leave the others waiting
        outcomes = [None] * world
        dist.all_gather_object(outcomes, error, group=group)
        failed = [f"rank {r}: {e}" for r, e in enumerate(outcomes) if e is not None]
        if failed:
            self.tensor = None
            self._release(barrier=False)    # nothing was written through the mappings yet
            raise RuntimeError("peer buffers could not be mapped (" + "; ".join(failed) + ")")
        with self._guard(self.device):
            self.tensor = torch.as_tensor(_DeviceBytes(self.own, nbytes), device=self.device)

    def close(self):
        """Unmap the peers' slabs, then (after a barrier) free the own one.  Collective."""
        self._release(barrier=True)

    def _release(self, barrier: bool):
        if self.own is None and not self._opened:
            if barrier and dist.is_initialized():
                dist.barrier(group=self._group)
            return
        lib = self._lib.load()
        self.tensor = None
        with self._guard(self.device):
            torch.cuda.synchronize(self.device)
            for p in self._opened:
                lib.dsa_peer_slab_close(p)
            self._opened = []
            if barrier and dist.is_initialized():
                dist.barrier(group=self._group)
            if self.own is not None:
                lib.dsa_peer_slab_destroy(self.own)
        self.own = None


class PeerPushPlan:
    """Head-sharded layout without NCCL in the data path: same interface as `HeadShardedPlan`
    (`local_rows`, `gather()`, `all_rows`), but `gather()` is one kernel of this library
    (`dsa_index_rows_exchange`) that stores the rank's rows as (id, epoch) pairs straight into
    every peer's staging buffer over NVLink and takes the peers' rows out of its own as soon as
    their pairs carry the step's epoch (a poll with a time limit).

    Every rank owns one slab -- two staging buffers of B x width pairs, used alternately -- and maps
    its peers' slabs through CUDA IPC handles (exchanged once, through the process group; `close()`
    releases them, collectively).  The index tensor itself is ordinary device memory: the indexer
    writes the rank's rows into `local_rows`, a view of it, and the attention reads `all_rows`, the
    whole of it, so there is no copy on this GPU either.  One process per GPU."""

    def __init__(self, counts, rank, device, group=None, width=TOPK, wait_limit_ns=5_000_000_000):
        import ctypes
        from . import _lib, workspace
        self.counts = [int(c) for c in counts]
        self.rank, self.group, self.world = rank, group, len(self.counts)
        if self.world > 8:
            raise ValueError("PeerPushPlan: at most 8 ranks")
        self.total, self.width = sum(self.counts), width
        self.offset = sum(self.counts[:rank])
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("PeerPushPlan: the exchange kernel needs CUDA devices (use HeadShardedPlan "
                               "for other process groups)")
        self.wait_limit_ns = int(wait_limit_ns)
        self.all_rows = torch.full((self.total, width), -1, dtype=torch.int32, device=self.device)
        self.local_rows = self.all_rows[self.offset: self.offset + self.counts[rank]]
        stage_bytes = self.total * width * 8
        if self.world > 1:
            self._slabs = _PeerSlabs(2 * stage_bytes, self.device, group)
            bases = self._slabs.ptrs
        else:
            self._slabs = None
            self._own = torch.zeros(2 * stage_bytes, dtype=torch.uint8, device=self.device)
            bases = [self._own.data_ptr()]
        self._stage_ptrs = [(ctypes.c_void_p * self.world)(*[b + p * stage_bytes for b in bases]) for p in range(2)]
        self._ctypes = ctypes
        self._lib, self._workspace = _lib, workspace
        self.epoch = 0
        self._sent = 0

    def close(self):
        """Release the shared buffers (collective: every rank calls it)."""
        if self._slabs is not None:
            self._slabs.close()
            self._slabs = None

    def abandon(self):
        """Release this rank's side without meeting the others (for a set-up that another rank could
        not complete: nothing has been exchanged yet)."""
        if self._slabs is not None:
            self._slabs._release(barrier=False)
            self._slabs = None

    def _epoch_word(self, epoch):
        return ((epoch - 1) % 0xFFFFFFFF) + 1     # never 0

    def run_indexer(self, q_index_fp8, k_index_cache_fp8, weights, seq_lens, block_table):
        """The rank's indexer with the sends fused into its selection kernel: writes `local_rows`
        and stores every finished row into the peers' staging buffers of the step that the next
        `gather()` completes (which then only takes)."""
        from . import indexer
        nxt = self.epoch + 1
        send = None
        if self.world > 1 and q_index_fp8.shape[0] > 0 and block_table.shape[1] > 0:
            send = (self._ctypes.addressof(self._stage_ptrs[nxt & 1]), self.world, self.rank, self.offset,
                    self._epoch_word(nxt))
        indexer.kernel(q_index_fp8, k_index_cache_fp8, weights, seq_lens, block_table, self.local_rows,
                       send=send)
        if send is not None:
            self._sent = nxt

    def gather(self):
        self.epoch += 1
        mode = 2 if self._sent == self.epoch else 3
        lib = self._lib.load()
        with self._workspace.device_guard(self.device):
            rc = lib.dsa_index_rows_exchange(
                self.all_rows.data_ptr(), self._ctypes.addressof(self._stage_ptrs[self.epoch & 1]),
                self.world, self.rank, self.counts[self.rank], self.offset, self.total,
                self.all_rows.stride(0), self.width, self._epoch_word(self.epoch), mode,
                self.wait_limit_ns, self._workspace.status_word(self.device).data_ptr(),
                self._workspace.stream_handle(self.device))
        self._lib.check(rc, "dsa_index_rows_exchange")
        return self.all_rows


def gather_indices(local_indices: torch.Tensor, counts, group=None) -> torch.Tensor:
    """All-gather of the per-rank index rows into the full [B, 2048] tensor (rank order), for
    callers without a plan: allocates its result.  `counts[r]` = requests of rank r."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return local_indices
    rank = dist.get_rank(group)
    plan = HeadShardedPlan(counts, rank, local_indices.device, group, local_indices.shape[1])
    plan.local_rows.copy_(local_indices)
    return plan.gather()


def decode_block_head_sharded(idx_args_local, counts, q_nope_heads, q_pe_heads, ckv_cache, kpe_cache,
                              sm_scale, output, lse, local_indices=None, group=None, indexer_fn=None,
                              attention_fn=None, plan=None):
    """Head-sharded layout of the full 128-head block (128 heads = 8 ranks x 16).

    idx_args_local : indexer inputs of this rank's request shard (q, cache, weights, seq_lens,
                     block_table); the cache holds (at least) this shard's pages
    counts         : requests per rank, in rank order (sum = B)
    q_nope_heads   : [B, 16, 512] bf16, this rank's heads of ALL tokens; q_pe_heads likewise
    ckv/kpe caches : replicated, identical page numbering on every rank
    output, lse    : [B, 16, 512] bf16 / [B, 16] fp32 for this rank's heads
    plan           : a HeadShardedPlan kept across steps (no per-step allocation); without one a
                     plan is made for this call (and `local_indices`, if given, receives a copy
                     of the rank's own rows)
    Returns the gathered [B, 2048] index tensor.
    """
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    fused = indexer_fn is None and hasattr(plan, "run_indexer")
    if indexer_fn is None or attention_fn is None:
        default_indexer, default_attention = _default_ops()
        indexer_fn = indexer_fn or default_indexer
        attention_fn = attention_fn or default_attention
    if plan is None:
        plan = HeadShardedPlan(counts, rank, q_nope_heads.device, group)
    if fused:
        plan.run_indexer(*idx_args_local)      # the selection kernel sends the rows itself
    else:
        indexer_fn(*idx_args_local, plan.local_rows)
    all_indices = plan.gather()
    if local_indices is not None:
        local_indices.copy_(plan.local_rows)
    attention_fn(q_nope_heads, q_pe_heads, ckv_cache, kpe_cache, all_indices, sm_scale, output, lse)
    return all_indices


def prefill_block_token_sharded(idx_args, q_nope, q_pe, ckv_cache, kpe_cache, sm_scale, rank, world,
                                indexer_fn=None, attention_fn=None):
    """Chunked prefill of ONE request with the chunk's query tokens sharded over the ranks (query
    tokens are independent in both definitions, the key pages and ckv/kpe caches are replicated,
    so there is no collective).  idx_args = (q [T,64,128], cache, weights [T,64], seq_lens [T],
    block_table [1 or T, pages]) for the whole chunk; every rank runs its contiguous token range
    (`shard_range`) and returns (range, topk_indices, output, lse) for it.  A block_table of one
    row, or of T identical rows, is passed on with row stride 0 so that the shared-pages scorer
    is used."""
    if indexer_fn is None or attention_fn is None:
        indexer_fn, attention_fn = _default_ops()
    q, cache, weights, seq_lens, table = idx_args
    mine = shard_range(q.shape[0], rank, world)
    sel = slice(mine.start, mine.stop)
    n = len(mine)
    shared = table[:1].expand(n, -1)
    topk = torch.empty(n, TOPK, dtype=torch.int32, device=q.device)
    indexer_fn(q[sel].contiguous(), cache, weights[sel].contiguous(), seq_lens[sel].contiguous(), shared, topk)
    out = torch.empty(n, q_nope.shape[1], q_nope.shape[2], dtype=q_nope.dtype, device=q.device)
    lse = torch.empty(n, q_nope.shape[1], dtype=torch.float32, device=q.device)
    attention_fn(q_nope[sel].contiguous(), q_pe[sel].contiguous(), ckv_cache, kpe_cache, topk, sm_scale, out, lse)
    return mine, topk, out, lse
