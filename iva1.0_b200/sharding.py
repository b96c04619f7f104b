"""Multi-GPU forms of the decode path: one process per GPU.

* Request sharding -- sequences (with their page pools and block tables) are partitioned across
  ranks at admission; every rank runs append / gather / attention on its own pool and NOTHING is
  exchanged on the hot path.  ``shard_requests`` and ``balance_by_pages`` are the partitioners.
* Head-parallel decode of one very long sequence -- KV heads (and the query heads attached to
  them) are sliced across ranks; the pool layout ``[1,H_kv,S,D]`` makes each rank's slab
  self-contained and the block table is replicated.  After the local attention one all-gather
  (NCCL over NVLink on GPUs) reassembles ``out [B,H_q,D]`` and ``lse [B,H_q]``.  No K/V ever
  crosses a link.

The reference has no parallel decode path (its distributed wrappers,
src/utils/distributed.py:106-150, have no caller); its backend choice -- NCCL through
``torch.distributed`` (src/utils/distributed.py:29-34) -- is kept.
"""

from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

__all__ = ["shard_requests", "balance_by_pages", "head_slice", "HeadParallelDecoder", "PeerExchange"]


def shard_requests(n_seq: int, world: int, rank: int) -> range:
    """Contiguous, balanced share of ``n_seq`` sequences for ``rank`` (the first ``n_seq % world``
    ranks get one more)."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    per, rem = divmod(n_seq, world)
    lo = rank * per + min(rank, rem)
    return range(lo, lo + per + (1 if rank < rem else 0))


def balance_by_pages(ctx_lens: Sequence[int], world: int, page_size: int = 16) -> List[List[int]]:
    """Partition sequences so that every rank reads about the same number of pages per step
    (longest-processing-time greedy).  Returns the sequence ids of each rank."""
    order = sorted(range(len(ctx_lens)), key=lambda s: -int(ctx_lens[s]))
    load = [0] * world
    parts: List[List[int]] = [[] for _ in range(world)]
    for s in order:
        r = min(range(world), key=lambda i: (load[i], i))
        parts[r].append(s)
        load[r] += (int(ctx_lens[s]) + page_size - 1) // page_size
    for p in parts:
        p.sort()
    return parts


def head_slice(n_q_heads: int, n_kv_heads: int, world: int, rank: int) -> Tuple[slice, slice]:
    """(query-head slice, kv-head slice) owned by ``rank``; query heads follow their KV head."""
    if n_kv_heads % world:
        raise ValueError(f"{n_kv_heads} KV heads do not split over {world} ranks")
    group = n_q_heads // n_kv_heads
    per = n_kv_heads // world
    return slice(rank * per * group, (rank + 1) * per * group), slice(rank * per, (rank + 1) * per)


class PeerExchange:
    """All-gather of one small fp32 block per rank through peer-mapped memory: this library's own kernel
    (``ivab_peer_allgather``: plain NVLink stores of {payload, step tag} words, a bounded wait per word)
    instead of an NCCL collective.  ``torch.distributed``'s symmetric memory allocates the buffer and maps it
    into every peer -- plumbing; the data path is the kernel.  All ranks must construct it together and make
    the same sequence of ``gather`` calls.

    ``gather(block)`` enqueues the exchange on the current stream and returns ``[world, block.numel()]``
    (a view of this rank's buffer, valid until the call after next); it can be recorded in a CUDA graph.
    """

    SLOTS = 2

    def __init__(self, numel: int, group: Optional[dist.ProcessGroup] = None, device=None, wait_limit_ns: int = 2_000_000_000):
        import ctypes
        import os

        import torch.distributed._symmetric_memory as symm

        from . import _lib

        # only plain peer loads and stores are used here: no multicast binding is needed, and none is wanted
        # (a rank that dies while its memory is bound to a multicast object disturbs its peers' GPUs)
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.numel = int(numel)
        self.block_bytes = (self.numel * 4 + 15) // 16 * 16
        self.flags_off = self.SLOTS * self.world * self.block_bytes
        # result rows, then the staging area the peers write: every payload word as a {payload, step tag} pair
        total_words = (self.flags_off + self.SLOTS * self.world * 2 * self.block_bytes) // 4
        self.buf = symm.empty(total_words, dtype=torch.float32, device=self.device)
        self.buf.zero_()
        torch.cuda.synchronize(self.device)
        self.handle = symm.rendezvous(self.buf, self.group)
        dist.barrier(self.group)                       # every rank's staging area is zero before anyone sends
        torch.cuda.synchronize(self.device)
        # the address of every rank's copy of THIS tensor in this process's address space (the tensor may sit at
        # an offset inside a larger symmetric allocation, so the allocation's base pointers are not enough)
        self._remote = [self.handle.get_remote_tensor(r, tuple(self.buf.shape), self.buf.dtype) for r in range(self.world)]
        ptrs = [int(t.data_ptr()) for t in self._remote]
        if ptrs[self.rank] != self.buf.data_ptr():
            raise RuntimeError("symmetric memory: this rank's own mapping does not coincide with the local tensor")
        self._peer_array = (ctypes.c_void_p * self.world)(*ptrs)
        self._epoch = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._lib, self._check = _lib.load_library(), _lib.check
        self._stream_ptr = _lib.stream_ptr
        self.wait_limit_ns = int(wait_limit_ns)
        self._rows = [self.buf.view(torch.uint8)[s * self.world * self.block_bytes:(s + 1) * self.world * self.block_bytes]
                      .view(self.world, self.block_bytes).view(torch.float32)[:, :self.numel] for s in range(self.SLOTS)]
        self._steps = 0

    def exchange_args(self, block: torch.Tensor) -> tuple:
        """The exchange arguments of ``ivab_peer_allgather`` / ``ivab_paged_decode_step_allgather`` for ``block``
        (everything between the block pointer and the stream)."""
        if block.dtype != torch.float32 or block.numel() != self.numel or not block.is_contiguous():
            raise ValueError("block must be a contiguous fp32 tensor of the size given at construction")
        return (block.data_ptr(), self.block_bytes, self._peer_array, self.world, self.rank, self.SLOTS, self.flags_off,
                self._epoch.data_ptr(), self.status.data_ptr(), self.wait_limit_ns)

    def enqueue(self, block: torch.Tensor) -> None:
        """Enqueue one exchange of ``block`` (fp32, ``numel`` elements, 16-byte aligned) on the current stream."""
        with torch.cuda.device(self.device):
            self._check(self._lib.ivab_peer_allgather(*self.exchange_args(block), self._stream_ptr(self.device)))

    def rows(self, step: int) -> torch.Tensor:
        """``[world, numel]`` view of the slot that the ``step``-th exchange (counted from 0) fills."""
        return self._rows[step % self.SLOTS]

    def gather(self, block: torch.Tensor) -> torch.Tensor:
        self.enqueue(block)
        out = self.rows(self._steps)
        self._steps += 1
        return out


class HeadParallelDecoder:
    """Decode attention for a batch whose KV heads are sliced across the ranks of ``group``.

    ``attn_fn(q_local, k_pool_local, v_pool_local, block_table, ctx_len, page_size, scale,
    return_lse=True) -> (out, lse)`` defaults to the CUDA operator; tests on CPU ranks inject a
    checker in its place to exercise the slicing and the all-gather.
    """

    def __init__(self, n_q_heads: int, n_kv_heads: int, group: Optional[dist.ProcessGroup] = None,
                 attn_fn: Optional[Callable] = None, exchange: str = "nccl"):
        """``exchange``: ``"nccl"`` reassembles the outputs with one ``all_gather_into_tensor``; ``"p2p"`` with
        this library's own kernel over peer-mapped memory (``PeerExchange``; CUDA ranks of one node)."""
        if exchange not in ("nccl", "p2p"):
            raise ValueError("exchange must be 'nccl' or 'p2p'")
        self.exchange = exchange
        self._peer: Optional[PeerExchange] = None
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.n_q_heads, self.n_kv_heads = n_q_heads, n_kv_heads
        self.q_slice, self.kv_slice = head_slice(n_q_heads, n_kv_heads, self.world, self.rank)
        self._native = attn_fn is None
        if attn_fn is None:
            from .attention import paged_decode_attention as attn_fn
        self.attn_fn = attn_fn

    def local_pools(self, k_pool: torch.Tensor, v_pool: torch.Tensor):
        """This rank's slab of full ``[1,H_kv,S,D]`` pools (a view, no copy)."""
        return k_pool[:, self.kv_slice], v_pool[:, self.kv_slice]

    # One collective carries both results.  Every rank contributes one flat fp32 block: its output rows
    # ``[B, H_q/world, D]`` followed by its logsumexp ``[B, H_q/world]``.  Both parts are contiguous views of
    # the block, so the attention kernels store straight into it (fp32 output) -- no packing pass.

    def _block(self, B: int, Hl: int, D: int, device):
        flat = torch.empty(B * Hl * (D + 1), dtype=torch.float32, device=device)
        return flat, flat[:B * Hl * D].view(B, Hl, D), flat[B * Hl * D:].view(B, Hl)

    def _peer_exchange(self, numel: int, device) -> PeerExchange:
        if self._peer is None or self._peer.numel != numel:
            self._peer = PeerExchange(numel, self.group, device)     # collective: every rank gets here together
        return self._peer

    def _local(self, q, k_pool_local, v_pool_local, block_table, ctx_len, page_size, scale, out_view, lse_view,
               new_tokens=None, **kw):
        if self._native and new_tokens is not None:
            from .attention import paged_decode_step
            paged_decode_step(q, new_tokens[0], new_tokens[1], k_pool_local, v_pool_local, block_table, ctx_len,
                              page_size, scale, out=out_view, lse=lse_view, out_dtype=torch.float32, **kw)
        elif self._native:
            # (``exchange`` in kw: the library's own attention entry point takes it; the step then ends with the
            #  all-gather, run by the merge kernel's last CTA)
            self.attn_fn(q, k_pool_local, v_pool_local, block_table, ctx_len, page_size, scale, out=out_view,
                         lse=lse_view, out_dtype=torch.float32, **kw)
        else:
            o, l = self.attn_fn(q, k_pool_local, v_pool_local, block_table, ctx_len, page_size, scale, return_lse=True)
            out_view.copy_(o)
            lse_view.copy_(l)

    def _unpack(self, gathered: torch.Tensor, B: int, Hl: int, D: int):
        """``gathered [world, B*Hl*(D+1)]`` -> fp32 ``out [B,H_q,D]`` and ``lse [B,H_q]`` (views when ``B == 1``)."""
        w = self.world
        out = gathered[:, :B * Hl * D].view(w, B, Hl, D).permute(1, 0, 2, 3).reshape(B, w * Hl, D)
        lse = gathered[:, B * Hl * D:].view(w, B, Hl).permute(1, 0, 2).reshape(B, w * Hl)
        return out, lse

    def decode(self, q: torch.Tensor, k_pool_local: torch.Tensor, v_pool_local: torch.Tensor,
               block_table: torch.Tensor, ctx_len: torch.Tensor, page_size: int = 16,
               scale: Optional[float] = None):
        """``q`` is the full ``[B,H_q,D]`` query (replicated) or already this rank's slice.  Returns the
        full ``out [B,H_q,D]`` (in q's dtype) and ``lse [B,H_q]`` on every rank."""
        B = q.shape[0]
        if q.shape[1] == self.n_q_heads and self.world > 1:
            q = q[:, self.q_slice]
        q = q.contiguous()
        Hl, D = q.shape[1], q.shape[2]
        flat, out_view, lse_view = self._block(B, Hl, D, q.device)
        self._local(q, k_pool_local, v_pool_local, block_table, ctx_len, page_size, scale, out_view, lse_view)
        if self.world == 1:
            return out_view.to(q.dtype), lse_view
        if self.exchange == "p2p":
            rows = self._peer_exchange(flat.numel(), q.device).gather(flat)
            out, lse = self._unpack(rows, B, Hl, D)
            return out.to(q.dtype), lse.contiguous()
        gathered = torch.empty(self.world * flat.numel(), dtype=torch.float32, device=q.device)
        dist.all_gather_into_tensor(gathered, flat, group=self.group)
        out, lse = self._unpack(gathered.view(self.world, -1), B, Hl, D)
        return out.to(q.dtype), lse.contiguous()

    def capture_local(self, q: torch.Tensor, k_pool_local: torch.Tensor, v_pool_local: torch.Tensor,
                      block_table: torch.Tensor, ctx_len: torch.Tensor, page_size: int = 16,
                      scale: Optional[float] = None, before: Optional[Callable[[], None]] = None,
                      new_tokens: Optional[Tuple[torch.Tensor, torch.Tensor]] = None, graph: bool = True):
        """Record this rank's share of a step -- the attention kernels, which store their fp32 result
        straight into the block the collective sends -- in a CUDA graph, and return ``step()``.
        ``new_tokens=(k_new, v_new)`` (this rank's KV heads, ``[B, H_kv/world, D]``) makes it the fused decode
        step: the new token of every sequence is appended by the attention launch itself (``ctx_len`` then
        includes it).  ``before`` (optional) is called first inside the recording, for anything else the step
        has to do on this stream.

        ``graph=False`` prepares the same step without recording it: ``step()`` then launches the kernels eagerly
        on the current stream (with ``exchange="p2p"`` that is one library call per step).  Programmatic dependent
        launches then overlap the step's start with whatever runs before it in the stream, which a graph launch
        does not; the price is the host time of the call.

        At 131072 tokens over 8 GPUs each rank reads 67 MB per step (about 10 microseconds of HBM
        time), so the step is bound by launch latency.  The recording reads the query from ``step.q`` (this
        rank's heads, copied from ``q`` here; overwrite it in place between steps), the block table, the
        lengths and the pools in place.  ``step()`` replays the graph and then issues
        ONE eager ``all_gather_into_tensor``; it returns fp32 ``(out [B,H_q,D], lse [B,H_q])``
        (views of the gathered buffer, no further kernels, when ``B == 1``).  The collective is deliberately
        kept outside the capture: recording an NCCL collective of ``torch.distributed`` inside a
        CUDA-graph capture hung on the CUDA 12.9 / NCCL 2.28 stack this was developed on.
        """
        dev = q.device
        B = q.shape[0]
        if q.shape[1] == self.n_q_heads and self.world > 1:
            q = q[:, self.q_slice]
        q = q.contiguous()
        Hl, D = q.shape[1], q.shape[2]
        flat, out_view, lse_view = self._block(B, Hl, D, dev)
        gathered = torch.empty(self.world * flat.numel(), dtype=torch.float32, device=dev)
        # The graph records the scratch pointer: it must be a buffer this object owns, not the shared
        # per-stream one, which a later call on the same stream may replace.
        extra = {}
        if self._native:
            from .attention import decode_workspace_bytes
            n_kv_local = k_pool_local.shape[1]      # both pool layouts keep the KV heads on axis 1
            extra["workspace"] = torch.empty(decode_workspace_bytes(B, Hl, n_kv_local, D), dtype=torch.uint8, device=dev)

        peer = self._peer_exchange(flat.numel(), dev) if (self.exchange == "p2p" and self.world > 1) else None

        fused_exchange = peer is not None and self._native
        if fused_exchange:
            extra["exchange"] = (peer, flat)   # the merge kernel's last CTA sends the block and collects the peers'

        def local():
            if before is not None:
                before()
            self._local(q, k_pool_local, v_pool_local, block_table, ctx_len, page_size, scale, out_view, lse_view,
                        new_tokens=new_tokens, **extra)
            if peer is not None and not fused_exchange:
                peer.enqueue(flat)           # the exchange is part of the recording: a step is one graph replay

        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            local()                      # one-time set-up of the kernels happens outside the capture
        side.synchronize()
        recorded = None
        if graph:
            recorded = torch.cuda.CUDAGraph()
            with torch.cuda.graph(recorded, stream=side):
                local()

        if peer is not None:
            # every rank ran the eager pass and the capture does not execute anything: one exchange so far
            peer._steps += 1
            dist.barrier(self.group)

        # Everything the recording points at must outlive it: the local query buffer made above is owned by
        # nobody else, so the returned function holds it (with the capture stream, the scratch and the block).
        def step(_keep=(side, extra, q, flat, local)):
            if recorded is not None:
                recorded.replay()
            else:
                local()
            if peer is not None:
                rows = peer.rows(peer._steps)
                peer._steps += 1
                return self._unpack(rows, B, Hl, D)
            if self.world > 1:
                dist.all_gather_into_tensor(gathered, flat, group=self.group)
                return self._unpack(gathered.view(self.world, -1), B, Hl, D)
            return out_view, lse_view

        # The graph reads this rank's query heads from ``step.q`` ([B, H_q/world, D]); a decode loop writes the
        # next step's query there (``step.q.copy_(q_new[:, decoder.q_slice])``) before it calls ``step()``.
        step.q = q
        return step
