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

__all__ = ["shard_requests", "balance_by_pages", "head_slice", "HeadParallelDecoder"]


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


class HeadParallelDecoder:
    """Decode attention for a batch whose KV heads are sliced across the ranks of ``group``.

    ``attn_fn(q_local, k_pool_local, v_pool_local, block_table, ctx_len, page_size, scale,
    return_lse=True) -> (out, lse)`` defaults to the CUDA operator; tests on CPU ranks inject a
    checker in its place to exercise the slicing and the all-gather.
    """

    def __init__(self, n_q_heads: int, n_kv_heads: int, group: Optional[dist.ProcessGroup] = None,
                 attn_fn: Optional[Callable] = None):
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

    def _local(self, q, k_pool_local, v_pool_local, block_table, ctx_len, page_size, scale, out_view, lse_view,
               new_tokens=None, **kw):
        if self._native and new_tokens is not None:
            from .attention import paged_decode_step
            paged_decode_step(q, new_tokens[0], new_tokens[1], k_pool_local, v_pool_local, block_table, ctx_len,
                              page_size, scale, out=out_view, lse=lse_view, out_dtype=torch.float32, **kw)
        elif self._native:
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
        gathered = torch.empty(self.world * flat.numel(), dtype=torch.float32, device=q.device)
        dist.all_gather_into_tensor(gathered, flat, group=self.group)
        out, lse = self._unpack(gathered.view(self.world, -1), B, Hl, D)
        return out.to(q.dtype), lse.contiguous()

    def capture_local(self, q: torch.Tensor, k_pool_local: torch.Tensor, v_pool_local: torch.Tensor,
                      block_table: torch.Tensor, ctx_len: torch.Tensor, page_size: int = 16,
                      scale: Optional[float] = None, before: Optional[Callable[[], None]] = None,
                      new_tokens: Optional[Tuple[torch.Tensor, torch.Tensor]] = None):
        """Record this rank's share of a step -- the attention kernels, which store their fp32 result
        straight into the block the collective sends -- in a CUDA graph, and return ``step()``.
        ``new_tokens=(k_new, v_new)`` (this rank's KV heads, ``[B, H_kv/world, D]``) makes it the fused decode
        step: the new token of every sequence is appended by the attention launch itself (``ctx_len`` then
        includes it).  ``before`` (optional) is called first inside the recording, for anything else the step
        has to do on this stream.

        At 131072 tokens over 8 GPUs each rank reads 67 MB per step (about 10 microseconds of HBM
        time), so the step is bound by launch latency.  ``step()`` replays the graph and then issues
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

        def local():
            if before is not None:
                before()
            self._local(q, k_pool_local, v_pool_local, block_table, ctx_len, page_size, scale, out_view, lse_view,
                        new_tokens=new_tokens, **extra)

        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            local()                      # one-time set-up of the kernels happens outside the capture
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            local()

        def step(_keep=(side, extra)):           # the capture stream and the scratch live as long as the closure
            graph.replay()
            if self.world > 1:
                dist.all_gather_into_tensor(gathered, flat, group=self.group)
                return self._unpack(gathered.view(self.world, -1), B, Hl, D)
            return out_view, lse_view

        return step
