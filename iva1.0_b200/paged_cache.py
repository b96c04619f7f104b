"""A paged KV cache that duck-types the reference's dense ``KVCache``.

The reference cache (src/core/rope_kv.py:71-137) is two dense ``[B,H,S,D]`` tensors that are
re-concatenated on every decode step (src/core/attention.py:61-63) and re-allocated on every
``resize``.  ``PagedKVCache`` keeps the same constructor keywords, attributes and methods, but
stores K and V in a pool of fixed-size pages addressed through a per-sequence block table, so
appending a token writes one row and nothing is ever copied.

Host side (Python): the free list, the block table and the per-sequence lengths -- the same
bookkeeping a serving engine keeps on the CPU.  Device side: the two pools, an int32 copy of the
block table and of the lengths, and the kernels of ``libivab.so`` for append / gather / decode
attention.
"""

from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from .kv_ops import kv_ops, paged_append, paged_gather

__all__ = ["PagedKVCache", "PoolExhausted"]


class PoolExhausted(RuntimeError):
    """No free page left in the pool."""


class PagedKVCache:
    """Page pools + block table for ``batch_size`` sequences of one or more attention layers.

    With ``n_layers > 1`` there is still ONE free list, ONE block table and ONE length vector --
    every layer stores a token in the same slot of its own pool -- so the host bookkeeping and the
    uploads of a decode step happen once, not once per layer.  ``layer(i)`` gives layer ``i``'s view
    (its pools, the shared tables), which is what ``AttentionB200`` takes as ``kv_cache``.  (The
    reference threads one dense cache object through all layers and reassigns it per block,
    src/core/transformer.py:229-238, so layer ``i+1`` sees layer ``i``'s keys; it also rebuilds the
    cache every step, transformer.py:273-290.  This is the corrected form.)

    Constructor keywords follow ``KVCache(batch_size, n_heads, head_dim, seq_len, device, dtype)``
    (rope_kv.py:73-81; default dtype fp16 as at rope_kv.py:80).  ``seq_len`` is the number of tokens
    considered already present (their K/V are zero, as in the reference, which zero-fills).
    Extra keywords: ``page_size`` (16), ``num_pages`` (pool capacity; default enough for
    ``max_seq_len`` tokens per sequence), ``shuffle_seed`` (hand out pages in a seeded random order
    instead of ascending, to exercise non-contiguous block tables).
    """

    def __init__(self, batch_size: int, n_heads: int, head_dim: int, seq_len: int = 0,
                 device="cuda", dtype: torch.dtype = torch.float16, *, page_size: int = 16,
                 num_pages: Optional[int] = None, max_seq_len: int = 4096,
                 shuffle_seed: Optional[int] = None, n_layers: int = 1,
                 k_scale: float = 1.0, v_scale: float = 1.0):
        self.batch_size = batch_size
        self.n_heads = n_heads
        self.head_dim = head_dim
        self.device = torch.device(device)
        self.dtype = dtype
        self.page_size = page_size
        max_seq_len = max(max_seq_len, seq_len, 1)
        self.max_pages_per_seq = (max_seq_len + page_size - 1) // page_size
        if num_pages is None:
            num_pages = batch_size * self.max_pages_per_seq
        self.num_pages = num_pages
        S = num_pages * page_size
        self.n_layers = n_layers
        self.k_scale, self.v_scale = k_scale, v_scale          # used by 8-bit (e4m3) pools only
        store = torch.uint8 if dtype == torch.float8_e4m3fn else dtype

        def new_pool():
            return torch.zeros(1, n_heads, S, head_dim, device=self.device, dtype=store).view(dtype)

        self._k_pools = [new_pool() for _ in range(n_layers)]
        self._v_pools = [new_pool() for _ in range(n_layers)]
        self.k_pool, self.v_pool = self._k_pools[0], self._v_pools[0]   # layer 0 (the only one by default)
        self._step = None                                      # an append that not every layer has made yet
        if shuffle_seed is None:
            order = list(range(num_pages))
        else:
            order = torch.randperm(num_pages, generator=torch.Generator().manual_seed(shuffle_seed)).tolist()
        self._free: List[int] = order[::-1]          # pop() hands out order[0] first
        self._lens: List[int] = [0] * batch_size
        self._tables: List[List[int]] = [[] for _ in range(batch_size)]
        self._bt_host = torch.full((batch_size, self.max_pages_per_seq), -1, dtype=torch.int32)
        self._len_host = torch.zeros(batch_size, dtype=torch.int32)
        self.block_table_dev = torch.full((batch_size, self.max_pages_per_seq), -1, dtype=torch.int32,
                                          device=self.device)
        self.ctx_len_dev = torch.zeros(batch_size, dtype=torch.int32, device=self.device)
        self._bt_dirty = False
        # Uploads of the host tables go through a small ring of pinned blocks that are allocated once:
        # an asynchronous copy reads host memory when it EXECUTES, so the block it reads must not be
        # rewritten before then; every block carries an event recorded behind its last copy.
        self._ring: List[dict] = []
        self._ring_pos = 0
        if seq_len:
            self._reserve([seq_len] * batch_size)
            self._sync_device()

    is_paged = True

    def layer(self, i: int) -> "_LayerView":
        """Layer ``i``'s view of the cache: its own pools, the shared block table and lengths."""
        if not 0 <= i < self.n_layers:
            raise IndexError(f"layer {i} of {self.n_layers}")
        return _LayerView(self, i)

    # ---- bookkeeping ------------------------------------------------------------------------

    @property
    def seq_len(self) -> int:
        """Longest sequence length (the reference cache has one length for the whole batch)."""
        return max(self._lens) if self._lens else 0

    @property
    def lengths(self) -> List[int]:
        return list(self._lens)

    @property
    def free_pages(self) -> int:
        return len(self._free)

    def _reserve(self, new_lens: Sequence[int]) -> None:
        """Grow block tables so that sequence ``s`` can hold ``new_lens[s]`` tokens."""
        ps, tables = self.page_size, self._tables
        needs = [(L + ps - 1) // ps for L in new_lens]
        grow = [(s, n) for s, n in enumerate(needs) if n > len(tables[s])]
        if grow:                                   # (most decode steps stay inside their last page)
            for s, n in grow:
                if n > self.max_pages_per_seq:
                    raise PoolExhausted(f"sequence {s} needs {n} pages, block table holds {self.max_pages_per_seq}")
            need_total = sum(n - len(tables[s]) for s, n in grow)
            if need_total > len(self._free):
                raise PoolExhausted(f"need {need_total} pages, {len(self._free)} free")
            for s, n in grow:
                tab = tables[s]
                while len(tab) < n:
                    page = self._free.pop()
                    self._bt_host[s, len(tab)] = page
                    tab.append(page)
            self._bt_dirty = True
        self._lens = [int(L) for L in new_lens]
        self._len_host.copy_(torch.tensor(self._lens, dtype=torch.int32))

    _RING = 4

    def _stage_block(self, n_slots: int) -> dict:
        """The next pinned block of the upload ring, free to be rewritten (its previous copies have run)
        and large enough for ``n_slots`` slot ids."""
        if not self._ring:
            self._ring = [None] * self._RING
        i = self._ring_pos
        self._ring_pos = (i + 1) % self._RING
        blk = self._ring[i]
        cuda = self.device.type == "cuda"
        if blk is None or blk["slots"].numel() < n_slots:
            def pinned(*shape, dtype):
                t = torch.empty(*shape, dtype=dtype)
                return t.pin_memory() if cuda else t
            blk = {"bt": pinned(self.batch_size, self.max_pages_per_seq, dtype=torch.int32),
                   "len": pinned(self.batch_size, dtype=torch.int32),
                   "slots": pinned(max(n_slots, self.batch_size), dtype=torch.int64),
                   "event": torch.cuda.Event() if cuda else None, "used": False}
            self._ring[i] = blk
        elif blk["used"] and blk["event"] is not None:
            blk["event"].synchronize()          # normally long complete: the ring is several steps deep
        return blk

    def _sync_device(self, slots: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Upload the lengths, the block table if it changed, and optionally a slot mapping (int64 host
        tensor); returns the slot mapping on the device.  One pinned staging block per call."""
        n = 0 if slots is None else slots.numel()
        blk = self._stage_block(n)
        slot_dev = None
        if self._bt_dirty:
            blk["bt"].copy_(self._bt_host)
            self.block_table_dev.copy_(blk["bt"], non_blocking=True)
            self._bt_dirty = False
        blk["len"].copy_(self._len_host)
        self.ctx_len_dev.copy_(blk["len"], non_blocking=True)
        if slots is not None:
            blk["slots"][:n].copy_(slots)
            slot_dev = blk["slots"][:n].to(self.device, non_blocking=True)
        if blk["event"] is not None:
            blk["event"].record(torch.cuda.current_stream(self.device))
            blk["used"] = True
        return slot_dev

    def slots(self, seq: int, start: int, stop: int) -> List[int]:
        ps, tab = self.page_size, self._tables[seq]
        return [tab[p // ps] * ps + p % ps for p in range(start, stop)]

    def _slots_all(self, start, count: int) -> torch.Tensor:
        """Slot ids of positions ``start[s] .. start[s]+count-1`` of every sequence, flattened sequence-major
        (int64 host tensor); ``start`` is an int or one int per sequence.  Tensor arithmetic on the host
        block table: no per-token Python loop."""
        ps = self.page_size
        st = torch.as_tensor(start, dtype=torch.int64).reshape(-1, 1).expand(self.batch_size, 1)
        pos = st + torch.arange(count, dtype=torch.int64).view(1, count)
        pages = torch.gather(self._bt_host, 1, (pos // ps).clamp_(max=self.max_pages_per_seq - 1)).to(torch.int64)
        return (pages * ps + pos % ps).reshape(-1)

    # ---- the hot path -----------------------------------------------------------------------

    def append(self, k_new: torch.Tensor, v_new: torch.Tensor, write: bool = True) -> List[int]:
        """Append ``S`` tokens to every sequence (layer 0; use ``layer(i).append`` for the others).
        ``k_new`` / ``v_new`` are ``[B,S,H,D]`` (projection output order) or ``[B,H,D]`` for one token.
        ``write=False`` does the bookkeeping only (pages, lengths, table upload) and leaves the rows to the
        caller, who hands them to ``paged_decode_step``.  Returns the lengths before the append."""
        return self._append_layer(0, k_new, v_new, write)

    def _append_layer(self, layer: int, k_new: torch.Tensor, v_new: torch.Tensor, write: bool = True) -> List[int]:
        """One layer's share of a step.  The first layer to arrive reserves pages, computes the slot
        mapping and uploads it with the new lengths; the others reuse it.  The step is complete when
        every layer has appended."""
        if k_new.dim() == 3:
            k_new, v_new = k_new.unsqueeze(1), v_new.unsqueeze(1)
        B, S, H, D = k_new.shape
        if B != self.batch_size or H != self.n_heads or D != self.head_dim:
            raise ValueError(f"expected [{self.batch_size},S,{self.n_heads},{self.head_dim}], got {list(k_new.shape)}")
        if self._step is None:
            prior = list(self._lens)
            self._reserve([L + S for L in prior])
            # the slot mapping is only needed by a layer that writes through the copy kernel; a step whose
            # layers all use the fused decode step (write=False) never computes or uploads it
            slot_dev = self._sync_device(self._slots_all(prior, S) if write else None)
            self._step = {"prior": prior, "slots": slot_dev, "S": S, "done": set()}
        st = self._step
        if S != st["S"] or layer in st["done"]:
            raise RuntimeError(f"layer {layer} appended twice, or with a different token count, within one step")
        if write:
            if st["slots"] is None:
                st["slots"] = self._slots_all(st["prior"], S).to(self.device)
            paged_append(self._k_pools[layer], self._v_pools[layer], st["slots"], k_new.reshape(B * S, H, D),
                         v_new.reshape(B * S, H, D), self.page_size, k_scale=self.k_scale, v_scale=self.v_scale)
        st["done"].add(layer)
        if len(st["done"]) == self.n_layers:
            self._step = None
        return st["prior"]

    def gather(self, layout: str = "head_major"):
        """Contiguous K and V of every sequence (lists of ``[1,H,L_s,D]`` for ``head_major``, packed
        ``[sum L,H,D]`` for ``token_major``)."""
        k = paged_gather(self.k_pool, self.block_table_dev, self.ctx_len_dev, self.page_size, layout=layout)
        v = paged_gather(self.v_pool, self.block_table_dev, self.ctx_len_dev, self.page_size, layout=layout)
        return k, v

    # ---- KVCache duck type (rope_kv.py:83-137) ----------------------------------------------------

    def _dense(self, pool: torch.Tensor) -> torch.Tensor:
        L = self.seq_len
        B, H, D = self.batch_size, self.n_heads, self.head_dim
        if L and min(self._lens) == L:
            # every sequence has the same length (the reference cache knows no other case): sequence s of the
            # head-major gather is [H,L,D] at offset s*L*H*D, i.e. the kernel writes the dense tensor itself
            out = torch.empty(B, H, L, D, device=self.device, dtype=self.dtype)
            offs = torch.arange(B + 1, dtype=torch.int64, device=self.device) * L
            paged_gather(pool, self.block_table_dev, self.ctx_len_dev, self.page_size, layout="head_major",
                         out_offsets=offs, total_tokens=B * L, out=out)
            return out
        seqs = paged_gather(pool, self.block_table_dev, self.ctx_len_dev, self.page_size, layout="head_major")
        out = torch.zeros(B, H, L, D, device=self.device, dtype=self.dtype)
        for s, t in enumerate(seqs):
            out[s, :, :t.shape[2]] = t[0]
        return out

    @property
    def k(self) -> torch.Tensor:
        """Dense ``[B,H,seq_len,D]`` view of the keys, gathered on demand (shorter sequences are
        zero-padded at the end)."""
        return self._dense(self.k_pool)

    @property
    def v(self) -> torch.Tensor:
        return self._dense(self.v_pool)

    def update(self, new_k: torch.Tensor, new_v: torch.Tensor, start_pos: int) -> None:
        """Write ``[B,H,S,D]`` tokens at positions ``start_pos..start_pos+S-1`` of every sequence
        (rope_kv.py:98-110), growing the block tables as needed."""
        B, H, S, D = new_k.shape
        end = start_pos + S
        self._reserve([max(L, end) for L in self._lens])
        slot_dev = self._sync_device(self._slots_all(start_pos, S))
        paged_append(self.k_pool, self.v_pool, slot_dev,
                     new_k.permute(0, 2, 1, 3).reshape(B * S, H, D).contiguous(),
                     new_v.permute(0, 2, 1, 3).reshape(B * S, H, D).contiguous(), self.page_size)

    def resize(self, new_seq_len: int) -> None:
        """Make room for ``new_seq_len`` tokens per sequence (rope_kv.py:112-130).  Pages are taken
        from the free list; nothing is copied.  New positions read as zero only if their pages were
        never used, so callers should write them before reading."""
        self._reserve([max(L, new_seq_len) for L in self._lens])
        self._sync_device()

    def clear(self) -> None:
        """Zero the pools (rope_kv.py:132-134); lengths and block tables are kept, as the reference
        keeps ``seq_len``."""
        for pool in self._k_pools + self._v_pools:
            pool.view(torch.uint8).zero_() if pool.dtype == torch.float8_e4m3fn else pool.zero_()

    def get_slice(self, start: int, end: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """Dense ``[B,H,end-start,D]`` K and V (rope_kv.py:136-137)."""
        return self.k[:, :, start:end], self.v[:, :, start:end]

    def reset(self, seq: Optional[int] = None) -> None:
        """Return the pages of one sequence (or of all) to the free list."""
        for s in (range(self.batch_size) if seq is None else [seq]):
            # entries that evict_before() already handed back are -1: they are not pages
            self._free.extend(p for p in reversed(self._tables[s]) if p >= 0)
            self._tables[s] = []
            self._lens[s] = 0
            self._len_host[s] = 0
            self._bt_host[s].fill_(-1)
        self._bt_dirty = True
        self._sync_device()


    def evict_before(self, begin: Sequence[int], keep_sink_tokens: int = 0) -> int:
        """Return to the pool every page that lies wholly before position ``begin[s]`` of sequence
        ``s`` (the keys a sliding window no longer needs), except the pages that hold the first
        ``keep_sink_tokens`` keys.  The block-table entries of those pages
        become ``-1``; decode attention called with ``ctx_begin >= begin`` never reads them.  Dense
        views (``.k``, ``gather``) of an evicted range are no longer available.  Returns the number
        of pages freed."""
        freed = 0
        for s, b in enumerate(begin):
            first_kept = min(int(b), self._lens[s]) // self.page_size
            tab = self._tables[s]
            for p in range((keep_sink_tokens + self.page_size - 1) // self.page_size, first_kept):
                if tab[p] >= 0:
                    self._free.append(tab[p])
                    tab[p] = -1
                    self._bt_host[s, p] = -1
                    self._bt_dirty = True
                    freed += 1
        if freed:
            self._sync_device()
        return freed

    def compact(self, keep: Sequence[torch.Tensor]) -> List[int]:
        """Drop tokens inside the sequences: ``keep[s]`` is a boolean mask (or 0/1 tensor) over the
        ``lengths[s]`` tokens of sequence ``s``; the survivors are packed, in order, into fresh pages
        and every page that is no longer needed goes back to the pool.

        This is what the reference's ``kv_compact_triton`` (src/kernels_t/kv_ops_triton.py:159-181)
        is meant to do on its dense cache -- its kernel writes surviving row ``s`` to output row ``s``
        of a tensor with only ``num_valid`` rows (kv_ops_triton.py:83-92), so it cannot be used as
        is.  Four launches of this library's kernels: gather the kept rows of K and of V through
        their slot lists, then one append of both into the new pages.  Returns the new lengths.
        """
        if len(keep) != self.batch_size:
            raise ValueError("one mask per sequence")
        src_slots: List[int] = []
        new_lens: List[int] = []
        for s, m in enumerate(keep):
            m = torch.as_tensor(m).reshape(-1).cpu() != 0
            if m.numel() != self._lens[s]:
                raise ValueError(f"mask of sequence {s} has {m.numel()} entries for {self._lens[s]} tokens")
            kept = torch.nonzero(m).flatten().tolist()
            tab, ps = self._tables[s], self.page_size
            if any(tab[p // ps] < 0 for p in kept):
                raise ValueError(f"sequence {s}: a kept token lies on an evicted page")
            src_slots.extend(tab[p // ps] * ps + p % ps for p in kept)
            new_lens.append(len(kept))
        idx = torch.tensor(src_slots, dtype=torch.int64).to(self.device)
        # the survivors of every layer are copied out before any page is released, so re-using pages is safe
        rows = [(kv_ops(kp, idx, None, "gather", compat=False), kv_ops(vp, idx, None, "gather", compat=False))
                for kp, vp in zip(self._k_pools, self._v_pools)]                       # [1,H,T,D] each
        self.reset()
        self._reserve(new_lens)
        dst: List[int] = []
        for s, L in enumerate(new_lens):
            dst.extend(self.slots(s, 0, L))
        self._sync_device()
        if dst:
            dst_dev = torch.tensor(dst, dtype=torch.int64).to(self.device)
            for (k_rows, v_rows), kp, vp in zip(rows, self._k_pools, self._v_pools):
                # the rows are already in storage format: a raw copy, not a second quantisation
                raw = (lambda t: t.view(torch.uint8)) if kp.dtype == torch.float8_e4m3fn else (lambda t: t)
                paged_append(raw(kp), raw(vp), dst_dev, raw(k_rows)[0].permute(1, 0, 2), raw(v_rows)[0].permute(1, 0, 2),
                             self.page_size)
        return new_lens


class _LayerView:
    """Layer ``i`` of a multi-layer ``PagedKVCache``: own pools, shared tables and lengths.  Everything
    else is forwarded to the parent."""

    is_paged = True

    def __init__(self, parent: PagedKVCache, index: int):
        self._parent, self._index = parent, index
        self.k_pool, self.v_pool = parent._k_pools[index], parent._v_pools[index]

    def __getattr__(self, name):
        return getattr(self._parent, name)

    def append(self, k_new: torch.Tensor, v_new: torch.Tensor, write: bool = True) -> List[int]:
        return self._parent._append_layer(self._index, k_new, v_new, write)

    @property
    def k(self) -> torch.Tensor:
        return self._parent._dense(self.k_pool)

    @property
    def v(self) -> torch.Tensor:
        return self._parent._dense(self.v_pool)

    def gather(self, layout: str = "head_major"):
        p = self._parent
        return (paged_gather(self.k_pool, p.block_table_dev, p.ctx_len_dev, p.page_size, layout=layout),
                paged_gather(self.v_pool, p.block_table_dev, p.ctx_len_dev, p.page_size, layout=layout))
