"""CPU restatement of the reference's KV append / gather / decode-attention path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this module; it is
the checker used by ``tests/``, by ``__graft_entry__.smoke()`` and by the CPU-baseline
and ``--impl reference`` legs of ``bench.py``.

The reference is pure PyTorch/Triton, so the restatement uses the same PyTorch CPU
operators its call sites use (``torch.matmul``, ``F.softmax``, ``torch.cat``) and
index operations that were checked, in this repository's golden fixtures, to be
bit-equal to the reference's Triton gather/scatter kernels executed under
``TRITON_INTERPRET=1``.

Parity status: the reference holds no golden vectors or known-answer tests for this
path, so the oracle is pinned against outputs of the reference's own code
(``tests/golden/make_golden.py`` runs ``kv_ops_triton`` and ``AttentionTorch`` and
commits what they return; ``tests/test_oracle_golden.py`` replays them).

Each function cites the reference lines it follows (paths within the reference
project).
"""

from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch
import torch.nn.functional as F

FP8_MAX = 448.0   # largest finite e4m3 value


def quantize_fp8_ref(x: torch.Tensor, scale: float) -> torch.Tensor:
    """``fp8_e4m3( clamp(x * (1/scale)) )`` -- the storage format of the 8-bit pools.  The multiply
    is done in fp32 with the fp32 reciprocal of ``scale``, round to nearest even, saturating at
    +-448.  (No reference counterpart: fp8 KV is only named in configs/quant_infer.yaml:52.)"""
    inv = torch.tensor(1.0, dtype=torch.float32) / torch.tensor(scale, dtype=torch.float32)
    return (x.float() * inv).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)


def dequantize_fp8_ref(pool: torch.Tensor, scale: float) -> torch.Tensor:
    """fp32 view of an 8-bit pool: ``scale * stored`` (the widening is exact)."""
    return pool.to(torch.float32) * scale


__all__ = [
    "quantize_fp8_ref",
    "dequantize_fp8_ref",
    "kv_gather_ref",
    "kv_scatter_ref",
    "kv_ops_ref",
    "kv_compact_ref",
    "slots_for_sequence",
    "paged_append_ref",
    "paged_gather_ref",
    "attention_math_ref",
    "paged_decode_ref",
    "attention_module_ref",
    "KVCacheRef",
    "decode_step_ref",
]


# --------------------------------------------------------------------------------------------
# KV operators  (src/kernels_t/kv_ops_triton.py)
# --------------------------------------------------------------------------------------------

def kv_gather_ref(kv_cache: torch.Tensor, indices: torch.Tensor, compat_fp32: bool = True) -> torch.Tensor:
    """``out[b,h,n,:] = kv_cache[b,h,indices[n],:]``.

    Follows kv_gather_kernel (src/kernels_t/kv_ops_triton.py:33-40): one index vector
    shared by every batch row and head.  The reference allocates the output without a
    dtype (kv_ops_triton.py:112), so its result is always fp32; ``compat_fp32=False``
    keeps the cache dtype instead (values are identical, the upcast is lossless).
    """
    out = kv_cache.index_select(2, indices.to(torch.int64))
    return out.to(torch.float32) if compat_fp32 else out


def kv_scatter_ref(kv_cache: torch.Tensor, indices: torch.Tensor, values: torch.Tensor) -> torch.Tensor:
    """``out = clone(kv_cache); out[b,h,indices[n],:] = values[b,h,n,:]``.

    Follows kv_scatter_kernel (src/kernels_t/kv_ops_triton.py:58-65) and the clone at
    kv_ops_triton.py:129: the input cache is left untouched.
    """
    return kv_cache.clone().index_copy_(2, indices.to(torch.int64), values.to(kv_cache.dtype))


def kv_ops_ref(kv_cache, indices, values=None, operation="gather"):
    """Dispatch with the reference's error behaviour (kv_ops_triton.py:111-143)."""
    if operation == "gather":
        return kv_gather_ref(kv_cache, indices)
    if operation == "scatter":
        if values is None:
            raise ValueError("Values tensor required for scatter operation")
        return kv_scatter_ref(kv_cache, indices, values)
    raise ValueError(f"Unknown operation: {operation}")


# --------------------------------------------------------------------------------------------
# Paging = the reference operators on a flattened slot axis
# --------------------------------------------------------------------------------------------

def kv_compact_ref(kv_cache: torch.Tensor, mask: torch.Tensor, compat_fp32: bool = True):
    """The intent of kv_compact_triton (src/kernels_t/kv_ops_triton.py:159-181): per batch row, the
    positions where ``mask [B,S]`` is non-zero (the test at :82-84), packed in order.  The reference
    kernel stores survivor ``s`` at output row ``s`` (:86) of an output with ``mask.sum()`` rows (:166-168),
    which overruns it, so there is no reference output to pin this against; the restatement defines the
    result as ``out[b, :, :count_b] = kv_cache[b][:, kept_b]`` with ``num_valid = max_b count_b`` and zeros
    behind shorter rows.  Returns ``(out, counts)``."""
    B, H, S, D = kv_cache.shape
    m = mask.reshape(B, S) != 0
    counts = m.sum(1).to(torch.int32)
    n = int(counts.max()) if B else 0
    out = torch.zeros(B, H, n, D, dtype=torch.float32 if compat_fp32 else kv_cache.dtype)
    for b in range(B):
        keep = torch.nonzero(m[b]).flatten()
        out[b, :, :keep.numel()] = kv_cache[b].index_select(1, keep).to(out.dtype)
    return out, counts


def slots_for_sequence(block_row: torch.Tensor, length: int, page_size: int, start: int = 0) -> torch.Tensor:
    """Slot ids of logical positions ``start..length-1``: ``page_id*page_size + offset``."""
    pos = torch.arange(start, length, dtype=torch.int64)
    return block_row.to(torch.int64)[pos // page_size] * page_size + pos % page_size


def paged_append_ref(pool: torch.Tensor, slot_mapping: torch.Tensor, new_tokens: torch.Tensor) -> torch.Tensor:
    """Block-table append = the reference scatter on the slot axis.

    ``pool`` is ``[1,H,S,D]``, ``new_tokens`` is ``[T,H,D]`` (token-major), which is the
    reference's ``values[1,H,T,D]`` transposed.  Returns the updated clone.
    """
    values = new_tokens.permute(1, 0, 2).unsqueeze(0)
    return kv_scatter_ref(pool, slot_mapping, values)


def paged_gather_ref(pool: torch.Tensor, block_table: torch.Tensor, ctx_len: torch.Tensor,
                     page_size: int) -> List[torch.Tensor]:
    """Per sequence, the reference gather with that sequence's slot list; result ``[1,H,L,D]``
    in the pool's dtype (values equal the reference's fp32 result exactly)."""
    out = []
    for s in range(block_table.shape[0]):
        slots = slots_for_sequence(block_table[s], int(ctx_len[s]), page_size)
        out.append(kv_gather_ref(pool, slots, compat_fp32=False))
    return out


# --------------------------------------------------------------------------------------------
# Attention math  (src/core/attention.py)
# --------------------------------------------------------------------------------------------

def attention_math_ref(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                       scale: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """``softmax(q k^T * scale) v`` on ``[B,H,S,D]`` tensors, plus ``logsumexp`` of the
    scaled scores.

    Follows AttentionTorch.forward lines 77 (scores), 99 (softmax) and 102 (weights @ v)
    of src/core/attention.py, with every mask of lines 79-97 absent -- the decode query
    may see all cached keys, which is what the module computes with ``causal=False``.
    The logsumexp is not produced by the reference; it is taken from the same ``scores``
    tensor as line 77.
    """
    q32, k32, v32 = q.float(), k.float(), v.float()
    scores = torch.matmul(q32, k32.transpose(-2, -1)) * scale
    weights = F.softmax(scores, dim=-1)
    out = torch.matmul(weights, v32)
    lse = torch.logsumexp(scores, dim=-1)
    return out, lse


def paged_decode_ref(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                     block_table: torch.Tensor, ctx_len: torch.Tensor, page_size: int,
                     scale: Optional[float] = None,
                     seqs: Optional[List[int]] = None,
                     ctx_begin: Optional[torch.Tensor] = None,
                     sink_tokens: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Single-query attention read through the block table.

    ``q`` is ``[B,H_q,D]``; pools are ``[1,H_kv,S,D]``.  Per sequence: gather its slots
    (kv_ops_triton.py:33-40), then the attention math of attention.py:77,99,102 in fp32
    on the stored values.  Grouped-query attention (``H_q > H_kv``) repeats every KV head
    for its ``H_q/H_kv`` query heads; the reference itself is multi-head only
    (attention.py:28-31), so this is the same math applied per group.

    ``ctx_begin`` (optional) limits sequence ``s`` to the keys ``ctx_begin[s] <= j < ctx_len[s]``:
    the keys a sliding-window mask leaves visible to the newest query (attention.py:115-129 keeps
    ``[i-w+1, i]`` for query ``i``); the hidden keys are not gathered at all.  ``sink_tokens`` keeps
    the keys ``j < sink_tokens`` as well (the first ``sink_tokens`` columns of the sink mask,
    attention.py:144-145).

    Returns ``out [B,H_q,D]`` fp32 and ``lse [B,H_q]`` fp32.  A sequence of length 0
    (or an empty window) yields zeros and ``-inf``.  ``seqs`` restricts the computation to some sequences
    (rows of the others are left zero).
    """
    B, Hq, D = q.shape
    Hkv = k_pool.shape[1]
    group = Hq // Hkv
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    out = torch.zeros(B, Hq, D, dtype=torch.float32)
    lse = torch.full((B, Hq), float("-inf"), dtype=torch.float32)
    for s in (range(B) if seqs is None else seqs):
        L = int(ctx_len[s])
        b = 0 if ctx_begin is None else min(max(int(ctx_begin[s]), 0), L)
        n_sink = min(int(sink_tokens), b)
        if L == 0 or (b >= L and n_sink == 0):
            continue
        slots = slots_for_sequence(block_table[s], L, page_size, start=b)
        if n_sink:
            slots = torch.cat([slots_for_sequence(block_table[s], n_sink, page_size), slots])
        k = kv_gather_ref(k_pool, slots)            # [1,Hkv,L-b,D] fp32
        v = kv_gather_ref(v_pool, slots)
        if group > 1:
            k = k.repeat_interleave(group, dim=1)
            v = v.repeat_interleave(group, dim=1)
        o, l = attention_math_ref(q[s].view(1, Hq, 1, D), k, v, scale)
        out[s] = o.view(Hq, D)
        lse[s] = l.view(Hq)
    return out, lse


def decode_step_ref(wl, seqs: Optional[List[int]] = None):
    """One decode step on a workload: append one token per sequence, then attend over
    ``ctx_len + 1`` keys.  Returns ``(k_pool', v_pool', out, lse)``."""
    k_pool = paged_append_ref(wl.k_pool, wl.slot_mapping, wl.k_new)
    v_pool = paged_append_ref(wl.v_pool, wl.slot_mapping, wl.v_new)
    out, lse = paged_decode_ref(wl.q, k_pool, v_pool, wl.block_table, wl.ctx_len + wl.new_tokens_per_seq,
                                wl.page_size, wl.scale, seqs=seqs)
    return k_pool, v_pool, out, lse


# --------------------------------------------------------------------------------------------
# Module-level contract  (src/core/attention.py:37-110, src/core/rope_kv.py:71-137)
# --------------------------------------------------------------------------------------------

class KVCacheRef:
    """Dense cache container restated from KVCache (src/core/rope_kv.py:71-137); that file
    cannot be imported (syntax error at rope_kv.py:199-203)."""

    def __init__(self, batch_size, n_heads, head_dim, seq_len, device, dtype=torch.float16):
        self.batch_size, self.n_heads, self.head_dim = batch_size, n_heads, head_dim
        self.seq_len, self.device, self.dtype = seq_len, device, dtype
        self.k = torch.zeros(batch_size, n_heads, seq_len, head_dim, device=device, dtype=dtype)
        self.v = torch.zeros(batch_size, n_heads, seq_len, head_dim, device=device, dtype=dtype)

    def update(self, new_k, new_v, start_pos):          # rope_kv.py:98-110
        end_pos = start_pos + new_k.size(2)
        if end_pos > self.seq_len:
            self.resize(end_pos)
        self.k[:, :, start_pos:end_pos] = new_k
        self.v[:, :, start_pos:end_pos] = new_v

    def resize(self, new_seq_len):                      # rope_kv.py:112-130
        if new_seq_len <= self.seq_len:
            return
        shape = (self.batch_size, self.n_heads, new_seq_len, self.head_dim)
        nk = torch.zeros(shape, device=self.device, dtype=self.dtype)
        nv = torch.zeros(shape, device=self.device, dtype=self.dtype)
        nk[:, :, :self.seq_len] = self.k
        nv[:, :, :self.seq_len] = self.v
        self.k, self.v, self.seq_len = nk, nv, new_seq_len

    def clear(self):                                    # rope_kv.py:132-134
        self.k.zero_()
        self.v.zero_()

    def get_slice(self, start, end):                    # rope_kv.py:136-137
        return self.k[:, :, start:end], self.v[:, :, start:end]


def attention_module_ref(x, wq, wk, wv, wo, n_heads, cache_k=None, cache_v=None, sliding_window=None,
                         attention_mask=None):
    """AttentionTorch.forward (src/core/attention.py:46-110) with ``causal=False``, eval mode:
    projections (:49-55), cache concat (:61-63), attention (:77,99,102), optional sliding-window
    mask (:83-87,115-129; query ``i`` keeps keys ``max(0,i-w+1)..i``), optional key padding mask
    ``[B,L]`` (:95-97), output projection (:104-108).  Returns ``(output, k_all, v_all)``."""
    B, S, dm = x.shape
    hd = dm // n_heads
    q = F.linear(x, wq).view(B, S, n_heads, hd).transpose(1, 2)
    k = F.linear(x, wk).view(B, S, n_heads, hd).transpose(1, 2)
    v = F.linear(x, wv).view(B, S, n_heads, hd).transpose(1, 2)
    if cache_k is not None:
        k = torch.cat([cache_k, k], dim=2)
        v = torch.cat([cache_v, v], dim=2)
    scores = torch.matmul(q, k.transpose(-2, -1)) * (1.0 / math.sqrt(hd))
    if sliding_window is not None:
        mask = torch.zeros(S, k.size(2))
        for i in range(S):
            mask[i, max(0, i - sliding_window + 1):min(k.size(2), i + 1)] = 1
        scores = scores.masked_fill(mask == 0, float("-inf"))
    if attention_mask is not None:
        scores = scores.masked_fill(attention_mask.unsqueeze(1).unsqueeze(2) == 0, float("-inf"))
    w = F.softmax(scores, dim=-1)
    o = torch.matmul(w, v).transpose(1, 2).contiguous().view(B, S, dm)
    return F.linear(o, wo), k, v
