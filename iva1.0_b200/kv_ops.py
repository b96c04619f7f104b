"""KV-cache gather / scatter operators with the reference's signatures.

``kv_ops`` keeps the contract of ``kv_ops_triton`` (src/kernels_t/kv_ops_triton.py:150-156):
``kv_cache [B,H,S,D]``, one int64 index vector shared by all batch rows and heads, gather
returns ``[B,H,N,D]``, scatter takes ``values [B,H,N,D]``; a missing ``values`` or an unknown
operation raises ``ValueError`` with the reference's messages (kv_ops_triton.py:126-127,143).

Two reference behaviours are kept behind ``compat=True`` (the default, so the function is a
drop-in) and can be switched off:

* gather returns fp32 whatever the cache dtype (kv_ops_triton.py:112);
* scatter clones the cache and leaves its input untouched (kv_ops_triton.py:129).

With ``compat=False`` gather keeps the cache dtype and scatter writes in place and returns
its first argument.  ``paged_append`` / ``paged_gather`` are the block-table forms of the same
two operators on a page pool.
"""

from __future__ import annotations

from typing import List, Optional, Sequence, Union

import torch

from . import _lib

__all__ = ["kv_ops", "kv_compact", "paged_append", "paged_gather", "read_status"]

_status_words = {}


def _status_word(device: torch.device) -> torch.Tensor:
    """One int32 per device that kernels OR error bits into (out-of-range indices are skipped
    on the device, never dereferenced)."""
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    t = _status_words.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[key] = t
    return t


def read_status(device, reset: bool = True) -> int:
    """Synchronise and return the status bits accumulated by gather/scatter calls on ``device``."""
    t = _status_word(torch.device(device))
    v = int(t.item())
    if reset and v:
        t.zero_()
    return v


def _check_status(device, check: bool) -> None:
    if check:
        v = read_status(device)
        if v:
            raise IndexError(f"iva_b200: {_lib.status_message(v)}")


def _prep_indices(indices: torch.Tensor, device) -> torch.Tensor:
    if indices.dim() != 1:
        raise ValueError("indices must be 1-D")
    return indices.to(device=device, dtype=torch.int64).contiguous()


def _inner_contiguous(t: torch.Tensor) -> torch.Tensor:
    return t if t.stride(-1) == 1 else t.contiguous()


def kv_ops(kv_cache: torch.Tensor, indices: torch.Tensor, values: Optional[torch.Tensor] = None,
           operation: str = "gather", *, compat: bool = True, check: bool = False) -> torch.Tensor:
    """Gather rows of, or scatter rows into, a ``[B,H,S,D]`` KV cache along ``S``.

    ``check=True`` synchronises and raises ``IndexError`` if an index was outside ``[0,S)``
    (such rows are skipped on the device either way).
    """
    if operation not in ("gather", "scatter"):
        raise ValueError(f"Unknown operation: {operation}")
    if operation == "scatter" and values is None:
        raise ValueError("Values tensor required for scatter operation")
    if kv_cache.dim() != 4:
        raise ValueError("kv_cache must be [batch, heads, seq, head_dim]")
    _lib.require_cuda(kv_cache, values)
    if kv_cache.requires_grad or (values is not None and values.requires_grad):
        raise RuntimeError("kv_ops is inference-only (the reference's backward returns no gradients)")
    lib = _lib.load_library()
    dev = kv_cache.device
    B, H, S, D = kv_cache.shape
    idx = _prep_indices(indices, dev)
    N = idx.numel()
    code = _lib.dtype_code(kv_cache.dtype)
    status = _status_word(dev)
    with torch.cuda.device(dev):
        stream = _lib.stream_ptr(dev)
        if operation == "gather":
            cache = _inner_contiguous(kv_cache)
            out_dtype = torch.float32 if compat else kv_cache.dtype
            out = torch.empty(B, H, N, D, device=dev, dtype=out_dtype)
            _lib.check(lib.ivab_kv_gather(
                cache.data_ptr(), idx.data_ptr(), out.data_ptr(), code, _lib.dtype_code(out_dtype),
                B, H, S, D, N, cache.stride(0), cache.stride(1), cache.stride(2),
                out.stride(0), out.stride(1), out.stride(2), status.data_ptr(), stream))
            _check_status(dev, check)
            return out
        if values.shape != (B, H, N, D):
            raise ValueError(f"values must be {[B, H, N, D]}, got {list(values.shape)}")
        vals = _inner_contiguous(values.to(kv_cache.dtype))
        if compat:
            out = kv_cache.clone(memory_format=torch.contiguous_format)
        else:
            if kv_cache.stride(-1) != 1:
                raise ValueError("in-place scatter needs a cache with a contiguous head_dim axis")
            out = kv_cache
        _lib.check(lib.ivab_kv_scatter(
            out.data_ptr(), idx.data_ptr(), vals.data_ptr(), code, B, H, S, D, N,
            out.stride(0), out.stride(1), out.stride(2), vals.stride(0), vals.stride(1), vals.stride(2),
            status.data_ptr(), stream))
        _check_status(dev, check)
        return out


def kv_compact(kv_cache: torch.Tensor, mask: torch.Tensor, *, compat: bool = True, return_counts: bool = False):
    """Keep the positions where ``mask`` is non-zero: ``[B,H,S,D] -> [B,H,num_valid,D]``.

    Signature of ``kv_compact_triton`` (src/kernels_t/kv_ops_triton.py:159-181): ``mask`` is ``[B,S]`` and
    every batch row keeps its own positions.  The reference kernel writes surviving row ``s`` to output
    row ``s`` of a tensor that only has ``num_valid`` rows (kv_ops_triton.py:83-92), which is out of
    bounds as soon as the mask has a hole; this function implements the documented intent instead: the
    survivors of row ``b`` are packed in order into ``out[b, :, :count_b]``, ``num_valid`` is the largest
    count of any row, and rows with fewer survivors are zero-filled behind them
    (``return_counts=True`` also returns the int32 counts).  Two launches -- one prefix scan per mask row,
    one row copy -- and, like the reference (kv_ops_triton.py:166), one host synchronisation to size the
    output.  ``compat=True`` returns fp32 whatever the cache dtype, as the reference allocates its output
    without a dtype (kv_ops_triton.py:168).
    """
    _lib.require_cuda(kv_cache, mask)
    if kv_cache.dim() != 4:
        raise ValueError("kv_cache must be [batch, heads, seq, head_dim]")
    if kv_cache.requires_grad:
        raise RuntimeError("kv_compact is inference-only")
    lib = _lib.load_library()
    dev = kv_cache.device
    B, H, S, D = kv_cache.shape
    if mask.numel() != B * S:
        raise ValueError(f"mask must be [{B},{S}]")
    m = (mask.reshape(B, S) != 0).to(torch.uint8).contiguous()
    idx = torch.empty(B, S, dtype=torch.int64, device=dev)
    counts = torch.empty(B, dtype=torch.int32, device=dev)
    cache = _inner_contiguous(kv_cache)
    out_dtype = torch.float32 if compat else kv_cache.dtype
    status = _status_word(dev)
    with torch.cuda.device(dev):
        stream = _lib.stream_ptr(dev)
        _lib.check(lib.ivab_compact_indices(m.data_ptr(), B, S, idx.data_ptr(), counts.data_ptr(), stream))
        n = int(counts.max().item()) if B else 0            # the host synchronisation
        out = torch.zeros(B, H, n, D, device=dev, dtype=out_dtype)
        if n:
            _lib.check(lib.ivab_kv_gather_rows(
                cache.data_ptr(), idx.data_ptr(), idx.stride(0), out.data_ptr(), _lib.dtype_code(kv_cache.dtype),
                _lib.dtype_code(out_dtype), B, H, S, D, n, cache.stride(0), cache.stride(1), cache.stride(2),
                out.stride(0), out.stride(1), out.stride(2), status.data_ptr(), stream))
    return (out, counts) if return_counts else out


def _pool_strides(pool: torch.Tensor, page_size: int):
    """(head stride, page stride) in elements of a ``[1,H,S,D]`` (head-major) or
    ``[num_pages,H,page,D]`` (page-major) pool."""
    if pool.dim() != 4 or pool.stride(-1) != 1:
        raise ValueError("pool must be 4-D with a contiguous head_dim axis")
    D = pool.shape[-1]
    if pool.shape[0] == 1 and pool.shape[2] % page_size == 0 and pool.stride(2) == D:
        return pool.shape[1], pool.shape[2] // page_size, pool.stride(1), page_size * D
    if pool.shape[2] == page_size and pool.stride(2) == D:
        return pool.shape[1], pool.shape[0], pool.stride(1), pool.stride(0)
    raise ValueError("pool must be [1,H,num_pages*page_size,D] or [num_pages,H,page_size,D]")


def paged_append(k_pool: torch.Tensor, v_pool: torch.Tensor, slot_mapping: torch.Tensor,
                 k_new: torch.Tensor, v_new: torch.Tensor, page_size: int, *, check: bool = False,
                 k_scale: float = 1.0, v_scale: float = 1.0) -> None:
    """Write ``T`` new tokens' K and V (``[T,H_kv,D]``) into their slots, in place, one launch.

    The slot mapping plays the role of ``indices`` in the reference scatter
    (src/kernels_t/kv_ops_triton.py:58-65) on the flattened slot axis of the pool; this is what
    replaces the O(L) concat of AttentionTorch.forward (src/core/attention.py:61-63).

    Pools of dtype ``torch.float8_e4m3fn`` store ``fp8(x * (1/scale))`` (saturating, round to nearest
    even) of fp16 / bf16 tokens, K with ``k_scale`` and V with ``v_scale``.
    """
    _lib.require_cuda(k_pool, v_pool, k_new, v_new)
    lib = _lib.load_library()
    dev = k_pool.device
    H, num_pages, sh, sp = _pool_strides(k_pool, page_size)
    if _pool_strides(v_pool, page_size) != (H, num_pages, sh, sp) or v_pool.dtype != k_pool.dtype:
        raise ValueError("k_pool and v_pool must have the same shape, strides and dtype")
    if k_new.dim() != 3 or k_new.shape != v_new.shape or k_new.shape[1] != H or k_new.shape[2] != k_pool.shape[-1]:
        raise ValueError("k_new / v_new must be [T, H_kv, D]")
    fp8 = k_pool.dtype == torch.float8_e4m3fn
    if fp8:
        if k_new.dtype not in (torch.float16, torch.bfloat16) or v_new.dtype != k_new.dtype:
            raise ValueError("8-bit pools take fp16 or bf16 tokens")
        k_new, v_new = _inner_contiguous(k_new), _inner_contiguous(v_new)
    else:
        k_new = _inner_contiguous(k_new.to(k_pool.dtype))
        v_new = _inner_contiguous(v_new.to(k_pool.dtype))
    if v_new.stride() != k_new.stride():
        v_new = v_new.contiguous()
        k_new = k_new.contiguous()
    slots = _prep_indices(slot_mapping, dev)
    T = k_new.shape[0]
    if slots.numel() != T:
        raise ValueError(f"slot_mapping has {slots.numel()} entries for {T} tokens")
    status = _status_word(dev)
    with torch.cuda.device(dev):
        if fp8:
            _lib.check(lib.ivab_paged_append_fp8(
                k_new.data_ptr(), v_new.data_ptr(), k_new.stride(0), k_new.stride(1), slots.data_ptr(),
                k_pool.data_ptr(), v_pool.data_ptr(), sh, sp, _lib.dtype_code(k_new.dtype), float(k_scale),
                float(v_scale), T, H, k_pool.shape[-1], page_size, num_pages, status.data_ptr(), _lib.stream_ptr(dev)))
            _check_status(dev, check)
            return
        _lib.check(lib.ivab_paged_append(
            k_new.data_ptr(), v_new.data_ptr(), k_new.stride(0), k_new.stride(1), slots.data_ptr(),
            k_pool.data_ptr(), v_pool.data_ptr(), sh, sp, _lib.dtype_code(k_pool.dtype),
            T, H, k_pool.shape[-1], page_size, num_pages, status.data_ptr(), _lib.stream_ptr(dev)))
    _check_status(dev, check)


def paged_gather(pool: torch.Tensor, block_table: torch.Tensor, ctx_len: torch.Tensor, page_size: int,
                 *, layout: str = "token_major", out_offsets: Optional[torch.Tensor] = None,
                 total_tokens: Optional[int] = None, check: bool = False, out: Optional[torch.Tensor] = None
                 ) -> Union[torch.Tensor, List[torch.Tensor]]:
    """Gather every sequence's tokens from the pool to contiguous storage in one launch.

    ``layout="token_major"`` returns one packed tensor ``[sum(L), H, D]`` (sequence ``s`` occupies
    rows ``out_offsets[s]:out_offsets[s+1]``); ``layout="head_major"`` returns a list of
    ``[1,H,L_s,D]`` views, the reference gather's output layout
    (src/kernels_t/kv_ops_triton.py:112-123).  Pass ``out_offsets`` (int64 ``[B+1]`` on the
    device) and ``total_tokens`` to avoid the host synchronisation that sizing the output
    otherwise needs.  ``out`` (with both of those) is a contiguous tensor of ``total_tokens * H * D`` elements
    to gather into; it is returned as it is.
    """
    _lib.require_cuda(pool, block_table, ctx_len)
    if layout not in ("token_major", "head_major"):
        raise ValueError(f"unknown layout {layout}")
    lib = _lib.load_library()
    dev = pool.device
    H, num_pages, sh, sp = _pool_strides(pool, page_size)
    D = pool.shape[-1]
    B = ctx_len.numel()
    bt = block_table.to(device=dev, dtype=torch.int32)
    if bt.dim() != 2 or bt.shape[0] != B or bt.stride(1) != 1:
        bt = bt.reshape(B, -1).contiguous()
    cl = ctx_len.to(device=dev, dtype=torch.int32).contiguous()
    lens_host = None
    if out_offsets is None or total_tokens is None:
        offs = torch.zeros(B + 1, dtype=torch.int64, device=dev)
        offs[1:] = torch.cumsum(cl.to(torch.int64), 0)
        lens_host = cl.cpu()
        total_tokens = int(lens_host.sum())
    else:
        offs = out_offsets.to(device=dev, dtype=torch.int64).contiguous()
    given = out
    if given is not None:
        if out_offsets is None or not given.is_contiguous() or given.dtype != pool.dtype or given.numel() != total_tokens * H * D:
            raise ValueError("out must be contiguous, of the pool's dtype, hold total_tokens*H*D elements, and come with out_offsets")
        buf = given
    else:
        # (an empty result still needs a real base pointer for the library's argument check)
        buf = torch.empty(max(total_tokens, 1), H, D, device=dev, dtype=pool.dtype)
        out = buf[:total_tokens]
    status = _status_word(dev)
    with torch.cuda.device(dev):
        _lib.check(lib.ivab_paged_gather(
            pool.data_ptr(), sh, sp, bt.data_ptr(), bt.stride(0), cl.data_ptr(), offs.data_ptr(),
            buf.data_ptr(), _lib.OUT_HEAD_MAJOR if layout == "head_major" else _lib.OUT_TOKEN_MAJOR,
            _lib.dtype_code(pool.dtype), B, H, D, page_size, num_pages, bt.shape[1],
            status.data_ptr(), _lib.stream_ptr(dev)))
    _check_status(dev, check)
    if given is not None:
        return given
    if layout == "token_major":
        return out
    if lens_host is None:
        lens_host = cl.cpu()
    flat = out.view(-1)
    res, off = [], 0
    for L in lens_host.tolist():
        res.append(flat[off * H * D:(off + L) * H * D].view(1, H, L, D))
        off += L
    return res
