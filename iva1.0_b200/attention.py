"""Single-query decode attention through a block table, behind the reference's contracts.

* ``paged_decode_attention`` -- the native operator: q ``[B,H_q,D]``, page pools, block table,
  context lengths -> ``out [B,H_q,D]`` (+ per-head logsumexp).
* ``attention(q, k, v, scale, dropout_prob, training)`` -- the signature of ``attention_triton``
  (src/kernels_t/attention_triton.py:215-223) on ``[B,H,S,D]`` tensors.  The reference kernel
  behind that signature cannot run; the math implemented here is the one the model really
  uses, AttentionTorch.forward lines 77, 99, 102 (src/core/attention.py) without masks.
* ``AttentionB200`` -- an ``nn.Module`` with AttentionTorch's parameters and forward signature
  (src/core/attention.py:19-45), so ``load_state_dict`` round-trips with the reference module;
  ``get_attention(config)`` mirrors the reference factory (attention.py:190-194).

Inference only: no dropout, no autograd.
"""

from __future__ import annotations

import ctypes
import math
from typing import Any, Dict, Optional, Tuple

import torch
import torch.nn as nn

from . import _lib
from .kv_ops import _pool_strides

__all__ = ["paged_decode_attention", "paged_decode_step", "attention", "AttentionB200", "get_attention",
           "decode_workspace_bytes", "decode_status"]

_workspaces: Dict[Tuple[int, int], torch.Tensor] = {}   # insertion order = least recently used first
_MAX_WORKSPACES = 8


def decode_workspace_bytes(batch: int, q_heads: int, kv_heads: int, head_dim: int) -> int:
    """Scratch bytes one ``paged_decode_attention`` call needs on the current device."""
    lib = _lib.load_library()
    n = ctypes.c_size_t(0)
    _lib.check(lib.ivab_decode_workspace_bytes(batch, q_heads, kv_heads, head_dim, ctypes.byref(n)))
    return int(n.value)


def _workspace(device: torch.device, stream: int, nbytes: int) -> torch.Tensor:
    """One scratch buffer per (device, stream), grown on demand.  Calls on the same stream are
    ordered, so they can share it; calls on different streams get different buffers."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream)
    ws = _workspaces.pop(key, None)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
    _workspaces[key] = ws                       # (re)inserted as the most recently used
    # Streams come and go; keep the cache bounded.  A dropped buffer was allocated while its stream was
    # current, so the caching allocator only reuses it in that stream's order -- after the calls that used it.
    while len(_workspaces) > _MAX_WORKSPACES:
        _workspaces.pop(next(iter(_workspaces)))
    return ws


def decode_status(workspace: torch.Tensor) -> int:
    """Synchronise and return the device status bits of the last decode call on ``workspace``
    (0 = fine)."""
    lib = _lib.load_library()
    v = ctypes.c_int32(0)
    with torch.cuda.device(workspace.device):
        rc = lib.ivab_decode_status(workspace.data_ptr(), ctypes.byref(v), _lib.stream_ptr(workspace.device))
    if rc not in (_lib.OK, _lib.ERR_DEVICE):
        _lib.check(rc)
    return int(v.value)


def paged_decode_attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                           block_table: torch.Tensor, ctx_len: torch.Tensor, page_size: int = 16,
                           scale: Optional[float] = None, *, out: Optional[torch.Tensor] = None,
                           lse: Optional[torch.Tensor] = None, return_lse: bool = False,
                           workspace: Optional[torch.Tensor] = None, check: bool = False,
                           ctx_begin: Optional[torch.Tensor] = None, sink_tokens: int = 0,
                           k_scale: float = 1.0, v_scale: float = 1.0, out_dtype: Optional[torch.dtype] = None,
                           exchange=None):
    """``out[s,h] = softmax(q[s,h] . K_s^T * scale) . V_s`` over the ``ctx_len[s]`` cached tokens of
    sequence ``s``, K/V read in place from the page pool through ``block_table``.

    q ``[B,H_q,D]``; pools ``[1,H_kv,num_pages*page_size,D]`` (or ``[num_pages,H_kv,page_size,D]``);
    ``block_table`` int32 ``[B,max_pages]``; ``ctx_len`` int32 ``[B]``.  ``H_q/H_kv`` from 1 to 8, or larger and divisible into equal groups of at most 8 (12, 16, 32, 64 ...).
    Returns ``out`` (dtype of q) or ``(out, lse)`` with ``lse`` fp32 ``[B,H_q]`` (natural log).
    ``out_dtype=torch.float32`` (or an fp32 ``out`` tensor) returns the kernels' fp32 result without the
    final rounding to q's 16-bit type, as the reference does for fp32 inputs.
    ``check=True`` synchronises and raises if the kernels flagged a bad page id / length or a
    timed-out wait.  ``ctx_begin`` (int32 ``[B]``, optional) restricts sequence ``s`` to the keys
    ``ctx_begin[s] <= j < ctx_len[s]`` -- a sliding window; pages wholly before it are not read.
    ``sink_tokens`` keeps the first keys of every sequence visible in front of the window.
    Pools of dtype ``torch.float8_e4m3fn`` (written by ``paged_append`` with the same scales) are read
    as ``K = k_scale * stored``, ``V = v_scale * stored``; q must then be fp16 or bf16.
    """
    _lib.require_cuda(q, k_pool, v_pool, block_table, ctx_len)
    Hkv, num_pages, sh, sp = _pool_strides(k_pool, page_size)
    if _pool_strides(v_pool, page_size) != (Hkv, num_pages, sh, sp) or v_pool.dtype != k_pool.dtype:
        raise ValueError("k_pool and v_pool must have the same shape, strides and dtype")
    fp8 = k_pool.dtype == torch.float8_e4m3fn
    if k_pool.shape[-1] != q.shape[-1] or (k_pool.dtype != q.dtype and not fp8):
        raise ValueError("q and the pools must share dtype and head_dim")
    if fp8 and q.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("8-bit pools need fp16 or bf16 queries")
    return _decode(q, k_pool, v_pool, Hkv, num_pages, sh, sp, block_table, ctx_len, page_size, scale,
                   out, lse, return_lse, workspace, check, ctx_begin, sink_tokens,
                   (float(k_scale), float(v_scale)) if fp8 else None, out_dtype, exchange=exchange)


def paged_decode_step(q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, k_pool: torch.Tensor,
                      v_pool: torch.Tensor, block_table: torch.Tensor, ctx_len: torch.Tensor, page_size: int = 16,
                      scale: Optional[float] = None, *, out: Optional[torch.Tensor] = None,
                      lse: Optional[torch.Tensor] = None, return_lse: bool = False,
                      workspace: Optional[torch.Tensor] = None, check: bool = False,
                      ctx_begin: Optional[torch.Tensor] = None, sink_tokens: int = 0,
                      k_scale: float = 1.0, v_scale: float = 1.0, out_dtype: Optional[torch.dtype] = None,
                      exchange=None):
    """One decode step in one call: append one new token per sequence (``k_new`` / ``v_new`` ``[B,H_kv,D]`` in q's
    dtype) and attend over the cache including it -- ``paged_append`` followed by ``paged_decode_attention``
    without the separate copy launch (the concat-append plus attention of src/core/attention.py:61-63,77,99,102
    for a one-token step).  ``ctx_len`` INCLUDES the new token, which is stored at position ``ctx_len[s] - 1``
    through the block table (its page must already be in the table).  The pools end up bit-identical to the
    two-call sequence, and so does the result.  Other arguments as for ``paged_decode_attention``."""
    # q, the new tokens and the lengths may also be pinned host tensors, read in place by the kernels (the pools and
    # the block table, which are read many times, have to be in device memory)
    _lib.require_cuda(k_pool, v_pool, block_table)
    _lib.require_device_readable(q, k_new, v_new, ctx_len)
    Hkv, num_pages, sh, sp = _pool_strides(k_pool, page_size)
    if _pool_strides(v_pool, page_size) != (Hkv, num_pages, sh, sp) or v_pool.dtype != k_pool.dtype:
        raise ValueError("k_pool and v_pool must have the same shape, strides and dtype")
    fp8 = k_pool.dtype == torch.float8_e4m3fn
    if k_pool.shape[-1] != q.shape[-1] or (k_pool.dtype != q.dtype and not fp8):
        raise ValueError("q and the pools must share dtype and head_dim")
    if fp8 and q.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("8-bit pools need fp16 or bf16 queries")
    B, D = q.shape[0], q.shape[-1]
    if k_new.shape != (B, Hkv, D) or v_new.shape != k_new.shape or k_new.dtype != q.dtype or v_new.dtype != q.dtype:
        raise ValueError("k_new / v_new must be [B, H_kv, D] in q's dtype")
    if k_new.stride(-1) != 1 or v_new.stride() != k_new.stride():
        k_new, v_new = k_new.contiguous(), v_new.contiguous()
    return _decode(q, k_pool, v_pool, Hkv, num_pages, sh, sp, block_table, ctx_len, page_size, scale,
                   out, lse, return_lse, workspace, check, ctx_begin, sink_tokens,
                   (float(k_scale), float(v_scale)) if fp8 else None, out_dtype, new_tokens=(k_new, v_new), exchange=exchange)


def _decode(q, k_base, v_base, Hkv, num_pages, sh, sp, block_table, ctx_len, page_size, scale,
            out, lse, return_lse, workspace, check, ctx_begin=None, sink_tokens=0, fp8_scales=None, out_dtype=None,
            new_tokens=None, exchange=None):
    """Argument checks and the library call; ``k_base`` / ``v_base`` only supply base pointers, the
    pool geometry is given by ``Hkv, num_pages, sh, sp`` (element strides of head and page).
    ``new_tokens=(k_new, v_new)`` selects the fused step (append + attention)."""
    if q.requires_grad:
        raise RuntimeError("paged_decode_attention is inference-only")
    lib = _lib.load_library()
    dev = k_base.device
    if q.dim() != 3:
        raise ValueError("q must be [batch, q_heads, head_dim]")
    B, Hq, D = q.shape
    if Hq % Hkv:
        raise ValueError("q_heads must be a multiple of kv_heads")
    if q.stride(-1) != 1:
        q = q.contiguous()
    if block_table.dtype != torch.int32 or block_table.dim() != 2 or block_table.stride(1) != 1:
        block_table = block_table.to(torch.int32).reshape(B, -1).contiguous()
    if ctx_len.dtype != torch.int32 or not ctx_len.is_contiguous():
        ctx_len = ctx_len.to(torch.int32).contiguous()
    if block_table.shape[0] != B or ctx_len.numel() != B:
        raise ValueError("block_table / ctx_len batch size does not match q")
    if ctx_begin is not None:
        _lib.require_cuda(ctx_begin)
        if ctx_begin.dtype != torch.int32 or not ctx_begin.is_contiguous():
            ctx_begin = ctx_begin.to(torch.int32).contiguous()
        if ctx_begin.numel() != B:
            raise ValueError("ctx_begin batch size does not match q")
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    if out_dtype is None:
        out_dtype = out.dtype if out is not None else q.dtype
    if out_dtype not in (q.dtype, torch.float32):
        raise ValueError("out_dtype must be q's dtype or torch.float32")
    if out is None:
        out = torch.empty(B, Hq, D, device=dev, dtype=out_dtype)
    elif out.shape != (B, Hq, D) or out.dtype != out_dtype or out.stride(-1) != 1:
        raise ValueError("out must be [B,H_q,D] in q's dtype (or fp32) with a contiguous last axis")
    if lse is None and return_lse:
        lse = torch.empty(B, Hq, device=dev, dtype=torch.float32)
    if lse is not None and (lse.shape != (B, Hq) or lse.dtype != torch.float32 or not lse.is_contiguous()):
        raise ValueError("lse must be a contiguous fp32 [B,H_q] tensor")
    with torch.cuda.device(dev):
        stream = _lib.stream_ptr(dev)
        if workspace is None:
            workspace = _workspace(dev, stream, decode_workspace_bytes(B, Hq, Hkv, D))
        tail = (block_table.data_ptr(), block_table.stride(0), ctx_len.data_ptr(),
                ctx_begin.data_ptr() if ctx_begin is not None else None, int(sink_tokens),
                out.data_ptr(), out.stride(0), out.stride(1), lse.data_ptr() if lse is not None else None,
                _lib.dtype_code(q.dtype), _lib.dtype_code(out_dtype), B, Hq, Hkv, D, page_size, num_pages,
                block_table.shape[1],
                float(scale), workspace.data_ptr(), workspace.numel(), stream)
        head = (q.data_ptr(), q.stride(0), q.stride(1), k_base.data_ptr(), v_base.data_ptr(), sh, sp)
        if exchange is not None:
            # head-parallel step: ``exchange = (PeerExchange, block)``; out / lse are fp32 views into ``block``, which the
            # merge kernel's last CTA sends to the peers (sharding.HeadParallelDecoder sets this up)
            px, block = exchange
            if out_dtype != torch.float32 or lse is None:
                raise ValueError("a step with an exchange writes fp32 rows and the logsumexp into the exchanged block")
            kn, vn = new_tokens if new_tokens is not None else (None, None)
            ks, vs = fp8_scales if fp8_scales is not None else (1.0, 1.0)
            _lib.check(lib.ivab_paged_decode_step_allgather(
                q.data_ptr(), q.stride(0), q.stride(1), kn.data_ptr() if kn is not None else None,
                vn.data_ptr() if vn is not None else None, kn.stride(0) if kn is not None else 0,
                kn.stride(1) if kn is not None else 0, k_base.data_ptr(), v_base.data_ptr(), sh, sp,
                _lib.F8E4M3 if fp8_scales is not None else _lib.dtype_code(q.dtype), ks, vs,
                block_table.data_ptr(), block_table.stride(0), ctx_len.data_ptr(),
                ctx_begin.data_ptr() if ctx_begin is not None else None, int(sink_tokens),
                out.data_ptr(), out.stride(0), out.stride(1), lse.data_ptr(), _lib.dtype_code(q.dtype),
                B, Hq, Hkv, D, page_size, num_pages, block_table.shape[1], float(scale), workspace.data_ptr(), workspace.numel(),
                *px.exchange_args(block), stream))
        elif new_tokens is not None:
            kn, vn = new_tokens
            ks, vs = fp8_scales if fp8_scales is not None else (1.0, 1.0)
            _lib.check(lib.ivab_paged_decode_step(
                q.data_ptr(), q.stride(0), q.stride(1), kn.data_ptr(), vn.data_ptr(), kn.stride(0), kn.stride(1),
                k_base.data_ptr(), v_base.data_ptr(), sh, sp,
                _lib.F8E4M3 if fp8_scales is not None else _lib.dtype_code(q.dtype), ks, vs, *tail))
        elif fp8_scales is None:
            _lib.check(lib.ivab_paged_decode_attn(*head, *tail))
        else:
            _lib.check(lib.ivab_paged_decode_attn_fp8(*head, fp8_scales[0], fp8_scales[1], *tail))
    if check:
        st = decode_status(workspace)
        if st:
            raise _lib.IvabError(_lib.ERR_DEVICE, _lib.status_message(st))
    return (out, lse) if (return_lse or lse is not None) else out


_PAGE = 16


def _mask_to_key_range(attention_mask: torch.Tensor, B: int, L: int):
    """A key padding mask ``[B,L]`` (non-zero = visible, src/core/attention.py:95-97) as the key range
    ``[begin_b, end_b)`` of every row.  Only what padding produces is representable without a mask
    tensor in the kernels: one contiguous run of visible keys per row (right padding, left padding, or
    both).  Anything else raises.  Costs one host synchronisation (the check)."""
    m = attention_mask.reshape(B, -1) != 0
    if m.shape[1] != L:
        raise ValueError(f"attention_mask covers {m.shape[1]} keys, the layer sees {L}")
    idx = torch.arange(L, device=m.device, dtype=torch.int32)
    count = m.sum(1, dtype=torch.int32)
    begin = torch.where(m, idx, L).amin(1).to(torch.int32)
    end = (torch.where(m, idx, -1).amax(1) + 1).to(torch.int32)
    begin = torch.where(count > 0, begin, torch.zeros_like(begin))
    if not bool((end - begin == count).all()):
        raise NotImplementedError("attention_mask must keep one contiguous run of keys per row (padding at either end)")
    return begin.contiguous(), end.contiguous()


def _dense_as_pool(k: torch.Tensor, v: torch.Tensor):
    """View dense ``[B,H,L,D]`` K/V as a page pool plus a block table.

    With ``L`` a multiple of 16, rows ``16p..16p+15`` of (batch b, head h) are already one
    contiguous page; numbering pages ``b*H*L/16 + p`` with a head stride of ``L*D`` addresses
    them without moving a byte.  Other lengths are zero-padded to the next multiple first."""
    B, H, L, D = k.shape
    Lp = (L + _PAGE - 1) // _PAGE * _PAGE
    if Lp != L or not k.is_contiguous() or not v.is_contiguous():
        kp = k.new_zeros(B, H, Lp, D)
        vp = v.new_zeros(B, H, Lp, D)
        kp[:, :, :L] = k
        vp[:, :, :L] = v
        k, v = kp, vp
    pages_per_row = Lp // _PAGE
    n_pages = B * H * pages_per_row
    bt = (torch.arange(B, device=k.device, dtype=torch.int32).view(B, 1) * (H * pages_per_row)
          + torch.arange(pages_per_row, device=k.device, dtype=torch.int32).view(1, -1))
    # pool geometry: head stride Lp*D, page stride 16*D (elements)
    return k, v, bt.contiguous(), n_pages, Lp * D, _PAGE * D


def _pack_queries(q: torch.Tensor, Hkv: int):
    """Queries of one batch row that see the same keys can share one pass over them: ``q [B,S,H_q,D]`` becomes
    ``[B*ceil(S/Sc), H_kv*Sc*G, D]`` -- pseudo-sequences of ``Sc = 8 // G`` queries whose ``Sc*G`` rows per KV head
    the kernels treat as one query-head group (K/V pages are read once per group).  Returns the packed tensor,
    ``Sc`` and the number of pseudo-sequences per row; ``Sc == 1`` means nothing is gained."""
    B, S, Hq, D = q.shape
    G = Hq // Hkv
    Sc = max(1, min(8 // G if G <= 8 else 1, S))
    nS = (S + Sc - 1) // Sc
    if Sc == 1:
        return q.reshape(B * S, Hq, D), 1, S
    if nS * Sc != S:
        q = torch.cat([q, q.new_zeros(B, nS * Sc - S, Hq, D)], dim=1)      # padding rows, dropped again by _unpack_rows
    q2 = q.view(B, nS, Sc, Hkv, G, D).permute(0, 1, 3, 2, 4, 5).reshape(B * nS, Hkv * Sc * G, D)
    return q2, Sc, nS


def _unpack_rows(o2: torch.Tensor, B: int, S: int, Hkv: int, G: int, Sc: int, nS: int) -> torch.Tensor:
    """Inverse of ``_pack_queries`` for results ``[B*nS, H_kv*Sc*G, ...]`` -> ``[B, S, H_q, ...]``."""
    tail = o2.shape[2:]
    o = o2.view(B, nS, Hkv, Sc, G, *tail).transpose(2, 3).reshape(B, nS * Sc, Hkv * G, *tail)
    return o[:, :S]


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, dropout_prob: float = 0.0,
              training: bool = True, *, ctx_len: Optional[torch.Tensor] = None,
              ctx_begin: Optional[torch.Tensor] = None, return_lse: bool = False,
              out_dtype: Optional[torch.dtype] = None):
    """``softmax(q k^T * scale) v`` on ``[B,H,S,D]`` queries against ``[B,H,L,D]`` keys/values.

    Signature of ``attention_triton`` (src/kernels_t/attention_triton.py:215-223).  Every query
    row sees all ``L`` keys (the reference module's behaviour with ``causal=False``,
    src/core/attention.py:77-102); pass ``ctx_len`` (int32 ``[B,S]`` or ``[B]``) to limit the keys
    each query sees, e.g. ``prior + i + 1`` for causal prefill, and ``ctx_begin`` (same shapes) for
    the first key it sees (sliding window).  ``out_dtype=torch.float32`` returns the fp32 result for
    16-bit inputs.  Dropout is not implemented:
    a non-zero ``dropout_prob`` with ``training=True`` raises, as does ``requires_grad``.
    """
    _lib.require_cuda(q, k, v)
    if q.dim() != 4 or k.dim() != 4 or k.shape != v.shape:
        raise ValueError("q, k, v must be [batch, heads, seq, head_dim]")
    if dropout_prob != 0.0 and training:
        raise NotImplementedError("attention dropout is not implemented (inference-only backend)")
    if q.requires_grad or k.requires_grad or v.requires_grad:
        raise RuntimeError("attention is inference-only: call it under torch.no_grad() on detached tensors")
    B, Hq, S, D = q.shape
    Bk, Hkv, L, Dk = k.shape
    if Bk != B or Dk != D or Hq % Hkv:
        raise ValueError("q and k/v shapes do not match")
    kd, vd, bt, n_pages, sh, sp = _dense_as_pool(k.to(q.dtype), v.to(q.dtype))
    shared = S > 1 and (ctx_len is None or ctx_len.numel() == B) and (ctx_begin is None or ctx_begin.numel() == B)
    if shared:
        # every query of a row sees the same keys: up to eight (query, head) rows per KV head share one pass over them
        q2, Sc, nS = _pack_queries(q.permute(0, 2, 1, 3), Hkv)
        if Sc > 1:
            cl = (torch.full((B,), L, dtype=torch.int32, device=q.device) if ctx_len is None
                  else ctx_len.to(device=q.device, dtype=torch.int32).reshape(B)).repeat_interleave(nS).contiguous()
            cb = None if ctx_begin is None else ctx_begin.to(device=q.device, dtype=torch.int32).reshape(B).repeat_interleave(nS).contiguous()
            res = _decode(q2.contiguous(), kd, vd, Hkv, n_pages, sh, sp, bt.repeat_interleave(nS, dim=0), cl, _PAGE, scale,
                          None, None, return_lse, None, False, cb, out_dtype=out_dtype)
            o2, lse = res if return_lse else (res, None)
            G = Hq // Hkv
            o = _unpack_rows(o2, B, S, Hkv, G, Sc, nS).permute(0, 2, 1, 3)
            if return_lse:
                return o, _unpack_rows(lse, B, S, Hkv, G, Sc, nS).permute(0, 2, 1)
            return o
    # one pseudo-sequence per (batch row, query position), all sharing the row's block table
    q2 = q.permute(0, 2, 1, 3).reshape(B * S, Hq, D)
    bt2 = bt.repeat_interleave(S, dim=0) if S > 1 else bt
    if ctx_len is None:
        cl = torch.full((B * S,), L, dtype=torch.int32, device=q.device)
    else:
        cl = ctx_len.to(device=q.device, dtype=torch.int32)
        cl = (cl.view(B, 1).expand(B, S) if cl.numel() == B else cl.reshape(B, S)).reshape(-1).contiguous()
    cb = None
    if ctx_begin is not None:
        cb = ctx_begin.to(device=q.device, dtype=torch.int32)
        cb = (cb.view(B, 1).expand(B, S) if cb.numel() == B else cb.reshape(B, S)).reshape(-1).contiguous()
    res = _decode(q2, kd, vd, Hkv, n_pages, sh, sp, bt2, cl, _PAGE, scale, None, None, return_lse, None, False, cb,
                  out_dtype=out_dtype)
    o2, lse = res if return_lse else (res, None)
    o = o2.view(B, S, Hq, D).permute(0, 2, 1, 3)
    if return_lse:
        return o, lse.view(B, S, Hq).permute(0, 2, 1)
    return o


class AttentionB200(nn.Module):
    """Drop-in for the reference attention modules (src/core/attention.py:17-110,151-187).

    Same parameters (bias-free ``q_proj/k_proj/v_proj/o_proj``, ``d_model -> d_model``), same
    ``forward`` signature and return value ``(output [B,S,d_model], new_kv_cache)``.

    * ``kv_cache`` is a ``PagedKVCache`` (or one layer of it, ``cache.layer(i)``): the new tokens' K/V are appended to its page pool in
      place and attention reads the pool through the block table; the same cache object is
      returned.
    * ``kv_cache`` is any object with dense ``.k/.v [B,H,L,D]`` (the reference ``KVCache``): the
      reference's concat semantics are kept (attention.py:61-73) and a new cache object of the
      same type is returned.
    * ``kv_cache`` is ``None``: attention over the ``S`` tokens of ``x`` only.

    ``config.causal`` is honoured as "query ``i`` sees the cache and tokens ``0..i``".  (The
    reference builds ``tril(ones(S, L+S))`` (attention.py:80), which with a cache hides all but
    the first ``i+1`` *cached* keys; that is not reproduced.  With ``causal=False`` the results
    equal the reference's.)  ``sliding_window=w`` limits query ``i`` (absolute position) to the keys
    ``i-w+1 .. i``, which is the reference's window mask (attention.py:115-129) for a call without a
    cache; with a cache the reference's mask indexes queries from 0 and hides everything but the
    oldest keys, so there the documented meaning is implemented instead.  Keys outside the window
    are not masked but skipped: their pages are never read and a ``PagedKVCache`` can hand them back
    (``evict_before``).  ``sink_cfg={"sink_tokens": n}`` together with a sliding window keeps the first
    ``n`` keys visible in front of the window (the reference ANDs its sink mask, attention.py:131-148,
    with the window mask, which keeps nothing extra; the streaming-attention meaning of the option is
    implemented).  ``attention_mask`` is the reference's key padding mask ``[B,L]`` (attention.py:95-97):
    it is translated into a key range per row (padding at either end; a mask with holes raises), which
    costs one host synchronisation per call.  A row whose mask hides every key yields zeros (the
    reference's softmax over an all-masked row yields NaN).  RoPE state is ignored, as in the reference.
    """

    def __init__(self, config):
        super().__init__()
        self.config = config
        self.d_model = config.d_model
        self.n_heads = config.n_heads
        self.head_dim = config.d_model // config.n_heads
        self.dropout = getattr(config, "dropout", 0.0)
        self.causal = getattr(config, "causal", True)
        self.q_proj = nn.Linear(self.d_model, self.d_model, bias=False)
        self.k_proj = nn.Linear(self.d_model, self.d_model, bias=False)
        self.v_proj = nn.Linear(self.d_model, self.d_model, bias=False)
        self.o_proj = nn.Linear(self.d_model, self.d_model, bias=False)
        self.scale = 1.0 / math.sqrt(self.head_dim)

    @torch.no_grad()
    def forward(self, x: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
                kv_cache: Optional[Any] = None, rope_state: Optional[torch.Tensor] = None,
                sliding_window: Optional[int] = None, sink_cfg: Optional[Dict[str, Any]] = None
                ) -> Tuple[torch.Tensor, Optional[Any]]:
        sink = int(sink_cfg.get("sink_tokens", 4)) if sink_cfg is not None else 0
        if sink and (sliding_window is None or not getattr(kv_cache, "is_paged", False) or x.shape[1] != 1):
            raise NotImplementedError("sink_cfg is supported for single-token decode on a PagedKVCache with a sliding window")
        if self.training and self.dropout:
            raise NotImplementedError("AttentionB200 is inference-only: call .eval()")
        B, S, dm = x.shape
        H, D = self.n_heads, self.head_dim
        q = self.q_proj(x).view(B, S, H, D)
        k = self.k_proj(x).view(B, S, H, D)
        v = self.v_proj(x).view(B, S, H, D)
        # rope_state is accepted and ignored, like the reference's _apply_rope (attention.py:112-113)

        if getattr(kv_cache, "is_paged", False):
            # a plain one-token step writes the new token inside the attention launch (paged_decode_step);
            # the cache then only does this step's bookkeeping (pages, lengths, table upload)
            fused = S == 1 and attention_mask is None
            prior = kv_cache.append(k, v, write=not fused)    # [B] lengths before the append (host list)
            bt, cl = kv_cache.block_table_dev, kv_cache.ctx_len_dev
            if attention_mask is not None:
                # padding: keys [m_begin, m_end) of each row are real (attention.py:95-97 hides the others)
                if S != 1:
                    raise NotImplementedError("attention_mask with a paged cache is supported for single-token decode")
                m_begin, m_end = _mask_to_key_range(attention_mask, B, max(prior) + 1)
                cl = torch.minimum(cl, m_end)
                cb = m_begin if sliding_window is None else torch.maximum(m_begin, (cl - int(sliding_window)).clamp_(min=0))
                if sink:
                    raise NotImplementedError("sink_cfg together with attention_mask")
                o = paged_decode_attention(q.reshape(B, H, D), kv_cache.k_pool, kv_cache.v_pool, bt, cl,
                                           kv_cache.page_size, self.scale, ctx_begin=cb)
            elif S == 1:
                cb = None if sliding_window is None else (cl - int(sliding_window)).clamp_(min=0)
                scales = dict(k_scale=kv_cache.k_scale, v_scale=kv_cache.v_scale)
                o = paged_decode_step(q.reshape(B, H, D), k.reshape(B, H, D), v.reshape(B, H, D), kv_cache.k_pool,
                                      kv_cache.v_pool, bt, cl, kv_cache.page_size, self.scale, ctx_begin=cb,
                                      sink_tokens=sink, **scales)
            elif not self.causal and sliding_window is None and 8 // max(1, H // kv_cache.n_heads) > 1:
                # every query of the chunk sees the whole cache (the reference's working configuration): up to eight
                # (query, head) rows per KV head share one pass over the pages
                q2, Sc, nS = _pack_queries(q, kv_cache.n_heads)
                o2 = paged_decode_attention(q2.contiguous(), kv_cache.k_pool, kv_cache.v_pool, bt.repeat_interleave(nS, dim=0),
                                            cl.repeat_interleave(nS).contiguous(), kv_cache.page_size, self.scale,
                                            k_scale=kv_cache.k_scale, v_scale=kv_cache.v_scale)
                o = _unpack_rows(o2, B, S, kv_cache.n_heads, H // kv_cache.n_heads, Sc, nS)
            else:
                q2 = q.reshape(B * S, H, D)
                bt2 = bt.repeat_interleave(S, dim=0)
                if self.causal:
                    base = torch.tensor(prior, dtype=torch.int32, device=x.device).view(B, 1)
                    cl2 = (base + torch.arange(1, S + 1, dtype=torch.int32, device=x.device).view(1, S)).reshape(-1)
                else:
                    cl2 = cl.repeat_interleave(S)
                cb2 = None
                if sliding_window is not None:   # query i of the chunk sits at absolute position prior + i
                    base = torch.tensor(prior, dtype=torch.int32, device=x.device).view(B, 1)
                    pos = base + torch.arange(S, dtype=torch.int32, device=x.device).view(1, S)
                    cb2 = (pos + 1 - int(sliding_window)).clamp_(min=0).reshape(-1).contiguous()
                    cl2 = torch.minimum(cl2.view(B, S), pos + 1).reshape(-1) if not self.causal else cl2
                o = paged_decode_attention(q2, kv_cache.k_pool, kv_cache.v_pool, bt2, cl2.contiguous(),
                                           kv_cache.page_size, self.scale, ctx_begin=cb2,
                                           k_scale=kv_cache.k_scale, v_scale=kv_cache.v_scale)
            new_cache = kv_cache
            o = o.reshape(B, S, dm)
        else:
            kh, vh = k.transpose(1, 2), v.transpose(1, 2)     # [B,H,S,D]
            prior_len = 0
            new_cache = None
            if kv_cache is not None:
                prior_len = kv_cache.k.size(2)
                kh = torch.cat([kv_cache.k.to(kh.dtype), kh], dim=2)
                vh = torch.cat([kv_cache.v.to(vh.dtype), vh], dim=2)
                new_cache = type(kv_cache)(batch_size=kv_cache.batch_size, n_heads=kv_cache.n_heads,
                                           head_dim=kv_cache.head_dim, seq_len=kv_cache.seq_len + S,
                                           device=x.device)
                new_cache.k, new_cache.v = kh, vh
            cl = cb = None
            pos1 = (prior_len + torch.arange(1, S + 1, dtype=torch.int32, device=x.device)).view(1, S).expand(B, S)
            if (self.causal and S > 1) or sliding_window is not None:
                cl = pos1                       # the window mask also hides the keys after the query
            if sliding_window is not None:
                cb = (pos1 - int(sliding_window)).clamp(min=0)
            if attention_mask is not None:
                m_begin, m_end = _mask_to_key_range(attention_mask, B, kh.shape[2])
                m_begin, m_end = m_begin.view(B, 1).expand(B, S), m_end.view(B, 1).expand(B, S)
                cl = m_end if cl is None else torch.minimum(cl.to(torch.int32), m_end)
                cb = m_begin if cb is None else torch.maximum(cb.to(torch.int32), m_begin)
            o = attention(q.transpose(1, 2), kh, vh, self.scale, 0.0, False, ctx_len=cl, ctx_begin=cb)
            o = o.transpose(1, 2).reshape(B, S, dm)
        return self.o_proj(o), new_cache


def get_attention(config) -> nn.Module:
    """Factory with the reference's name (src/core/attention.py:190-194).  The reference admits
    ``attn_impl in {"torch", "triton"}`` (src/core/transformer.py:71-72); this backend takes the
    ``"triton"`` slot and also answers to ``"b200"``.  Any other value raises: this package ships
    one CUDA implementation and no PyTorch fallback."""
    impl = getattr(config, "attn_impl", "triton")
    if impl in ("triton", "b200"):
        return AttentionB200(config)
    raise ValueError(f"attn_impl={impl!r}: iva_b200 provides the CUDA backend only ('triton' or 'b200')")
