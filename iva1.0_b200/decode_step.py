"""One decode step as a single CUDA-graph replay.

A decode step of one attention layer is one host->device copy of its inputs, the kernel launches of
append and attention, and the result's way back to the host (by default the kernels store it
straight into the pinned output buffer; ``direct_host_output=False`` writes a device buffer and
copies it).  Issued one by one from Python they cost more CPU time than the 64-token append takes on
the GPU, so the step is captured once in a CUDA graph and replayed: one driver call per step.

The caller owns the page pools and the block table (``PagedKVCache`` or its own allocator) and
writes each step's inputs straight into the pinned staging tensors of this object
(``q_host``, ``k_new_host``, ``v_new_host``, ``slot_mapping_host``, ``ctx_len_host``); ``run()``
replays the graph, ``result()`` waits for that step -- on an event recorded behind its last kernel,
not on the whole stream -- and returns the pinned output.

The staging tensors and the outputs exist ``n_buffers`` times (two by default).  The upload of a
step reads the pinned block when the copy EXECUTES, and the kernels write the pinned output when
they execute, so a host that prepares step k+1 while step k is still in flight must write into the
other buffer and read step k's result from the buffer it ran from: ``inputs(b)`` gives buffer ``b``'s
views, ``run(b)`` enqueues it, ``result(b)`` waits for it.  ``run()`` / ``result()`` without an
argument and the ``*_host`` attributes address buffer 0, for a host that takes one step at a time.

``zero_copy_inputs=True`` drops the upload: the kernels read the query, the new tokens and the lengths from the
pinned staging block in place (page-locked host memory is addressable from the device), so those bytes cross the
bus while the attention kernel streams the pools instead of in front of it.

What may overlap is the caller's business: inside one sequence, step k+1's query (and its K/V)
depend on step k's output, so that host has to read ``result()`` before it can fill the next inputs,
and nothing overlaps.  A server that keeps two independent batches in flight (each with its own
pools and its own ``GraphedDecodeStep``) hides one batch's upload and host turn-around under the
other batch's attention.  The reference has no counterpart: its decode loop re-runs the whole
sequence every step (src/core/transformer.py:284-290).
"""

from __future__ import annotations

import math
from types import SimpleNamespace
from typing import List, Optional

import torch

from .attention import decode_workspace_bytes, paged_decode_attention, paged_decode_step
from .kv_ops import _pool_strides, paged_append

__all__ = ["GraphedDecodeStep"]


class GraphedDecodeStep:
    """``append(k_new, v_new) -> attention(q)`` over a page pool, from and to pinned host memory.

    ``block_table`` (int32 ``[B,max_pages]``, on the device) is read in place: update it between
    steps when a sequence gets a new page.  ``ctx_len_host`` holds the lengths INCLUDING the token
    appended in this step; ``slot_mapping_host`` its destination slots.  ``out_dtype=torch.float32``
    returns the kernels' fp32 result instead of rounding it to the tokens' 16-bit type.
    """

    def __init__(self, k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor, n_q_heads: int,
                 page_size: int = 16, scale: Optional[float] = None, return_lse: bool = False,
                 use_graph: bool = True, direct_host_output: bool = True,
                 token_dtype: Optional[torch.dtype] = None, k_scale: float = 1.0, v_scale: float = 1.0,
                 n_buffers: int = 2, out_dtype: Optional[torch.dtype] = None,
                 stream: Optional[torch.cuda.Stream] = None, fused: bool = True, zero_copy_inputs: bool = False):
        if not k_pool.is_cuda:
            raise RuntimeError("GraphedDecodeStep needs CUDA tensors; there is no CPU implementation")
        if n_buffers < 1:
            raise ValueError("n_buffers must be at least 1")
        self.k_pool, self.v_pool, self.block_table = k_pool, v_pool, block_table
        self.page_size = page_size
        dev, dtype = k_pool.device, k_pool.dtype
        # 8-bit (e4m3) pools: queries and new tokens are 16-bit (``token_dtype``, bf16 unless given), the
        # append quantises with ``k_scale`` / ``v_scale`` and the attention reads with the same scales
        self.fp8 = dtype == torch.float8_e4m3fn
        if self.fp8:
            dtype = token_dtype or torch.bfloat16
            if dtype not in (torch.float16, torch.bfloat16):
                raise ValueError("8-bit pools take fp16 or bf16 queries and tokens")
        elif token_dtype is not None and token_dtype != dtype:
            raise ValueError("token_dtype differs from the dtype of the pools")
        out_dtype = out_dtype or dtype
        if out_dtype not in (dtype, torch.float32):
            raise ValueError("out_dtype must be the tokens' dtype or torch.float32")
        self.k_scale, self.v_scale = float(k_scale), float(v_scale)
        Hkv, _, _, _ = _pool_strides(k_pool, page_size)
        D = k_pool.shape[-1]
        B = block_table.shape[0]
        self.scale = scale if scale is not None else 1.0 / math.sqrt(D)

        # All inputs of a step live in ONE pinned block (and one device block), carved into typed
        # views, so that a step uploads them with a single host->device copy.
        esz = torch.empty(0, dtype=dtype).element_size()
        sizes = [B * n_q_heads * D * esz, B * Hkv * D * esz, B * Hkv * D * esz, B * 8, B * 4]
        offs, total = [], 0
        for n in sizes:
            offs.append(total)
            total += (n + 255) // 256 * 256

        def views(block):
            def v(i, dt, *shape):
                return block[offs[i]:offs[i] + sizes[i]].view(dt).view(*shape)
            return (v(0, dtype, B, n_q_heads, D), v(1, dtype, B, Hkv, D), v(2, dtype, B, Hkv, D),
                    v(3, torch.int64, B), v(4, torch.int32, B))

        self._bufs: List[SimpleNamespace] = []
        for _ in range(n_buffers):
            b = SimpleNamespace()
            b.stage_host = torch.zeros(total, dtype=torch.uint8).pin_memory()
            b.stage_dev = torch.empty(total, dtype=torch.uint8, device=dev)
            b.q_host, b.k_new_host, b.v_new_host, b.slot_mapping_host, b.ctx_len_host = views(b.stage_host)
            b.devs = views(b.stage_dev)
            b.out_host = torch.zeros(B, n_q_heads, D, dtype=out_dtype).pin_memory()
            b.lse_host = torch.zeros(B, n_q_heads, dtype=torch.float32).pin_memory() if return_lse else None
            b.out_dev = None if direct_host_output else torch.empty(B, n_q_heads, D, device=dev, dtype=out_dtype)
            b.lse_dev = (torch.empty(B, n_q_heads, device=dev, dtype=torch.float32)
                         if return_lse and not direct_host_output else None)
            b.graph = None
            b.done = torch.cuda.Event()
            b.runs = 0
            self._bufs.append(b)
        b0 = self._bufs[0]
        self.q_host, self.k_new_host, self.v_new_host = b0.q_host, b0.k_new_host, b0.v_new_host
        self.slot_mapping_host, self.ctx_len_host = b0.slot_mapping_host, b0.ctx_len_host
        self.out_host, self.lse_host = b0.out_host, b0.lse_host
        # one scratch for all buffers: their steps run in order on one stream
        self._ws = torch.empty(decode_workspace_bytes(B, n_q_heads, Hkv, D), dtype=torch.uint8, device=dev)
        self.h2d_bytes = total
        self.d2h_bytes = b0.out_host.numel() * b0.out_host.element_size() + (B * n_q_heads * 4 if return_lse else 0)
        # direct_host_output: the kernels store the result straight into the pinned output (pinned
        # host memory is device-accessible under unified addressing) instead of into a device buffer
        # that a device->host copy then drains; the same bytes cross the bus, without the extra pass.
        self.direct_host_output = direct_host_output
        self.stream = stream if stream is not None else torch.cuda.Stream(device=dev)
        self.use_graph = use_graph
        # fused: the new token is written inside the attention launch (paged_decode_step), at the position the
        # block table gives for ctx_len - 1; slot_mapping_host is then not used.  fused=False keeps the separate
        # append through the slot mapping.
        self.fused = fused
        # zero_copy_inputs (fused steps only): no upload at all -- the kernels read q, the new tokens and the lengths
        # from the pinned staging block in place, while they stream the pools, instead of waiting for a
        # host->device copy in front of the step.
        if zero_copy_inputs and not fused:
            raise ValueError("zero_copy_inputs needs the fused step")
        self.zero_copy_inputs = zero_copy_inputs
        self._last = 0

    @property
    def n_buffers(self) -> int:
        return len(self._bufs)

    @property
    def graph(self):
        """The CUDA graph of buffer 0 (``None`` until its second step, or with ``use_graph=False``)."""
        return self._bufs[0].graph

    def inputs(self, buf: int = 0) -> SimpleNamespace:
        """Pinned staging views of buffer ``buf``: ``q_host, k_new_host, v_new_host, slot_mapping_host,
        ctx_len_host`` to fill before ``run(buf)``; ``out_host`` / ``lse_host`` to read after ``result(buf)``."""
        return self._bufs[buf]

    def _enqueue(self, b: SimpleNamespace) -> None:
        if self.zero_copy_inputs:
            q, k_new, v_new, slots, lens = b.q_host, b.k_new_host, b.v_new_host, b.slot_mapping_host, b.ctx_len_host
        else:
            b.stage_dev.copy_(b.stage_host, non_blocking=True)
            q, k_new, v_new, slots, lens = b.devs
        scales = dict(k_scale=self.k_scale, v_scale=self.v_scale) if self.fp8 else {}
        out, lse = (b.out_host, b.lse_host) if self.direct_host_output else (b.out_dev, b.lse_dev)
        if self.fused:
            paged_decode_step(q, k_new, v_new, self.k_pool, self.v_pool, self.block_table, lens, self.page_size,
                              self.scale, out=out, lse=lse, workspace=self._ws, **scales)
        else:
            paged_append(self.k_pool, self.v_pool, slots, k_new, v_new, self.page_size, **scales)
            paged_decode_attention(q, self.k_pool, self.v_pool, self.block_table, lens, self.page_size, self.scale,
                                   out=out, lse=lse, workspace=self._ws, **scales)
        if self.direct_host_output:
            return
        b.out_host.copy_(b.out_dev, non_blocking=True)
        if b.lse_dev is not None:
            b.lse_host.copy_(b.lse_dev, non_blocking=True)

    def run(self, buf: int = 0) -> None:
        """Enqueue one step from buffer ``buf`` (asynchronous).  A buffer's first step runs eagerly,
        which performs every one-time set-up (kernel attributes, status words) outside a capture;
        its second call records the graph; from then on a step is one graph launch."""
        b = self._bufs[buf]
        with torch.cuda.stream(self.stream):
            if not self.use_graph or b.runs == 0:
                self._enqueue(b)
            else:
                if b.graph is None:
                    self.stream.synchronize()
                    b.graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(b.graph, stream=self.stream):
                        self._enqueue(b)
                b.graph.replay()
            b.done.record(self.stream)
        b.runs += 1
        self._last = buf

    def result(self, buf: Optional[int] = None) -> torch.Tensor:
        """Wait for the last step enqueued from buffer ``buf`` (default: the buffer of the most recent
        ``run``) and return its pinned output ``[B,H_q,D]``; later steps may still be in flight."""
        b = self._bufs[self._last if buf is None else buf]
        b.done.synchronize()
        return b.out_host
