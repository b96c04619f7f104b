"""One decode step as a single CUDA-graph replay.

A decode step of one attention layer is four small host->device copies, four kernel launches
(append, plan, attention, merge) and the result's way back to the host (by default the kernels
store it straight into the pinned output buffer; ``direct_host_output=False`` writes a device
buffer and copies it).  Issued one by one from Python they
cost more CPU time than the 64-token append takes on the GPU, so the step is captured once in a
CUDA graph and replayed: one driver call per step.

The caller owns the page pools and the block table (``PagedKVCache`` or its own allocator) and
writes each step's inputs straight into the pinned staging tensors of this object
(``q_host``, ``k_new_host``, ``v_new_host``, ``slot_mapping_host``, ``ctx_len_host``); ``run()``
replays the graph, ``result()`` waits for it and returns the pinned output.  The reference has
no counterpart: its decode loop re-runs the whole sequence every step
(src/core/transformer.py:284-290).
"""

from __future__ import annotations

import math
from typing import Optional

import torch

from .attention import decode_workspace_bytes, paged_decode_attention
from .kv_ops import _pool_strides, paged_append

__all__ = ["GraphedDecodeStep"]


class GraphedDecodeStep:
    """``append(k_new, v_new) -> attention(q)`` over a page pool, from and to pinned host memory.

    ``block_table`` (int32 ``[B,max_pages]``, on the device) is read in place: update it between
    steps when a sequence gets a new page.  ``ctx_len_host`` holds the lengths INCLUDING the token
    appended in this step; ``slot_mapping_host`` its destination slots.
    """

    def __init__(self, k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor, n_q_heads: int,
                 page_size: int = 16, scale: Optional[float] = None, return_lse: bool = False,
                 use_graph: bool = True, direct_host_output: bool = True,
                 token_dtype: Optional[torch.dtype] = None, k_scale: float = 1.0, v_scale: float = 1.0):
        if not k_pool.is_cuda:
            raise RuntimeError("GraphedDecodeStep needs CUDA tensors; there is no CPU implementation")
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
        self._stage_host = torch.zeros(total, dtype=torch.uint8).pin_memory()
        self._stage_dev = torch.empty(total, dtype=torch.uint8, device=dev)

        def views(block):
            def v(i, dt, *shape):
                return block[offs[i]:offs[i] + sizes[i]].view(dt).view(*shape)
            return (v(0, dtype, B, n_q_heads, D), v(1, dtype, B, Hkv, D), v(2, dtype, B, Hkv, D),
                    v(3, torch.int64, B), v(4, torch.int32, B))

        self._hosts = views(self._stage_host)
        self._devs = views(self._stage_dev)
        self.q_host, self.k_new_host, self.v_new_host, self.slot_mapping_host, self.ctx_len_host = self._hosts
        self.out_host = torch.zeros(B, n_q_heads, D, dtype=dtype).pin_memory()
        self.lse_host = torch.zeros(B, n_q_heads, dtype=torch.float32).pin_memory() if return_lse else None
        self._out = torch.empty(B, n_q_heads, D, device=dev, dtype=dtype)
        self._lse = torch.empty(B, n_q_heads, device=dev, dtype=torch.float32) if return_lse else None
        self._ws = torch.empty(decode_workspace_bytes(B, n_q_heads, Hkv, D), dtype=torch.uint8, device=dev)
        self.h2d_bytes = total
        self.d2h_bytes = self.out_host.numel() * self.out_host.element_size() + (
            self.lse_host.numel() * 4 if return_lse else 0)
        # direct_host_output: the kernels store the result straight into the pinned output (pinned
        # host memory is device-accessible under unified addressing) instead of into a device buffer
        # that a device->host copy then drains; the same bytes cross the bus, without the extra pass.
        self.direct_host_output = direct_host_output
        self.stream = torch.cuda.Stream(device=dev)
        self.use_graph = use_graph
        self.graph = None
        self._steps = 0

    def _enqueue(self) -> None:
        self._stage_dev.copy_(self._stage_host, non_blocking=True)
        q, k_new, v_new, slots, lens = self._devs
        scales = dict(k_scale=self.k_scale, v_scale=self.v_scale) if self.fp8 else {}
        paged_append(self.k_pool, self.v_pool, slots, k_new, v_new, self.page_size, **scales)
        if self.direct_host_output:
            paged_decode_attention(q, self.k_pool, self.v_pool, self.block_table, lens, self.page_size, self.scale,
                                   out=self.out_host, lse=self.lse_host, workspace=self._ws, **scales)
            return
        paged_decode_attention(q, self.k_pool, self.v_pool, self.block_table, lens, self.page_size, self.scale,
                               out=self._out, lse=self._lse, workspace=self._ws, **scales)
        self.out_host.copy_(self._out, non_blocking=True)
        if self._lse is not None:
            self.lse_host.copy_(self._lse, non_blocking=True)

    def run(self) -> None:
        """Enqueue one step (asynchronous).  The first step runs eagerly, which performs every
        one-time set-up (kernel attributes, status words) outside a capture; the second call
        records the graph; from then on a step is one graph launch."""
        with torch.cuda.stream(self.stream):
            if not self.use_graph or self._steps == 0:
                self._enqueue()
            else:
                if self.graph is None:
                    self.stream.synchronize()
                    self.graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(self.graph, stream=self.stream):
                        self._enqueue()
                self.graph.replay()
        self._steps += 1

    def result(self) -> torch.Tensor:
        """Wait for the last step and return the pinned output ``[B,H_q,D]``."""
        self.stream.synchronize()
        return self.out_host
