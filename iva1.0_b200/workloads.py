"""Seeded synthetic page pools, block tables and decode inputs.

The reference measures its KV operators on ``torch.randn`` tensors only
(src/kernels_t/kv_ops_triton.py:194-196) and ships no dataset for this path, so
every workload here is synthetic: lengths, page permutation and payload all come
from one ``torch.Generator`` seed.  Inputs are generated in fp32, rounded once to
the storage dtype, and the same rounded values are handed to the CUDA kernels and
to the CPU checker.

Layout conventions (shared by the whole package):

* pool          ``[1, H_kv, num_pages * page_size, D]`` -- the reference cache layout
                ``[B, H, S, D]`` (src/kernels_t/kv_ops_triton.py:105) with ``B = 1`` and
                the ``S`` axis read as the flattened slot axis of a page pool;
                ``slot = page_id * page_size + offset``.
* block_table   ``int32 [B, max_pages]``, unused entries ``-1``.
* ctx_len       ``int32 [B]``.
* slot_mapping  ``int64 [T]`` -- the ``indices`` argument of the reference operator.
* q             ``[B, H_q, D]``; new K/V tokens ``[T, H_kv, D]``.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

import torch

__all__ = [
    "PagedWorkload",
    "make_decode_workload",
    "make_append_gather_workload",
    "config_c1",
    "config_c2",
    "config_c3",
    "config_c4",
    "config_c5a",
    "config_c5b",
    "slots_for_range",
]


@dataclass
class PagedWorkload:
    name: str
    dtype: torch.dtype
    page_size: int
    n_q_heads: int
    n_kv_heads: int
    head_dim: int
    num_pages: int
    ctx_len: torch.Tensor          # int32 [B]  tokens already in the cache
    block_table: torch.Tensor      # int32 [B, max_pages]
    k_pool: torch.Tensor           # [1, H_kv, num_pages*page, D]
    v_pool: torch.Tensor
    q: Optional[torch.Tensor]      # [B, H_q, D]
    k_new: torch.Tensor            # [T, H_kv, D]
    v_new: torch.Tensor
    slot_mapping: torch.Tensor     # int64 [T] destination slot of every new token
    new_tokens_per_seq: int = 1
    meta: dict = field(default_factory=dict)

    @property
    def batch(self) -> int:
        return int(self.ctx_len.numel())

    @property
    def scale(self) -> float:
        return 1.0 / math.sqrt(self.head_dim)

    def to(self, device) -> "PagedWorkload":
        kw = {}
        for name, val in self.__dict__.items():
            kw[name] = val.to(device) if isinstance(val, torch.Tensor) else val
        return PagedWorkload(**kw)


def _randn(shape, dtype, gen, device):
    """N(0,1) in fp32 from ``gen``, rounded once to ``dtype``; chunked so a multi-GB
    pool never needs a full fp32 temporary."""
    out = torch.empty(shape, dtype=dtype, device=device)
    flat = out.view(-1)
    step = 1 << 26
    for lo in range(0, flat.numel(), step):
        hi = min(flat.numel(), lo + step)
        flat[lo:hi] = torch.randn(hi - lo, generator=gen, device=device, dtype=torch.float32).to(dtype)
    return out


def slots_for_range(block_row: torch.Tensor, start: int, stop: int, page_size: int) -> torch.Tensor:
    """Slot ids of logical positions ``start..stop-1`` of one sequence."""
    pos = torch.arange(start, stop, dtype=torch.int64, device=block_row.device)
    pages = block_row.to(torch.int64)[pos // page_size]
    return pages * page_size + pos % page_size


def _build(name, ctx_len, *, n_q_heads, n_kv_heads, head_dim, page_size, dtype, seed,
           new_tokens, num_pages, free_frac, device, with_q, poison_unused):
    gen_cpu = torch.Generator(device="cpu").manual_seed(seed + 1)
    ctx_len = ctx_len.to(torch.int64).cpu()
    B = ctx_len.numel()
    need = (ctx_len + new_tokens + page_size - 1) // page_size
    total = int(need.sum())
    if num_pages is None:
        num_pages = int(math.ceil(total * (1.0 + free_frac)))
    if total > num_pages:
        raise ValueError(f"pool of {num_pages} pages cannot hold {total} pages")
    perm = torch.randperm(num_pages, generator=gen_cpu).to(torch.int32)
    max_pages = int(need.max()) if B else 0
    block_table = torch.full((B, max(max_pages, 1)), -1, dtype=torch.int32)
    off = 0
    for s in range(B):
        n = int(need[s])
        block_table[s, :n] = perm[off:off + n]
        off += n
    slot_chunks = [
        slots_for_range(block_table[s], int(ctx_len[s]), int(ctx_len[s]) + new_tokens, page_size)
        for s in range(B)
    ]
    slot_mapping = torch.cat(slot_chunks) if slot_chunks else torch.zeros(0, dtype=torch.int64)

    dev = torch.device(device)
    gen = torch.Generator(device=dev).manual_seed(seed)
    S = num_pages * page_size
    k_pool = _randn((1, n_kv_heads, S, head_dim), dtype, gen, dev)
    v_pool = _randn((1, n_kv_heads, S, head_dim), dtype, gen, dev)
    if poison_unused:
        # Every slot that holds no token gets NaN: a kernel that reads past ctx_len,
        # or multiplies such a slot by a zero weight, shows up as NaN in the output.
        used = torch.zeros(S, dtype=torch.bool)
        for s in range(B):
            L = int(ctx_len[s])
            if L:
                used[slots_for_range(block_table[s], 0, L, page_size)] = True
        k_pool[:, :, ~used.to(dev)] = float("nan")
        v_pool[:, :, ~used.to(dev)] = float("nan")
    T = B * new_tokens
    q = _randn((B, n_q_heads, head_dim), dtype, gen, dev) if with_q else None
    k_new = _randn((T, n_kv_heads, head_dim), dtype, gen, dev)
    v_new = _randn((T, n_kv_heads, head_dim), dtype, gen, dev)
    return PagedWorkload(
        name=name, dtype=dtype, page_size=page_size, n_q_heads=n_q_heads, n_kv_heads=n_kv_heads,
        head_dim=head_dim, num_pages=num_pages, ctx_len=ctx_len.to(torch.int32).to(dev),
        block_table=block_table.to(dev), k_pool=k_pool, v_pool=v_pool, q=q, k_new=k_new, v_new=v_new,
        slot_mapping=slot_mapping.to(dev), new_tokens_per_seq=new_tokens,
        meta={"seed": seed, "total_pages": total},
    )


def make_decode_workload(name, ctx_len, *, n_q_heads, n_kv_heads, head_dim, page_size=16,
                         dtype=torch.bfloat16, seed=0, num_pages=None, free_frac=0.0,
                         device="cpu", poison_unused=False) -> PagedWorkload:
    """One decode step: every sequence appends one token, then attends over its cache."""
    return _build(name, ctx_len, n_q_heads=n_q_heads, n_kv_heads=n_kv_heads, head_dim=head_dim,
                  page_size=page_size, dtype=dtype, seed=seed, new_tokens=1, num_pages=num_pages,
                  free_frac=free_frac, device=device, with_q=True, poison_unused=poison_unused)


def make_append_gather_workload(name, prior_len, chunk, *, n_kv_heads, head_dim, page_size=16,
                                dtype=torch.float16, seed=0, device="cpu") -> PagedWorkload:
    """Every sequence appends a ``chunk``-token block after ``prior_len`` cached tokens."""
    return _build(name, prior_len, n_q_heads=n_kv_heads, n_kv_heads=n_kv_heads, head_dim=head_dim,
                  page_size=page_size, dtype=dtype, seed=seed, new_tokens=chunk, num_pages=None,
                  free_frac=0.0, device=device, with_q=False, poison_unused=False)


# --- the benchmark configurations -------------------------------------------------------------

def config_c1(device="cpu", seed=0) -> PagedWorkload:
    """CPU reference case: batch 4, 16 heads, head_dim 64, fp32, page 16, contexts U[1,512],
    fixed pool of 256 pages."""
    g = torch.Generator().manual_seed(seed)
    ctx = torch.randint(1, 513, (4,), generator=g)
    return make_decode_workload("c1_cpu_reference", ctx, n_q_heads=16, n_kv_heads=16, head_dim=64,
                                dtype=torch.float32, seed=seed, num_pages=256, device=device)


def config_c2(device="cpu", seed=0, batch=64, context=4096) -> PagedWorkload:
    """MHA decode: 32 heads, head_dim 128, bf16, every sequence at the same context."""
    ctx = torch.full((batch,), context, dtype=torch.int64)
    return make_decode_workload("c2_mha_decode", ctx, n_q_heads=32, n_kv_heads=32, head_dim=128,
                                dtype=torch.bfloat16, seed=seed, device=device)


def ragged_lengths(batch, seed, median=2048, sigma=1.0, lo=16, hi=32768) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    z = torch.randn(batch, generator=g, dtype=torch.float64)
    return torch.exp(math.log(median) + sigma * z).round().clamp(lo, hi).to(torch.int64)


def config_c3(device="cpu", seed=0, batch=128, median=2048, hi=32768) -> PagedWorkload:
    """GQA decode, ragged: 32 query / 8 KV heads, log-normal contexts, pool = need + 10 %."""
    ctx = ragged_lengths(batch, seed, median=median, hi=hi)
    return make_decode_workload("c3_gqa_ragged", ctx, n_q_heads=32, n_kv_heads=8, head_dim=128,
                                dtype=torch.bfloat16, seed=seed, free_frac=0.10, device=device)


def config_c4(device="cpu", seed=0, n_seq=256, chunk=512, max_prior=8192) -> PagedWorkload:
    """Append/gather stress: fp16, 32 KV heads, 512-token chunks after priors U[0,8192]."""
    g = torch.Generator().manual_seed(seed)
    prior = torch.randint(0, max_prior + 1, (n_seq,), generator=g)
    return make_append_gather_workload("c4_append_gather", prior, chunk, n_kv_heads=32, head_dim=128,
                                       dtype=torch.float16, seed=seed, device=device)


def config_c5a(device="cpu", seed=0, n_seq=1024, context=8192, rank=0, world=1) -> PagedWorkload:
    """Request-sharded decode: this rank's contiguous share of ``n_seq`` sequences, own pool."""
    per = n_seq // world
    ctx = torch.full((per,), context, dtype=torch.int64)
    return make_decode_workload("c5a_request_sharded", ctx, n_q_heads=32, n_kv_heads=8, head_dim=128,
                                dtype=torch.bfloat16, seed=seed + 1000 * rank, device=device)


def config_c5b(device="cpu", seed=0, context=131072, n_q_heads=32, n_kv_heads=8) -> PagedWorkload:
    """One very long sequence; the head-parallel mode slices KV heads across ranks."""
    ctx = torch.full((1,), context, dtype=torch.int64)
    return make_decode_workload("c5b_head_parallel", ctx, n_q_heads=n_q_heads, n_kv_heads=n_kv_heads,
                                head_dim=128, dtype=torch.bfloat16, seed=seed, device=device)
