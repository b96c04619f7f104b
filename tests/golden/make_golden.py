"""Generate ``reference_outputs.npz`` by running the reference's own code on CPU.

Run from the repository root, in a container that has the reference checked out:

    python tests/golden/make_golden.py /path/to/reference

What runs is the reference's code, not a restatement:

* ``kv_ops_triton`` (src/kernels_t/kv_ops_triton.py:150-156) under ``TRITON_INTERPRET=1``
  on CPU tensors, for gather, scatter and a paged append -> gather round trip;
* ``AttentionTorch.forward`` (src/core/attention.py:37-110) with ``causal=False`` in eval
  mode.  ``src/core/__init__.py`` cannot be imported (syntax error in rope_kv.py:199-203),
  so ``src.core`` is registered as an empty namespace package and ``src.core.attention`` is
  imported alone.  ``F.softmax`` is wrapped for the duration of the call to record the
  reference's own ``scores`` tensor (attention.py:77), from which the golden logsumexp is
  taken.

Inputs are re-derived from seeds by the tests (``iva_b200.workloads`` and the small
generators below), so only outputs are stored.
"""

from __future__ import annotations

import hashlib
import importlib
import json
import os
import sys
import types

os.environ["TRITON_INTERPRET"] = "1"
sys.dont_write_bytecode = True

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

import iva_b200  # noqa: E402
from iva_b200 import workloads  # noqa: E402


# ---- seeded inputs shared with tests/test_oracle_golden.py ---------------------------------

def kvops_inputs(dtype, seed=11):
    g = torch.Generator().manual_seed(seed)
    cache = torch.randn(2, 3, 48, 32, generator=g).to(dtype)
    gather_idx = torch.randint(0, 48, (20,), generator=g)
    scatter_idx = torch.randperm(48, generator=g)[:20]
    values = torch.randn(2, 3, 20, 32, generator=g).to(dtype)
    return cache, gather_idx, scatter_idx, values


def roundtrip_inputs(seed=12):
    g = torch.Generator().manual_seed(seed)
    page, H, D, n_pages = 16, 4, 64, 8
    lens = [5, 16, 37]
    perm = torch.randperm(n_pages, generator=g)
    tables, off = [], 0
    for L in lens:
        n = (L + page - 1) // page
        tables.append(perm[off:off + n])
        off += n
    pool = torch.randn(1, H, n_pages * page, D, generator=g).to(torch.float16)
    toks = [torch.randn(1, H, L, D, generator=g).to(torch.float16) for L in lens]
    return page, lens, tables, pool, toks


def module_inputs(seed=13):
    g = torch.Generator().manual_seed(seed)
    B, H, hd, L = 2, 4, 32, 7
    dm = H * hd
    w = [torch.randn(dm, dm, generator=g) / dm ** 0.5 for _ in range(4)]
    x = torch.randn(B, 1, dm, generator=g)
    ck = torch.randn(B, H, L, hd, generator=g)
    cv = torch.randn(B, H, L, hd, generator=g)
    return B, H, hd, L, w, x, ck, cv


def window_inputs(seed=14):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(2, 12, 4 * 32, generator=g)


def padding_masks():
    """Key padding masks (attention.py:95-97) for the 12-token input (row 0 padded on the right, row 1 on
    the left) and for the 7-key cache plus one new token (row 0 left, row 1 right)."""
    m12 = torch.ones(2, 12)
    m12[0, 9:] = 0
    m12[1, :3] = 0
    m8 = torch.ones(2, 8)
    m8[0, :2] = 0
    m8[1, 6:] = 0
    return m12, m8


def c1_module_workload():
    """Config C1 with the new token's K and V equal to q: with identity projections the
    reference module appends ``k = v = x`` (attention.py:50-51,62-63)."""
    wl = workloads.config_c1()
    wl.k_new = wl.q.clone()
    wl.v_new = wl.q.clone()
    return wl


class _Cache:
    """Minimal object with the attributes AttentionTorch touches (attention.py:62-73)."""

    def __init__(self, batch_size, n_heads, head_dim, seq_len, device):
        self.batch_size, self.n_heads, self.head_dim, self.seq_len = batch_size, n_heads, head_dim, seq_len
        self.k = self.v = None


def main(ref_root):
    sys.path.insert(0, ref_root)
    from src.kernels_t.kv_ops_triton import kv_ops_triton
    core = types.ModuleType("src.core")
    core.__path__ = [os.path.join(ref_root, "src", "core")]
    sys.modules["src.core"] = core
    att = importlib.import_module("src.core.attention")

    out = {}

    for name, dtype in (("f32", torch.float32), ("f16", torch.float16)):
        cache, gi, si, vals = kvops_inputs(dtype)
        out[f"gather_{name}"] = kv_ops_triton(cache, gi, None, "gather").numpy()
        before = cache.clone()
        res = kv_ops_triton(cache, si, vals, "scatter")
        assert torch.equal(cache, before), "reference scatter must not touch its input"
        out[f"scatter_{name}"] = res.float().numpy()

    page, lens, tables, pool, toks = roundtrip_inputs()
    for s, L in enumerate(lens):
        pos = torch.arange(L)
        slots = tables[s][pos // page] * page + pos % page
        pool = kv_ops_triton(pool, slots, toks[s], "scatter")
    out["roundtrip_pool"] = pool.float().numpy()
    for s, L in enumerate(lens):
        pos = torch.arange(L)
        slots = tables[s][pos // page] * page + pos % page
        out[f"roundtrip_seq{s}"] = kv_ops_triton(pool, slots, None, "gather").numpy()

    captured = []
    real_softmax = att.F.softmax

    def spy(scores, dim=-1, **kw):
        captured.append(scores.detach().clone())
        return real_softmax(scores, dim=dim, **kw)

    B, H, hd, L, w, x, ck, cv = module_inputs()
    cfg = types.SimpleNamespace(d_model=H * hd, n_heads=H, dropout=0.0, causal=False)
    mod = att.AttentionTorch(cfg).eval()
    with torch.no_grad():
        for lin, wt in zip((mod.q_proj, mod.k_proj, mod.v_proj, mod.o_proj), w):
            lin.weight.copy_(wt)
        cache = _Cache(B, H, hd, L, "cpu")
        cache.k, cache.v = ck, cv
        y, new_cache = mod(x, kv_cache=cache)
    out["module_out"] = y.numpy()
    out["module_new_k"] = new_cache.k.numpy()
    out["module_new_v"] = new_cache.v.numpy()
    assert new_cache.seq_len == L + 1

    # the same module without a cache on a 12-token input, sliding window of 5 (attention.py:83-87)
    xw = window_inputs()
    with torch.no_grad():
        yw, none_cache = mod(xw, sliding_window=5)
    assert none_cache is None
    out["module_window_out"] = yw.numpy()

    # key padding masks (attention.py:95-97): the 12-token input alone, and one token on the 7-key cache
    m12, m8 = padding_masks()
    with torch.no_grad():
        yp, _ = mod(xw, attention_mask=m12)
        cache = _Cache(B, H, hd, L, "cpu")
        cache.k, cache.v = ck, cv
        ypc, _ = mod(x, kv_cache=cache, attention_mask=m8)
    out["module_padding_out"] = yp.numpy()
    out["module_padding_cache_out"] = ypc.numpy()

    wl = c1_module_workload()
    Hh, D = wl.n_q_heads, wl.head_dim
    cfg = types.SimpleNamespace(d_model=Hh * D, n_heads=Hh, dropout=0.0, causal=False)
    mod = att.AttentionTorch(cfg).eval()
    eye = torch.eye(Hh * D)
    c1_out, c1_lse = [], []
    att.F.softmax = spy
    try:
        with torch.no_grad():
            for lin in (mod.q_proj, mod.k_proj, mod.v_proj, mod.o_proj):
                lin.weight.copy_(eye)
            for s in range(wl.batch):
                Ls = int(wl.ctx_len[s])
                pos = torch.arange(Ls)
                slots = wl.block_table[s].long()[pos // wl.page_size] * wl.page_size + pos % wl.page_size
                cache = _Cache(1, Hh, D, Ls, "cpu")
                cache.k = kv_ops_triton(wl.k_pool, slots, None, "gather")
                cache.v = kv_ops_triton(wl.v_pool, slots, None, "gather")
                captured.clear()
                y, _ = mod(wl.q[s].reshape(1, 1, Hh * D), kv_cache=cache)
                c1_out.append(y.view(Hh, D))
                c1_lse.append(torch.logsumexp(captured[0], dim=-1).view(Hh))
    finally:
        att.F.softmax = real_softmax
    out["c1_out"] = torch.stack(c1_out).numpy()
    out["c1_lse"] = torch.stack(c1_lse).numpy()

    path = os.path.join(HERE, "reference_outputs.npz")
    np.savez_compressed(path, **out)
    digests = {k: hashlib.sha256(np.ascontiguousarray(v).tobytes()).hexdigest() for k, v in sorted(out.items())}
    meta = {
        "torch": torch.__version__,
        "triton_interpret": True,
        "arrays": {k: {"shape": list(v.shape), "dtype": str(v.dtype), "sha256": digests[k]} for k, v in sorted(out.items())},
    }
    with open(os.path.join(HERE, "reference_outputs.json"), "w") as f:
        json.dump(meta, f, indent=1, sort_keys=True)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <path to the reference checkout>")
    main(sys.argv[1])
