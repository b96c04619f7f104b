"""The allocation-free decode entry point against the regular one.

``ivab_paged_decode_attn_noalloc`` serves callers that cannot hand the library a scratch buffer
(fixed memory budgets, plugins without access to the host's allocator, paths where cudaMalloc's
device-wide synchronisation is not acceptable): its split-K scratch is a fixed array inside the
library.  Both entry points run the same kernels, so their results must agree -- here on two calls
in a row with different inputs, the second of which meets whatever the first left in the shared
array.  This file sorts last so that it runs after every other GPU test.
"""

import ctypes

import pytest
import torch

import iva_b200
from iva_b200 import _lib, workloads
from iva_b200.attention import decode_workspace_bytes
from oracle import paged_ref as ref
from util import assert_attn_close, assert_lse_close

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _call(lib, wl, noalloc):
    """One decode through the raw C ABI; returns (out, lse, status)."""
    B, Hq, D = wl.q.shape
    Hkv = wl.n_kv_heads
    out = torch.full((B, Hq, D), float("nan"), device=DEV, dtype=wl.dtype)
    lse = torch.full((B, Hq), float("nan"), device=DEV, dtype=torch.float32)
    stream = torch.cuda.current_stream().cuda_stream
    lens = wl.ctx_len.contiguous()
    common = (wl.q.data_ptr(), wl.q.stride(0), wl.q.stride(1), wl.k_pool.data_ptr(), wl.v_pool.data_ptr(),
              wl.k_pool.stride(1), wl.page_size * D, wl.block_table.data_ptr(), wl.block_table.stride(0),
              lens.data_ptr(), None, 0, out.data_ptr(), out.stride(0), out.stride(1), lse.data_ptr(),
              _lib.dtype_code(wl.dtype), _lib.dtype_code(wl.dtype),
              B, Hq, Hkv, D, wl.page_size, wl.num_pages, wl.block_table.shape[1], wl.scale)
    if noalloc:
        status = torch.full((1,), -1, dtype=torch.int32, device=DEV)
        rc = lib.ivab_paged_decode_attn_noalloc(*common, status.data_ptr(), stream)
        assert rc == 0, lib.ivab_last_error()
        torch.cuda.synchronize()
        return out, lse, int(status.item())
    ws = torch.empty(decode_workspace_bytes(B, Hq, Hkv, D), dtype=torch.uint8, device=DEV)
    rc = lib.ivab_paged_decode_attn(*common, ws.data_ptr(), ws.numel(), stream)
    assert rc == 0, lib.ivab_last_error()
    st = ctypes.c_int32(-1)
    lib.ivab_decode_status(ws.data_ptr(), ctypes.byref(st), stream)
    return out, lse, st.value


def test_noalloc_matches_regular_entry_point_twice_in_a_row():
    lib = iva_b200.load_library()
    cases = [
        # multi-chunk GQA sequences (split-K partials live in the built-in scratch), bf16
        workloads.make_decode_workload("na1", torch.tensor([6000, 129, 16, 2500, 1]), n_q_heads=16, n_kv_heads=4,
                                       head_dim=128, dtype=torch.bfloat16, seed=21, free_frac=0.2),
        # a different shape and dtype on the second call: fewer, longer chunks, multi-head fp16
        workloads.make_decode_workload("na2", torch.tensor([9000, 40]), n_q_heads=8, n_kv_heads=8,
                                       head_dim=64, dtype=torch.float16, seed=22),
    ]
    for wl in cases:
        d = wl.to(DEV)
        want_out, want_lse, want_st = _call(lib, d, noalloc=False)
        got_out, got_lse, got_st = _call(lib, d, noalloc=True)
        assert want_st == 0 and got_st == 0
        assert torch.isfinite(got_out.float()).all() and torch.isfinite(got_lse).all()
        # same kernels, same deterministic work split, only the scratch lives elsewhere: every bit agrees
        assert torch.equal(got_out, want_out) and torch.equal(got_lse, want_lse)
        # and the result is right, not merely the same: the CPU checker at the parity bar
        # (2e-3 bf16 / 1e-3 fp16 max-abs, 1e-3 on the logsumexp; contexts of 129 keys and more)
        out_ref, lse_ref = ref.paged_decode_ref(wl.q, wl.k_pool, wl.v_pool, wl.block_table, wl.ctx_len, wl.page_size,
                                                wl.scale)
        long_enough = wl.ctx_len >= 100
        assert_attn_close(got_out[long_enough.to(DEV)], out_ref[long_enough], wl.dtype, strict=True)
        assert_attn_close(got_out, out_ref, wl.dtype, strict=False)
        assert_lse_close(got_lse, lse_ref)


def test_noalloc_rejects_problems_beyond_the_built_in_scratch():
    lib = iva_b200.load_library()
    need = decode_workspace_bytes(4096, 64, 64, 128)
    assert need > 8 << 20
    rc = lib.ivab_paged_decode_attn_noalloc(None, 0, 0, None, None, 0, 0, None, 0, None, None, 0, None, 0, 0, None,
                                            _lib.BF16, _lib.BF16, 4096, 64, 64, 128, 16, 1, 1, 0.1, None, None)
    assert rc == _lib.ERR_WORKSPACE
    msg = lib.ivab_last_error().decode()
    assert "built-in buffer" in msg and "ivab_paged_decode_attn" in msg


def test_noalloc_empty_batch_still_defines_the_status_word():
    """A caller that pre-fills its status word and passes an empty batch must read 0, not its own filler."""
    lib = iva_b200.load_library()
    status = torch.full((1,), -1, dtype=torch.int32, device=DEV)
    rc = lib.ivab_paged_decode_attn_noalloc(None, 0, 0, None, None, 0, 0, None, 0, None, None, 0, None, 0, 0, None,
                                            _lib.BF16, _lib.BF16, 0, 8, 2, 128, 16, 1, 1, 0.1, status.data_ptr(),
                                            torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.ivab_last_error()
    torch.cuda.synchronize()
    assert int(status.item()) == 0
