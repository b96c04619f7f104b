"""GPU parity: KV append / gather kernels, called through the C ABI, against the CPU checker and the
reference's golden outputs.  Bit-exact."""

import pytest
import torch

import iva_b200
from iva_b200 import workloads
from iva_b200.kv_ops import read_status
from oracle import paged_ref as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_native_library_is_what_runs():
    lib = iva_b200.load_library()
    before = lib.ivab_launch_count()
    cache = torch.randn(1, 2, 32, 64, device=DEV)
    iva_b200.kv_ops(cache, torch.tensor([3, 1], device=DEV))
    assert lib.ivab_launch_count() == before + 1


@pytest.mark.parametrize("name,dtype", [("f32", torch.float32), ("f16", torch.float16)])
def test_gather_scatter_match_reference_golden(golden, golden_inputs, name, dtype):
    cache, gi, si, vals = golden_inputs.kvops_inputs(dtype)
    out = iva_b200.kv_ops(cache.to(DEV), gi.to(DEV), None, "gather")
    assert out.dtype == torch.float32                       # reference quirk kept in compat mode
    assert torch.equal(out.cpu(), torch.from_numpy(golden[f"gather_{name}"]))
    cache_dev = cache.to(DEV)
    res = iva_b200.kv_ops(cache_dev, si.to(DEV), vals.to(DEV), "scatter")
    assert torch.equal(cache_dev.cpu(), cache)              # input untouched in compat mode
    assert torch.equal(res.float().cpu(), torch.from_numpy(golden[f"scatter_{name}"]))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,H,S,D,N", [(1, 1, 16, 32, 1), (2, 3, 48, 32, 20), (4, 16, 512, 64, 128),
                                      (1, 32, 4096, 128, 1000), (3, 5, 77, 96, 33)])
def test_gather_scatter_vs_oracle(dtype, B, H, S, D, N):
    g = torch.Generator().manual_seed(B * 1000 + N)
    cache = torch.randn(B, H, S, D, generator=g).to(dtype)
    idx = torch.randperm(S, generator=g)[:min(N, S)]
    vals = torch.randn(B, H, idx.numel(), D, generator=g).to(dtype)
    got = iva_b200.kv_ops(cache.to(DEV), idx.to(DEV), None, "gather", compat=False, check=True)
    assert got.dtype == dtype and torch.equal(got.cpu(), ref.kv_gather_ref(cache, idx, compat_fp32=False))
    got32 = iva_b200.kv_ops(cache.to(DEV), idx.to(DEV), None, "gather", check=True)
    assert torch.equal(got32.cpu(), ref.kv_gather_ref(cache, idx))
    want = ref.kv_scatter_ref(cache, idx, vals)
    inplace = cache.to(DEV)
    ret = iva_b200.kv_ops(inplace, idx.to(DEV), vals.to(DEV), "scatter", compat=False, check=True)
    assert ret.data_ptr() == inplace.data_ptr() and torch.equal(inplace.cpu(), want)


def test_gather_with_repeated_indices_and_strided_cache():
    g = torch.Generator().manual_seed(1)
    big = torch.randn(2, 4, 40, 128, generator=g).to(torch.bfloat16)
    cache = big[:, :, :, :64]                               # head_dim contiguous, other strides padded
    idx = torch.tensor([5, 5, 0, 39, 5])
    got = iva_b200.kv_ops(cache.to(DEV)[:, :, :, :], idx.to(DEV), None, "gather", compat=False)
    assert torch.equal(got.cpu(), cache.index_select(2, idx))
    strided = big.to(DEV)[:, :, :, :64]
    got = iva_b200.kv_ops(strided, idx.to(DEV), None, "gather", compat=False)
    assert torch.equal(got.cpu(), cache.index_select(2, idx))


def test_empty_inputs():
    cache = torch.randn(2, 2, 16, 32, device=DEV)
    out = iva_b200.kv_ops(cache, torch.zeros(0, dtype=torch.int64, device=DEV))
    assert out.shape == (2, 2, 0, 32)
    res = iva_b200.kv_ops(cache, torch.zeros(0, dtype=torch.int64, device=DEV),
                          torch.zeros(2, 2, 0, 32, device=DEV), "scatter")
    assert torch.equal(res, cache)


def test_out_of_range_index_is_skipped_and_flagged():
    cache = torch.randn(1, 2, 16, 32, device=DEV)
    read_status(DEV)
    idx = torch.tensor([3, 16, -1, 7], device=DEV)
    out = iva_b200.kv_ops(cache, idx, None, "gather", compat=False)
    torch.cuda.synchronize()
    assert torch.equal(out[:, :, 0], cache[:, :, 3]) and torch.equal(out[:, :, 3], cache[:, :, 7])
    assert read_status(DEV) & 8
    with pytest.raises(IndexError):
        iva_b200.kv_ops(cache, idx, None, "gather", check=True)
    assert read_status(DEV) == 0


def test_paged_roundtrip_matches_reference_golden(golden, golden_inputs):
    page, lens, tables, pool, toks = golden_inputs.roundtrip_inputs()
    kp, vp = pool.to(DEV), pool.to(DEV).clone()
    for s, L in enumerate(lens):
        slots = ref.slots_for_sequence(tables[s], L, page)
        new = toks[s][0].permute(1, 0, 2).contiguous()
        iva_b200.paged_append(kp, vp, slots.to(DEV), new.to(DEV), new.to(DEV), page, check=True)
    assert torch.equal(kp.float().cpu(), torch.from_numpy(golden["roundtrip_pool"]))
    assert torch.equal(kp, vp)
    bt = torch.full((len(lens), 3), -1, dtype=torch.int32)
    for s, t in enumerate(tables):
        bt[s, :len(t)] = t.to(torch.int32)
    seqs = iva_b200.paged_gather(kp, bt.to(DEV), torch.tensor(lens, dtype=torch.int32, device=DEV), page,
                                 layout="head_major", check=True)
    for s in range(len(lens)):
        assert torch.equal(seqs[s].float().cpu(), torch.from_numpy(golden[f"roundtrip_seq{s}"]))


@pytest.mark.parametrize("dtype,H,D", [(torch.float16, 32, 128), (torch.bfloat16, 8, 128), (torch.float32, 16, 64),
                                       (torch.float16, 4, 64)])
def test_append_then_gather_vs_oracle(dtype, H, D):
    """A scaled copy of the append/gather stress configuration, including priors of 0 and
    lengths that end on, just before and just after a page boundary."""
    prior = torch.tensor([0, 1, 15, 16, 17, 100, 0, 250])
    wl = workloads.make_append_gather_workload("ag", prior, 37, n_kv_heads=H, head_dim=D, dtype=dtype, seed=7)
    k_want = ref.paged_append_ref(wl.k_pool, wl.slot_mapping, wl.k_new)
    v_want = ref.paged_append_ref(wl.v_pool, wl.slot_mapping, wl.v_new)
    d = wl.to(DEV)
    iva_b200.paged_append(d.k_pool, d.v_pool, d.slot_mapping, d.k_new, d.v_new, wl.page_size, check=True)
    assert torch.equal(d.k_pool.cpu(), k_want) and torch.equal(d.v_pool.cpu(), v_want)
    lens = wl.ctx_len + 37
    want = ref.paged_gather_ref(k_want, wl.block_table, lens, wl.page_size)
    got_h = iva_b200.paged_gather(d.k_pool, d.block_table, lens.to(DEV), wl.page_size, layout="head_major", check=True)
    got_t = iva_b200.paged_gather(d.k_pool, d.block_table, lens.to(DEV), wl.page_size, layout="token_major", check=True)
    off = 0
    for s, w in enumerate(want):
        assert torch.equal(got_h[s].cpu(), w)
        L = w.shape[2]
        assert torch.equal(got_t[off:off + L].cpu(), w[0].permute(1, 0, 2))
        off += L
    # the appended chunk comes back bit-exact
    off = 0
    for s in range(len(prior)):
        L = int(lens[s])
        assert torch.equal(got_t[off + int(prior[s]):off + L].cpu(), wl.k_new[s * 37:(s + 1) * 37])
        off += L


def test_page_major_pool_layout():
    """The same kernels on a [num_pages, H, page, D] pool (page-major)."""
    wl = workloads.make_append_gather_workload("pm", torch.tensor([5, 40]), 20, n_kv_heads=4, head_dim=64,
                                               dtype=torch.float16, seed=9)
    P = wl.num_pages
    to_pm = lambda t: t.view(4, P, 16, 64).permute(1, 0, 2, 3).contiguous()
    kp, vp = to_pm(wl.k_pool[0]).to(DEV), to_pm(wl.v_pool[0]).to(DEV)
    d = wl.to(DEV)
    iva_b200.paged_append(kp, vp, d.slot_mapping, d.k_new, d.v_new, 16, check=True)
    k_want = ref.paged_append_ref(wl.k_pool, wl.slot_mapping, wl.k_new)
    assert torch.equal(kp.cpu(), to_pm(k_want[0]))
    lens = wl.ctx_len + 20
    got = iva_b200.paged_gather(kp, d.block_table, lens.to(DEV), 16, layout="head_major", check=True)
    for s, w in enumerate(ref.paged_gather_ref(k_want, wl.block_table, lens, 16)):
        assert torch.equal(got[s].cpu(), w)


def test_gather_flags_bad_page_and_length():
    wl = workloads.make_append_gather_workload("bad", torch.tensor([20]), 4, n_kv_heads=2, head_dim=64, seed=2).to(DEV)
    read_status(DEV)
    bt = wl.block_table.clone()
    bt[0, 0] = wl.num_pages + 5
    iva_b200.paged_gather(wl.k_pool, bt, torch.tensor([24], dtype=torch.int32, device=DEV), 16)
    torch.cuda.synchronize()
    assert read_status(DEV) & 2
    iva_b200.paged_gather(wl.k_pool, wl.block_table, torch.tensor([24], dtype=torch.int32, device=DEV), 16,
                          out_offsets=torch.tensor([0, 24], device=DEV), total_tokens=24)
    assert read_status(DEV) == 0
    iva_b200.paged_gather(wl.k_pool, wl.block_table, torch.tensor([-3], dtype=torch.int32, device=DEV), 16,
                          out_offsets=torch.tensor([0, 0], device=DEV), total_tokens=0)
    assert read_status(DEV) & 4


def test_kv_compact_keeps_masked_rows_in_order():
    cache = torch.randn(2, 3, 20, 32, device=DEV)
    mask = torch.zeros(2, 20, device=DEV)
    mask[:, [1, 4, 5, 19]] = 1
    out = iva_b200.kv_compact(cache, mask)
    assert torch.equal(out, cache[:, :, [1, 4, 5, 19]].float())


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_kv_compact_with_independent_rows(dtype):
    """The reference signature takes a [B,S] mask whose rows differ (kv_ops_triton.py:159-181): every row's
    survivors are packed in order, shorter rows are zero-filled, the counts come back on request; rows
    that keep everything, nothing, and a sequence longer than one scan tile are all in the batch."""
    from oracle import paged_ref as ref

    g = torch.Generator().manual_seed(7)
    B, H, S, D = 5, 3, 2500, 64
    cache = torch.randn(B, H, S, D, generator=g).to(dtype)
    mask = (torch.rand(B, S, generator=g) < 0.3).float()
    mask[1] = 1
    mask[2] = 0
    mask[3, :2000] = 0
    want, want_counts = ref.kv_compact_ref(cache, mask)
    got, counts = iva_b200.kv_compact(cache.to(DEV), mask.to(DEV), return_counts=True)
    assert got.dtype == torch.float32 and torch.equal(counts.cpu(), want_counts)
    assert torch.equal(got.cpu(), want)
    same_dtype = iva_b200.kv_compact(cache.to(DEV), mask.to(DEV), compat=False)
    assert same_dtype.dtype == dtype and torch.equal(same_dtype.cpu().float(), want)
    empty = iva_b200.kv_compact(cache.to(DEV), torch.zeros(B, S, device=DEV))
    assert empty.shape == (B, H, 0, D)


def test_canary_guards_around_the_pools_stay_intact():
    """Pools, new tokens and outputs are carved out of larger buffers whose surroundings hold a
    sentinel; after append, gather and decode attention every guard byte must be unchanged."""
    wl = workloads.make_decode_workload("canary", torch.tensor([100, 5, 257]), n_q_heads=8, n_kv_heads=2,
                                        head_dim=128, dtype=torch.bfloat16, seed=31)
    guard = 4096

    def guarded(t):
        flat = torch.full((t.numel() + 2 * guard,), 12345.0, dtype=t.dtype, device=DEV)
        flat[guard:guard + t.numel()] = t.reshape(-1).to(DEV)
        return flat, flat[guard:guard + t.numel()].view(t.shape)

    bufs = {}
    views = {}
    for name in ("k_pool", "v_pool", "q", "k_new", "v_new"):
        bufs[name], views[name] = guarded(getattr(wl, name))
    out_buf, out = guarded(torch.zeros(3, 8, 128, dtype=torch.bfloat16))
    d = wl.to(DEV)
    iva_b200.paged_append(views["k_pool"], views["v_pool"], d.slot_mapping, views["k_new"], views["v_new"], 16, check=True)
    lens = (d.ctx_len + 1).contiguous()
    iva_b200.paged_decode_attention(views["q"], views["k_pool"], views["v_pool"], d.block_table, lens, 16, out=out,
                                    check=True)
    g = iva_b200.paged_gather(views["k_pool"], d.block_table, lens, 16, layout="token_major", check=True)
    torch.cuda.synchronize()
    for name, flat in list(bufs.items()) + [("out", out_buf)]:
        assert (flat[:guard] == 12345.0).all() and (flat[-guard:] == 12345.0).all(), f"guard of {name} was overwritten"
    k_ref, _, out_ref, _ = ref.decode_step_ref(wl)
    assert torch.equal(views["k_pool"].cpu(), k_ref)
    assert (out.float().cpu() - out_ref).abs().max().item() <= 2e-3 + 2 ** -8 * out_ref.abs().max().item()
    assert g.shape[0] == int(lens.sum())


def test_cache_compaction_packs_survivors_and_frees_pages():
    torch.manual_seed(5)
    B, H, D = 3, 4, 64
    cache = iva_b200.PagedKVCache(batch_size=B, n_heads=H, head_dim=D, device=DEV, dtype=torch.float16,
                                  max_seq_len=128, num_pages=24, shuffle_seed=7)
    k = torch.randn(B, 100, H, D).to(torch.float16)
    v = torch.randn(B, 100, H, D).to(torch.float16)
    cache.append(k.to(DEV), v.to(DEV))
    free0 = cache.free_pages
    masks = [torch.rand(100) < 0.3, torch.zeros(100, dtype=torch.bool), torch.ones(100, dtype=torch.bool)]
    new_lens = cache.compact(masks)
    assert new_lens == [int(m.sum()) for m in masks] and cache.lengths == new_lens
    assert cache.free_pages == 24 - sum((L + 15) // 16 for L in new_lens) and cache.free_pages > free0
    ks, vs = cache.gather(layout="head_major")
    for s, m in enumerate(masks):
        assert torch.equal(ks[s][0].cpu(), k[s][m].permute(1, 0, 2))         # survivors, in order, bit-exact
        assert torch.equal(vs[s][0].cpu(), v[s][m].permute(1, 0, 2))
    # the compacted cache keeps working: append one token and attend
    cache.append(torch.randn(B, H, D).to(torch.float16).to(DEV), torch.randn(B, H, D).to(torch.float16).to(DEV))
    q = torch.randn(B, H, D).to(torch.float16).to(DEV)
    out = iva_b200.paged_decode_attention(q, cache.k_pool, cache.v_pool, cache.block_table_dev, cache.ctx_len_dev, 16,
                                          check=True)
    assert torch.isfinite(out.float()).all()
