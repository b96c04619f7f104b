"""The CPU checker (oracle/) against outputs of the reference's own code (tests/golden/)."""

import torch

from oracle import paged_ref as ref


def _t(a):
    return torch.from_numpy(a)


def test_gather_matches_reference_kernel(golden, golden_inputs):
    for name, dtype in (("f32", torch.float32), ("f16", torch.float16)):
        cache, gi, _, _ = golden_inputs.kvops_inputs(dtype)
        out = ref.kv_gather_ref(cache, gi)
        assert out.dtype == torch.float32            # reference output is always fp32
        assert torch.equal(out, _t(golden[f"gather_{name}"]))


def test_scatter_matches_reference_kernel(golden, golden_inputs):
    for name, dtype in (("f32", torch.float32), ("f16", torch.float16)):
        cache, _, si, vals = golden_inputs.kvops_inputs(dtype)
        before = cache.clone()
        out = ref.kv_scatter_ref(cache, si, vals)
        assert torch.equal(cache, before)            # input untouched, like the reference's clone
        assert out.dtype == dtype
        assert torch.equal(out.float(), _t(golden[f"scatter_{name}"]))


def test_paged_roundtrip_matches_reference_kernels(golden, golden_inputs):
    page, lens, tables, pool, toks = golden_inputs.roundtrip_inputs()
    for s, L in enumerate(lens):
        slots = ref.slots_for_sequence(tables[s], L, page)
        pool = ref.paged_append_ref(pool, slots, toks[s][0].permute(1, 0, 2))
    assert torch.equal(pool.float(), _t(golden["roundtrip_pool"]))
    bt = torch.full((len(lens), 3), -1, dtype=torch.int32)
    for s, t in enumerate(tables):
        bt[s, :len(t)] = t.to(torch.int32)
    seqs = ref.paged_gather_ref(pool, bt, torch.tensor(lens), page)
    for s, L in enumerate(lens):
        assert torch.equal(seqs[s].float(), _t(golden[f"roundtrip_seq{s}"]))
        assert torch.equal(seqs[s], toks[s])         # append -> gather is the identity


def test_ops_error_behaviour():
    cache = torch.zeros(1, 1, 4, 32)
    idx = torch.tensor([0])
    try:
        ref.kv_ops_ref(cache, idx, None, "scatter")
        raise AssertionError
    except ValueError as e:
        assert "Values tensor required" in str(e)
    try:
        ref.kv_ops_ref(cache, idx, None, "compact")
        raise AssertionError
    except ValueError as e:
        assert "Unknown operation" in str(e)


def test_module_restatement_matches_attention_torch(golden, golden_inputs):
    B, H, hd, L, w, x, ck, cv = golden_inputs.module_inputs()
    y, k_all, v_all = ref.attention_module_ref(x, w[0], w[1], w[2], w[3], H, ck, cv)
    assert torch.allclose(y, _t(golden["module_out"]), atol=1e-6, rtol=1e-6)
    assert torch.equal(k_all, _t(golden["module_new_k"]))
    assert torch.equal(v_all, _t(golden["module_new_v"]))


def test_module_window_restatement_matches_attention_torch(golden, golden_inputs):
    """No cache, 12 tokens, sliding window 5: the reference's own window mask (attention.py:115-129)."""
    B, H, hd, L, w, x, ck, cv = golden_inputs.module_inputs()
    y, _, _ = ref.attention_module_ref(golden_inputs.window_inputs(), w[0], w[1], w[2], w[3], H, sliding_window=5)
    assert torch.allclose(y, _t(golden["module_window_out"]), atol=1e-6, rtol=1e-6)


def test_window_is_a_slice_of_the_keys():
    """ctx_begin in the checker = attention over the keys [begin, L) only."""
    from iva_b200 import workloads

    wl = workloads.make_decode_workload("w", torch.tensor([50, 20]), n_q_heads=4, n_kv_heads=4, head_dim=64,
                                        dtype=torch.float32, seed=9)
    begin = torch.tensor([37, 20])
    out, lse = ref.paged_decode_ref(wl.q, wl.k_pool, wl.v_pool, wl.block_table, wl.ctx_len, 16, ctx_begin=begin)
    slots = ref.slots_for_sequence(wl.block_table[0], 50, 16)[37:]
    k = ref.kv_gather_ref(wl.k_pool, slots)
    v = ref.kv_gather_ref(wl.v_pool, slots)
    o0, l0 = ref.attention_math_ref(wl.q[0].view(1, 4, 1, 64), k, v, wl.scale)
    assert torch.equal(out[0], o0.view(4, 64)) and torch.equal(lse[0], l0.view(4))
    assert not out[1].any() and torch.isinf(lse[1]).all()          # empty window


def test_composed_decode_matches_attention_torch_on_c1(golden, golden_inputs):
    """Config C1 through append -> paged gather -> attention, against AttentionTorch run on the
    reference-gathered cache (identity projections, causal=False)."""
    wl = golden_inputs.c1_module_workload()
    _, _, out, lse = ref.decode_step_ref(wl)
    assert (out - _t(golden["c1_out"])).abs().max().item() <= 1e-6
    assert (lse - _t(golden["c1_lse"])).abs().max().item() <= 1e-5


def test_gqa_equals_mha_with_repeated_heads():
    from iva_b200 import workloads

    wl = workloads.make_decode_workload("t", torch.tensor([40, 7]), n_q_heads=8, n_kv_heads=2, head_dim=64,
                                        dtype=torch.float32, seed=3)
    out, lse = ref.paged_decode_ref(wl.q, wl.k_pool, wl.v_pool, wl.block_table, wl.ctx_len, wl.page_size)
    k2 = wl.k_pool.repeat_interleave(4, dim=1)
    v2 = wl.v_pool.repeat_interleave(4, dim=1)
    out2, lse2 = ref.paged_decode_ref(wl.q, k2, v2, wl.block_table, wl.ctx_len, wl.page_size)
    assert torch.equal(out, out2) and torch.equal(lse, lse2)


def test_kv_cache_restatement():
    c = ref.KVCacheRef(2, 3, 8, 4, "cpu", torch.float32)
    k = torch.randn(2, 3, 3, 8)
    c.update(k, -k, 3)                                # grows to 6
    assert c.seq_len == 6 and torch.equal(c.k[:, :, 3:6], k) and torch.equal(c.v[:, :, 3:6], -k)
    assert torch.equal(c.k[:, :, :3], torch.zeros(2, 3, 3, 8))
    a, b = c.get_slice(3, 5)
    assert torch.equal(a, k[:, :, :2]) and torch.equal(b, -k[:, :, :2])
    c.clear()
    assert not c.k.any() and c.seq_len == 6


def test_padding_masks_match_attention_torch(golden, golden_inputs):
    """The checker's key padding mask against the reference module's own outputs (attention.py:95-97):
    a 12-token input without a cache, and one token on the 7-key cache."""
    B, H, hd, L, w, x, ck, cv = golden_inputs.module_inputs()
    m12, m8 = golden_inputs.padding_masks()
    y, _, _ = ref.attention_module_ref(golden_inputs.window_inputs(), *w, H, attention_mask=m12)
    assert (y - _t(golden["module_padding_out"])).abs().max().item() <= 1e-6
    y, _, _ = ref.attention_module_ref(x, *w, H, ck, cv, attention_mask=m8)
    assert (y - _t(golden["module_padding_cache_out"])).abs().max().item() <= 1e-6


def test_compaction_restatement_packs_rows_in_order():
    cache = torch.arange(2 * 1 * 6 * 2, dtype=torch.float32).view(2, 1, 6, 2)
    mask = torch.tensor([[0, 1, 0, 1, 1, 0], [1, 0, 0, 0, 0, 0]])
    out, counts = ref.kv_compact_ref(cache, mask)
    assert counts.tolist() == [3, 1] and out.shape == (2, 1, 3, 2)
    assert torch.equal(out[0, 0], cache[0, 0, [1, 3, 4]]) and torch.equal(out[1, 0, 0], cache[1, 0, 0])
    assert not out[1, 0, 1:].any()
