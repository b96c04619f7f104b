"""Host-side logic that needs no GPU: workloads, cache bookkeeping, partitioners, argument
errors, and the absence of any CPU fallback."""

import pytest
import torch

import iva_b200
from iva_b200 import workloads
from iva_b200.paged_cache import PagedKVCache, PoolExhausted
from iva_b200.sharding import balance_by_pages, head_slice, shard_requests


def test_c1_workload_shape_and_determinism():
    a, b = workloads.config_c1(), workloads.config_c1()
    assert a.batch == 4 and a.n_q_heads == 16 and a.head_dim == 64 and a.dtype == torch.float32
    assert a.num_pages == 256 and a.k_pool.shape == (1, 16, 4096, 64)
    assert int(a.ctx_len.min()) >= 1 and int(a.ctx_len.max()) <= 512
    assert torch.equal(a.k_pool, b.k_pool) and torch.equal(a.block_table, b.block_table)
    # block tables are non-contiguous slices of one permutation: every page used at most once
    used = a.block_table[a.block_table >= 0]
    assert used.numel() == used.unique().numel()
    # slot mapping points at position ctx_len of each sequence
    for s in range(a.batch):
        L = int(a.ctx_len[s])
        assert int(a.slot_mapping[s]) == int(a.block_table[s, L // 16]) * 16 + L % 16


def test_ragged_lengths_follow_the_config():
    L = workloads.ragged_lengths(128, 0)
    assert L.min() >= 16 and L.max() <= 32768 and 1200 < L.median() < 3500


def test_c3_pool_has_ten_percent_slack():
    wl = workloads.config_c3(batch=8, median=64, hi=256)
    need = int(((wl.ctx_len + 1 + 15) // 16).sum())
    assert wl.num_pages == -(-need * 11 // 10) or abs(wl.num_pages - need * 1.1) < 1.0


def test_append_gather_workload_slots_are_page_runs():
    wl = workloads.config_c4(n_seq=3, chunk=40, max_prior=50)
    assert wl.k_new.shape == (120, 32, 128) and wl.slot_mapping.numel() == 120
    assert wl.slot_mapping.unique().numel() == 120


def test_cache_bookkeeping_without_a_gpu():
    c = PagedKVCache(batch_size=2, n_heads=2, head_dim=32, seq_len=0, device="cpu", dtype=torch.float32,
                     num_pages=6, max_seq_len=64, shuffle_seed=1)
    assert c.free_pages == 6 and c.seq_len == 0
    c._reserve([17, 1])
    assert c.free_pages == 3 and c.lengths == [17, 1] and c.seq_len == 17
    s = c.slots(0, 15, 17)
    assert s[0] // 16 == c._tables[0][0] and s[0] % 16 == 15 and s[1] // 16 == c._tables[0][1] and s[1] % 16 == 0
    with pytest.raises(PoolExhausted):
        c._reserve([64, 64])
    assert c.lengths == [17, 1]            # a failed reservation changes nothing
    c.reset(0)
    assert c.free_pages == 5 and c.lengths == [0, 1]
    with pytest.raises(PoolExhausted):
        c._reserve([65, 1])                # beyond the block table


def test_window_eviction_bookkeeping_without_a_gpu():
    c = PagedKVCache(batch_size=2, n_heads=1, head_dim=16, seq_len=0, device="cpu", dtype=torch.float32,
                     num_pages=12, max_seq_len=96, shuffle_seed=3)
    c._reserve([80, 40])                      # 5 + 3 pages
    assert c.free_pages == 4
    pages0 = list(c._tables[0])
    # window starts at 50 / 20: pages wholly before it go back, page 0 stays for the 4 sink tokens
    freed = c.evict_before([50, 20], keep_sink_tokens=4)
    assert freed == 2 and c.free_pages == 6
    assert c._tables[0][:4] == [pages0[0], -1, -1, pages0[3]] and c._tables[1][0] >= 0
    assert c._bt_host[0, 1].item() == -1 and c._bt_host[0, 2].item() == -1
    assert c.evict_before([50, 20], keep_sink_tokens=4) == 0          # idempotent
    assert c.lengths == [80, 40]                                      # positions keep their numbering
    # a begin beyond the length is clipped to it: the 80 tokens fill pages 0-4 exactly, all of them go
    assert c.evict_before([10 ** 6, 0]) == 3 and c._tables[0] == [-1] * 5
    c._reserve([81, 40])                                              # the next token opens page 5
    assert len(c._tables[0]) == 6 and c._tables[0][5] >= 0 and c.slots(0, 80, 81)[0] == c._tables[0][5] * 16
    with pytest.raises(ValueError):
        c.compact([torch.ones(80), torch.ones(40)])                   # kept tokens on evicted pages


def test_pages_are_conserved_across_evict_reset_and_reserve():
    """Evicted block-table entries are -1; resetting the sequence afterwards must not hand those back
    as page ids (every page is either free or in exactly one table, and no id is negative)."""
    def conserved(c):
        live = [p for t in c._tables for p in t if p >= 0]
        assert all(p >= 0 for p in c._free)
        assert sorted(live + c._free) == list(range(c.num_pages))

    c = PagedKVCache(batch_size=2, n_heads=1, head_dim=16, seq_len=64, device="cpu", dtype=torch.float32,
                     num_pages=16, max_seq_len=128)
    conserved(c)
    assert c.evict_before([48, 48]) == 6
    conserved(c)
    c.reset()                                  # the sequences finish
    conserved(c)
    assert c.free_pages == 16
    c._reserve([90, 30])
    conserved(c)
    assert all(p >= 0 for t in c._tables for p in t)
    c.evict_before([40, 0])
    c.reset(0)                                 # one sequence finishes after an eviction
    conserved(c)
    assert c.lengths == [0, 30]


def test_partitioners():
    assert [len(shard_requests(10, 4, r)) for r in range(4)] == [3, 3, 2, 2]
    assert list(shard_requests(10, 4, 3)) == [8, 9]
    got = sorted(i for r in range(4) for i in shard_requests(10, 4, r))
    assert got == list(range(10))
    with pytest.raises(ValueError):
        shard_requests(4, 2, 2)
    parts = balance_by_pages([1000, 10, 10, 10, 500, 490], 2)
    loads = [sum(-(-[1000, 10, 10, 10, 500, 490][s] // 16) for s in p) for p in parts]
    assert abs(loads[0] - loads[1]) <= 2 and sorted(parts[0] + parts[1]) == list(range(6))
    q, kv = head_slice(32, 8, 4, 1)
    assert (q.start, q.stop, kv.start, kv.stop) == (8, 16, 2, 4)
    with pytest.raises(ValueError):
        head_slice(32, 8, 3, 0)


def test_kv_ops_argument_errors_match_the_reference():
    cache = torch.zeros(1, 1, 4, 32)
    idx = torch.tensor([0])
    with pytest.raises(ValueError, match="Values tensor required for scatter operation"):
        iva_b200.kv_ops(cache, idx, None, "scatter")
    with pytest.raises(ValueError, match="Unknown operation"):
        iva_b200.kv_ops(cache, idx, None, "compact")


def test_no_cpu_fallback():
    """Operators refuse CPU tensors instead of computing the result some other way."""
    cache = torch.zeros(1, 1, 16, 32)
    idx = torch.tensor([0])
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        iva_b200.kv_ops(cache, idx, None, "gather")
    q = torch.zeros(1, 1, 64)
    pool = torch.zeros(1, 1, 16, 64)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        iva_b200.paged_decode_attention(q, pool, pool, torch.zeros(1, 1, dtype=torch.int32),
                                        torch.ones(1, dtype=torch.int32))
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        iva_b200.attention(torch.zeros(1, 1, 1, 64), torch.zeros(1, 1, 4, 64), torch.zeros(1, 1, 4, 64), 0.125)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from iva_b200 import _lib

    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setenv("IVAB_LIBRARY", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no fallback"):
        _lib.load_library()


def test_get_attention_contract():
    from types import SimpleNamespace

    cfg = SimpleNamespace(d_model=64, n_heads=2, dropout=0.0, causal=False, attn_impl="triton")
    m = iva_b200.get_attention(cfg)
    assert isinstance(m, iva_b200.AttentionB200)
    assert sorted(m.state_dict()) == ["k_proj.weight", "o_proj.weight", "q_proj.weight", "v_proj.weight"]
    assert m.q_proj.weight.shape == (64, 64) and m.q_proj.bias is None and abs(m.scale - 32 ** -0.5) < 1e-12
    cfg.attn_impl = "torch"
    with pytest.raises(ValueError):
        iva_b200.get_attention(cfg)
