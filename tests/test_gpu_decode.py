"""GPU parity: single-query decode attention through the block table, called through the C ABI,
against the CPU checker, the reference's golden outputs, and itself under re-paging."""

import math
from types import SimpleNamespace

import pytest
import torch

import iva_b200
from iva_b200 import workloads
from iva_b200.attention import decode_status, decode_workspace_bytes
from oracle import paged_ref as ref
from util import assert_attn_close, assert_lse_close, check_decode

pytestmark = pytest.mark.gpu
DEV = "cuda"


def run_step(wl, check=True):
    """append one token per sequence, then attention over ctx_len+1 keys -- all on the GPU."""
    d = wl.to(DEV)
    iva_b200.paged_append(d.k_pool, d.v_pool, d.slot_mapping, d.k_new, d.v_new, wl.page_size, check=check)
    lens = (d.ctx_len + 1).contiguous()
    out, lse = iva_b200.paged_decode_attention(d.q, d.k_pool, d.v_pool, d.block_table, lens, wl.page_size,
                                               wl.scale, return_lse=True, check=check)
    return d, out, lse


def step_and_check(wl, out_ref, lse_ref):
    """run_step, checked with the output in q's type and again with the fp32 output (check_decode)."""
    d = wl.to(DEV)
    iva_b200.paged_append(d.k_pool, d.v_pool, d.slot_mapping, d.k_new, d.v_new, wl.page_size, check=True)
    lens = (d.ctx_len + 1).contiguous()
    out, lse = check_decode(lambda od: iva_b200.paged_decode_attention(
        d.q, d.k_pool, d.v_pool, d.block_table, lens, wl.page_size, wl.scale, return_lse=True, check=True,
        out_dtype=od), out_ref, lse_ref, wl.dtype)
    return d, out, lse


def test_c1_against_reference_golden(golden, golden_inputs):
    """Config C1 exactly as the reference module computed it (fp32)."""
    wl = golden_inputs.c1_module_workload()
    _, out, lse = run_step(wl)
    assert (out.cpu() - torch.from_numpy(golden["c1_out"])).abs().max().item() <= 2e-5
    assert (lse.cpu() - torch.from_numpy(golden["c1_lse"])).abs().max().item() <= 1e-4


def test_c1_against_oracle_bit_exact_pools():
    wl = workloads.config_c1()
    kp, vp, out_ref, lse_ref = ref.decode_step_ref(wl)
    d, out, lse = run_step(wl)
    assert torch.equal(d.k_pool.cpu(), kp) and torch.equal(d.v_pool.cpu(), vp)
    assert_attn_close(out, out_ref, torch.float32)
    assert_lse_close(lse, lse_ref)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("group", [1, 2, 3, 4, 5, 6, 7, 8])
def test_page_boundary_contexts(dtype, D, group):
    """Contexts around every page boundary, plus an empty sequence; stale slots hold NaN."""
    ctx = torch.tensor([0, 1, 14, 15, 16, 17, 31, 32, 33, 47, 48, 127, 128, 129, 255, 300])
    wl = workloads.make_decode_workload("edge", ctx, n_q_heads=2 * group, n_kv_heads=2, head_dim=D, dtype=dtype,
                                        seed=group * 10 + D, free_frac=0.2, poison_unused=True)
    _, _, out_ref, lse_ref = ref.decode_step_ref(wl)
    step_and_check(wl, out_ref, lse_ref)


@pytest.mark.parametrize("dtype,Hq,Hkv,D", [(torch.bfloat16, 32, 2, 128), (torch.float16, 24, 2, 64),
                                            (torch.bfloat16, 64, 1, 128), (torch.float32, 18, 2, 64)])
def test_head_ratios_above_eight(dtype, Hq, Hkv, D):
    """16, 12, 64 (multi-query) and 9 query heads per KV head: served as equal groups of at most 8."""
    ctx = torch.tensor([0, 1, 16, 33, 200, 5000])
    wl = workloads.make_decode_workload("ratio", ctx, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=D, dtype=dtype,
                                        seed=Hq + D, free_frac=0.2, poison_unused=True)
    _, _, out_ref, lse_ref = ref.decode_step_ref(wl)
    step_and_check(wl, out_ref, lse_ref)


def test_empty_sequence_gives_zeros_and_minus_inf():
    wl = workloads.make_decode_workload("z", torch.tensor([5, 0, 9]), n_q_heads=4, n_kv_heads=4, head_dim=128, seed=1)
    d = wl.to(DEV)
    out, lse = iva_b200.paged_decode_attention(d.q, d.k_pool, d.v_pool, d.block_table, d.ctx_len, 16,
                                               return_lse=True, check=True)
    assert not out[1].any() and torch.isinf(lse[1]).all() and (lse[1] < 0).all()
    out_ref, lse_ref = ref.paged_decode_ref(wl.q, wl.k_pool, wl.v_pool, wl.block_table, wl.ctx_len, 16)
    check_decode(lambda od: iva_b200.paged_decode_attention(d.q, d.k_pool, d.v_pool, d.block_table, d.ctx_len, 16,
                                                            return_lse=True, check=True, out_dtype=od),
                 out_ref, lse_ref, wl.dtype)


@pytest.mark.parametrize("dtype,Hq,Hkv", [(torch.bfloat16, 32, 32), (torch.bfloat16, 32, 8), (torch.float16, 16, 4)])
def test_long_contexts_take_the_split_path(dtype, Hq, Hkv):
    """Few long sequences: each is cut into several chunks and merged by logsumexp."""
    ctx = torch.tensor([5000, 9000, 4097, 70])
    wl = workloads.make_decode_workload("long", ctx, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=128, dtype=dtype, seed=4)
    _, _, out_ref, lse_ref = ref.decode_step_ref(wl)
    d, out, lse = run_step(wl)
    assert_attn_close(out, out_ref, dtype, strict=True)
    assert_lse_close(lse, lse_ref)


def test_ragged_gqa_batch_scaled_c3():
    wl = workloads.config_c3(batch=24, median=700, hi=6000, seed=3)
    _, _, out_ref, lse_ref = ref.decode_step_ref(wl)
    _, out, lse = run_step(wl)
    assert_attn_close(out, out_ref, wl.dtype, strict=True)
    assert_lse_close(lse, lse_ref)


def test_mha_uniform_batch_scaled_c2():
    wl = workloads.config_c2(batch=8, context=1024)
    _, _, out_ref, lse_ref = ref.decode_step_ref(wl)
    _, out, lse = run_step(wl)
    assert_attn_close(out, out_ref, wl.dtype, strict=True)
    assert_lse_close(lse, lse_ref)


def test_result_is_independent_of_page_placement():
    """Moving every page somewhere else in the pool (and updating the block table) must not change
    a single bit: the work list, the chunking and the arithmetic do not depend on page ids."""
    wl = workloads.make_decode_workload("perm", torch.tensor([333, 2000, 16]), n_q_heads=8, n_kv_heads=2,
                                        head_dim=128, seed=6, free_frac=0.5)
    d = wl.to(DEV)
    lens = d.ctx_len.contiguous()
    a = iva_b200.paged_decode_attention(d.q, d.k_pool, d.v_pool, d.block_table, lens, 16, check=True)
    P = wl.num_pages
    perm = torch.randperm(P, generator=torch.Generator().manual_seed(1)).to(DEV)
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(P, device=DEV)
    move = lambda pool: pool.view(1, 2, P, 16, 128)[:, :, inv].reshape(1, 2, P * 16, 128).contiguous()
    bt = d.block_table.clone()
    valid = bt >= 0
    bt[valid] = perm[bt[valid].long()].to(torch.int32)
    b = iva_b200.paged_decode_attention(d.q, move(d.k_pool), move(d.v_pool), bt, lens, 16, check=True)
    assert torch.equal(a, b)


def test_page_major_pool_layout():
    wl = workloads.make_decode_workload("pm", torch.tensor([100, 33]), n_q_heads=8, n_kv_heads=4, head_dim=128, seed=8)
    out_ref, lse_ref = ref.paged_decode_ref(wl.q, wl.k_pool, wl.v_pool, wl.block_table, wl.ctx_len, 16)
    P = wl.num_pages
    to_pm = lambda t: t.view(4, P, 16, 128).permute(1, 0, 2, 3).contiguous().to(DEV)
    d = wl.to(DEV)
    kpm, vpm = to_pm(wl.k_pool[0]), to_pm(wl.v_pool[0])
    check_decode(lambda od: iva_b200.paged_decode_attention(d.q, kpm, vpm, d.block_table, d.ctx_len, 16,
                                                            return_lse=True, check=True, out_dtype=od),
                 out_ref, lse_ref, wl.dtype)


def test_bad_page_id_and_length_are_flagged_not_dereferenced():
    wl = workloads.make_decode_workload("bad", torch.tensor([40, 40]), n_q_heads=2, n_kv_heads=2, head_dim=128, seed=2)
    d = wl.to(DEV)
    ws = torch.empty(decode_workspace_bytes(2, 2, 2, 128), dtype=torch.uint8, device=DEV)
    bt = d.block_table.clone()
    bt[1, 1] = 1 << 20
    iva_b200.paged_decode_attention(d.q, d.k_pool, d.v_pool, bt, d.ctx_len, 16, workspace=ws)
    assert decode_status(ws) & 2
    with pytest.raises(iva_b200.IvabError):
        iva_b200.paged_decode_attention(d.q, d.k_pool, d.v_pool, d.block_table,
                                        torch.tensor([40, 10 ** 6], dtype=torch.int32, device=DEV), 16,
                                        workspace=ws, check=True)
    iva_b200.paged_decode_attention(d.q, d.k_pool, d.v_pool, d.block_table, d.ctx_len, 16, workspace=ws, check=True)


@pytest.mark.parametrize("fill", ["zeros", "ones", "random"])
def test_workspace_contents_never_matter(fill):
    """The workspace is scratch the caller does not initialise.  A small batch (cut into work items inside the
    attention kernel) trusts the work counter in it only after one of its own calls has armed it: whatever the
    memory holds before the first call, every call gives the same bits -- also after a large batch (planned
    by the plan kernel) has used the same memory, and after the block of a finished call is scribbled over."""
    g = torch.Generator().manual_seed(21)
    ctx = torch.randint(600, 5000, (6,), generator=g)
    wl = workloads.make_decode_workload("wsfill", ctx, n_q_heads=8, n_kv_heads=2, head_dim=128, seed=22)
    out_ref, lse_ref = ref.paged_decode_ref(wl.q, wl.k_pool, wl.v_pool, wl.block_table, wl.ctx_len, 16)
    d = wl.to(DEV)
    big = workloads.make_decode_workload("wsbig", torch.randint(1, 700, (40,), generator=g), n_q_heads=8, n_kv_heads=2,
                                         head_dim=128, seed=23)
    big_ref = ref.paged_decode_ref(big.q, big.k_pool, big.v_pool, big.block_table, big.ctx_len, 16)
    bd = big.to(DEV)
    n = max(decode_workspace_bytes(6, 8, 2, 128), decode_workspace_bytes(40, 8, 2, 128))
    if fill == "random":
        ws = torch.randint(0, 256, (n,), dtype=torch.uint8, generator=g).to(DEV)
    else:
        ws = torch.full((n,), 0 if fill == "zeros" else 255, dtype=torch.uint8, device=DEV)
    call = lambda: iva_b200.paged_decode_attention(d.q, d.k_pool, d.v_pool, d.block_table, d.ctx_len, 16,
                                                   return_lse=True, check=True, workspace=ws, out_dtype=torch.float32)
    first = call()
    assert_attn_close(first[0], out_ref, wl.dtype, strict=True)
    assert_lse_close(first[1], lse_ref)
    for i in range(4):
        if i == 2:      # a planned batch in between, on the same memory
            ob, lb = iva_b200.paged_decode_attention(bd.q, bd.k_pool, bd.v_pool, bd.block_table, bd.ctx_len, 16,
                                                     return_lse=True, check=True, workspace=ws, out_dtype=torch.float32)
            assert_attn_close(ob, big_ref[0], big.dtype, strict=True)
        if i == 3:      # somebody else used the memory
            ws.fill_(0x5A)
        again = call()
        assert torch.equal(again[0], first[0]) and torch.equal(again[1], first[1])


def test_argument_errors():
    wl = workloads.make_decode_workload("e", torch.tensor([20]), n_q_heads=22, n_kv_heads=2, head_dim=128, seed=2).to(DEV)
    with pytest.raises(ValueError, match="supported: 1 to 8"):      # 11 query heads per KV head: no equal groups of <= 8
        iva_b200.paged_decode_attention(wl.q, wl.k_pool, wl.v_pool, wl.block_table, wl.ctx_len, 16)
    wl = workloads.make_decode_workload("e", torch.tensor([20]), n_q_heads=2, n_kv_heads=2, head_dim=128, seed=2).to(DEV)
    with pytest.raises(ValueError):
        iva_b200.paged_decode_attention(wl.q, wl.k_pool, wl.v_pool, wl.block_table, wl.ctx_len, 16,
                                        workspace=torch.empty(256, dtype=torch.uint8, device=DEV)[3:])
    with pytest.raises(iva_b200.IvabError, match="workspace"):
        iva_b200.paged_decode_attention(wl.q, wl.k_pool, wl.v_pool, wl.block_table, wl.ctx_len, 16,
                                        workspace=torch.empty(512, dtype=torch.uint8, device=DEV))
    with pytest.raises(RuntimeError, match="inference-only"):
        iva_b200.paged_decode_attention(wl.q.float().requires_grad_(), wl.k_pool.float(), wl.v_pool.float(),
                                        wl.block_table, wl.ctx_len, 16)


def test_bounded_wait_gives_up_instead_of_hanging():
    """Failure detection without a fault: a wait on a barrier nothing completes returns after its
    limit, reports IVAB_STATUS_WAIT_TIMEOUT, and the context stays usable."""
    lib = iva_b200.load_library()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    rc = lib.ivab_selftest_bounded_wait(status.data_ptr(), 50_000_000, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 1
    assert float(torch.ones(4, device=DEV).sum()) == 4.0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("L", [1, 16, 50, 256])
def test_attention_operator_on_dense_tensors(dtype, L):
    """attention(q,k,v,scale) with the reference operator's [B,H,S,D] signature, one query row."""
    g = torch.Generator().manual_seed(L)
    B, H, D = 3, 4, 64
    q = torch.randn(B, H, 1, D, generator=g).to(dtype)
    k = torch.randn(B, H, L, D, generator=g).to(dtype)
    v = torch.randn(B, H, L, D, generator=g).to(dtype)
    scale = 1 / math.sqrt(D)
    want, lse_want = ref.attention_math_ref(q, k, v, scale)
    got, lse = check_decode(lambda od: iva_b200.attention(q.to(DEV), k.to(DEV), v.to(DEV), scale, 0.0, False,
                                                          return_lse=True, out_dtype=od), want, lse_want, dtype)
    assert got.shape == (B, H, 1, D) and got.dtype == dtype


def test_attention_operator_multi_query_and_errors():
    g = torch.Generator().manual_seed(0)
    q = torch.randn(2, 4, 5, 64, generator=g)
    k = torch.randn(2, 4, 37, 64, generator=g)
    v = torch.randn(2, 4, 37, 64, generator=g)
    want, _ = ref.attention_math_ref(q, k, v, 0.125)
    got = iva_b200.attention(q.to(DEV), k.to(DEV), v.to(DEV), 0.125, 0.0, False)
    assert_attn_close(got, want, torch.float32)
    with pytest.raises(NotImplementedError):
        iva_b200.attention(q.to(DEV), k.to(DEV), v.to(DEV), 0.125, 0.1, True)
    with pytest.raises(RuntimeError, match="inference-only"):
        iva_b200.attention(q.to(DEV).requires_grad_(), k.to(DEV), v.to(DEV), 0.125)


@pytest.mark.parametrize("dtype,Hq,Hkv,S", [(torch.bfloat16, 8, 8, 8), (torch.bfloat16, 8, 8, 19), (torch.bfloat16, 8, 4, 7),
                                            (torch.float16, 8, 2, 5), (torch.float32, 4, 4, 3), (torch.bfloat16, 12, 4, 6),
                                            (torch.bfloat16, 16, 2, 4)])
def test_queries_that_share_their_keys_are_packed(dtype, Hq, Hkv, S):
    """Several query positions per row that all see the same keys (the reference module's chunk with
    causal=False): up to eight (query, head) rows per KV head go through the kernels as one head group, so the
    keys are read once per group instead of once per query.  Same results as the checker, with and without a
    per-row key limit; the last case (eight heads per KV head) has nothing to pack and takes the old route."""
    g = torch.Generator().manual_seed(100 * S + Hq)
    B, D, L = 3, 128 if dtype != torch.float32 else 64, 333
    q = torch.randn(B, Hq, S, D, generator=g).to(dtype)
    k = torch.randn(B, Hkv, L, D, generator=g).to(dtype)
    v = torch.randn(B, Hkv, L, D, generator=g).to(dtype)
    scale = 1 / math.sqrt(D)
    rep = Hq // Hkv
    kx, vx = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    want, lse_want = ref.attention_math_ref(q, kx, vx, scale)
    check_decode(lambda od: iva_b200.attention(q.to(DEV), k.to(DEV), v.to(DEV), scale, 0.0, False, return_lse=True,
                                               out_dtype=od), want, lse_want, dtype)
    lim = torch.tensor([L, 17, 200], dtype=torch.int32)
    for b in range(B):
        w_b, l_b = ref.attention_math_ref(q[b:b + 1], kx[b:b + 1, :, :int(lim[b])], vx[b:b + 1, :, :int(lim[b])], scale)
        want[b], lse_want[b] = w_b[0], l_b[0]
    check_decode(lambda od: iva_b200.attention(q.to(DEV), k.to(DEV), v.to(DEV), scale, 0.0, False, return_lse=True,
                                               out_dtype=od, ctx_len=lim.to(DEV)), want, lse_want, dtype)


def test_module_matches_attention_torch_golden(golden, golden_inputs):
    """AttentionB200 with the reference module's weights and a dense reference-style cache."""
    B, H, hd, L, w, x, ck, cv = golden_inputs.module_inputs()
    cfg = SimpleNamespace(d_model=H * hd, n_heads=H, dropout=0.0, causal=False, attn_impl="triton")
    mod = iva_b200.get_attention(cfg).to(DEV).eval()
    mod.load_state_dict({"q_proj.weight": w[0], "k_proj.weight": w[1], "v_proj.weight": w[2], "o_proj.weight": w[3]})
    cache = ref.KVCacheRef(B, H, hd, L, DEV, torch.float32)
    cache.k, cache.v = ck.to(DEV), cv.to(DEV)
    y, new_cache = mod(x.to(DEV), kv_cache=cache)
    assert isinstance(new_cache, ref.KVCacheRef) and new_cache.seq_len == L + 1
    assert torch.allclose(new_cache.k.cpu(), torch.from_numpy(golden["module_new_k"]), atol=1e-5)
    assert (y.cpu() - torch.from_numpy(golden["module_out"])).abs().max().item() <= 5e-5


def test_module_with_paged_cache_decodes_like_the_dense_reference():
    """Prefill 19 tokens, then 20 single-token steps through a PagedKVCache with a shuffled pool;
    every step must equal the reference module's math on the dense concatenated cache."""
    torch.manual_seed(0)
    B, H, hd = 3, 4, 64
    dm = H * hd
    cfg = SimpleNamespace(d_model=dm, n_heads=H, dropout=0.0, causal=False, attn_impl="b200")
    mod = iva_b200.AttentionB200(cfg).to(DEV).eval()
    w = [p.detach().cpu() for p in (mod.q_proj.weight, mod.k_proj.weight, mod.v_proj.weight, mod.o_proj.weight)]
    cache = iva_b200.PagedKVCache(batch_size=B, n_heads=H, head_dim=hd, seq_len=0, device=DEV, dtype=torch.float32,
                                  max_seq_len=64, shuffle_seed=3)
    dense_k = dense_v = None
    xs = [torch.randn(B, 19, dm)] + [torch.randn(B, 1, dm) for _ in range(20)]
    for x in xs:
        y, cache2 = mod(x.to(DEV), kv_cache=cache)
        assert cache2 is cache
        y_ref, dense_k, dense_v = ref.attention_module_ref(x, *w, H, dense_k, dense_v)
        assert (y.cpu() - y_ref).abs().max().item() <= 1e-4
    assert cache.seq_len == 39 and cache.lengths == [39] * B
    assert torch.allclose(cache.k.cpu(), dense_k, atol=1e-5) and torch.allclose(cache.v.cpu(), dense_v, atol=1e-5)
    k2, v2 = cache.get_slice(5, 9)
    assert torch.allclose(k2.cpu(), dense_k[:, :, 5:9], atol=1e-5)


@pytest.mark.parametrize("dtype,Hq,Hkv,D", [(torch.bfloat16, 8, 8, 128), (torch.bfloat16, 16, 4, 128),
                                            (torch.float16, 8, 2, 64), (torch.float32, 4, 2, 64)])
def test_sliding_window_begin(dtype, Hq, Hkv, D):
    """ctx_begin: windows starting on and inside pages, a full context, a one-key window and an empty
    one; stale slots (and everything a window hides on its first page) must not leak in."""
    ctx = torch.tensor([300, 300, 300, 47, 47, 16, 5000, 33])
    begin = torch.tensor([0, 256, 261, 46, 47, 15, 4096 - 7, 1])
    wl = workloads.make_decode_workload("win", ctx, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=D, dtype=dtype,
                                        seed=Hq + D, free_frac=0.2, poison_unused=True)
    out_ref, lse_ref = ref.paged_decode_ref(wl.q, wl.k_pool, wl.v_pool, wl.block_table, wl.ctx_len, 16, wl.scale,
                                            ctx_begin=begin)
    d = wl.to(DEV)
    out, lse = check_decode(lambda od: iva_b200.paged_decode_attention(
        d.q, d.k_pool, d.v_pool, d.block_table, d.ctx_len, 16, wl.scale, return_lse=True, check=True,
        ctx_begin=begin.to(DEV), out_dtype=od), out_ref, lse_ref, dtype)
    assert not out[4].any() and torch.isinf(lse[4]).all()


def test_window_never_reads_evicted_pages():
    """After evict_before() the dropped pages are back in the pool (and get overwritten with NaN
    here); a windowed decode must give the same bits as before the eviction."""
    torch.manual_seed(1)
    B, H, D = 2, 4, 128
    cache = iva_b200.PagedKVCache(batch_size=B, n_heads=H, head_dim=D, device=DEV, dtype=torch.bfloat16,
                                  max_seq_len=400, num_pages=60, shuffle_seed=2)
    cache.append(torch.randn(B, 333, H, D).to(torch.bfloat16).to(DEV), torch.randn(B, 333, H, D).to(torch.bfloat16).to(DEV))
    q = torch.randn(B, 8, D).to(torch.bfloat16).to(DEV)
    window = 100
    begin = (cache.ctx_len_dev - window).clamp(min=0)
    before = iva_b200.paged_decode_attention(q, cache.k_pool, cache.v_pool, cache.block_table_dev, cache.ctx_len_dev,
                                             16, ctx_begin=begin, check=True)
    free0 = cache.free_pages
    dropped = [cache._tables[s][:(333 - window) // 16] for s in range(B)]
    freed = cache.evict_before([333 - window] * B)
    assert freed == B * ((333 - window) // 16) and cache.free_pages == free0 + freed
    for pages in dropped:                               # whoever gets those pages next may write anything
        for p in pages:
            cache.k_pool[:, :, p * 16:(p + 1) * 16] = float("nan")
            cache.v_pool[:, :, p * 16:(p + 1) * 16] = float("nan")
    after = iva_b200.paged_decode_attention(q, cache.k_pool, cache.v_pool, cache.block_table_dev, cache.ctx_len_dev,
                                            16, ctx_begin=begin, check=True)
    assert torch.equal(before, after)


def test_module_sliding_window_matches_attention_torch_golden(golden, golden_inputs):
    """AttentionB200 without a cache, 12 tokens, sliding window 5 -- the reference's own mask."""
    B, H, hd, L, w, x, ck, cv = golden_inputs.module_inputs()
    cfg = SimpleNamespace(d_model=H * hd, n_heads=H, dropout=0.0, causal=False, attn_impl="triton")
    mod = iva_b200.get_attention(cfg).to(DEV).eval()
    mod.load_state_dict({"q_proj.weight": w[0], "k_proj.weight": w[1], "v_proj.weight": w[2], "o_proj.weight": w[3]})
    y, cache = mod(golden_inputs.window_inputs().to(DEV), sliding_window=5)
    assert cache is None
    assert (y.cpu() - torch.from_numpy(golden["module_window_out"])).abs().max().item() <= 5e-5


def test_module_padding_masks_match_attention_torch_golden(golden, golden_inputs):
    """AttentionB200 with the reference's key padding mask (attention.py:95-97), against the reference
    module's own outputs: a 12-token input without a cache (row 0 padded right, row 1 left), one token
    on the dense 7-key cache, and the same step on a PagedKVCache.  A mask with a hole is refused."""
    B, H, hd, L, w, x, ck, cv = golden_inputs.module_inputs()
    m12, m8 = golden_inputs.padding_masks()
    cfg = SimpleNamespace(d_model=H * hd, n_heads=H, dropout=0.0, causal=False, attn_impl="triton")
    mod = iva_b200.get_attention(cfg).to(DEV).eval()
    mod.load_state_dict({"q_proj.weight": w[0], "k_proj.weight": w[1], "v_proj.weight": w[2], "o_proj.weight": w[3]})
    y, _ = mod(golden_inputs.window_inputs().to(DEV), attention_mask=m12.to(DEV))
    assert (y.cpu() - torch.from_numpy(golden["module_padding_out"])).abs().max().item() <= 5e-5
    cache = ref.KVCacheRef(B, H, hd, L, DEV, torch.float32)
    cache.k, cache.v = ck.to(DEV), cv.to(DEV)
    y, _ = mod(x.to(DEV), kv_cache=cache, attention_mask=m8.to(DEV))
    assert (y.cpu() - torch.from_numpy(golden["module_padding_cache_out"])).abs().max().item() <= 5e-5
    # the same cache contents in pages: K/V of the 7 cached tokens are what the projections of some
    # prompt would have produced, so they are written straight into the pool
    paged = iva_b200.PagedKVCache(batch_size=B, n_heads=H, head_dim=hd, device=DEV, dtype=torch.float32,
                                  max_seq_len=32, shuffle_seed=9)
    paged.update(ck.to(DEV), cv.to(DEV), 0)
    y, same = mod(x.to(DEV), kv_cache=paged, attention_mask=m8.to(DEV))
    assert same is paged and paged.lengths == [L + 1] * B
    assert (y.cpu() - torch.from_numpy(golden["module_padding_cache_out"])).abs().max().item() <= 5e-5
    holes = m8.clone()
    holes[0, 4] = 0
    with pytest.raises(NotImplementedError, match="contiguous"):
        mod(x.to(DEV), kv_cache=cache, attention_mask=holes.to(DEV))


@pytest.mark.parametrize("dtype,Hq,Hkv,D", [(torch.bfloat16, 8, 8, 128), (torch.bfloat16, 16, 4, 128), (torch.float32, 4, 2, 64)])
@pytest.mark.parametrize("sink", [1, 4, 16, 20, 40])
def test_attention_sinks_in_front_of_a_window(dtype, Hq, Hkv, D, sink):
    """Keys [0, sink) + [begin, L): sink and window on different pages, on the same page, touching,
    overlapping (sink >= begin), with an empty window, and without any window."""
    ctx = torch.tensor([300, 300, 47, 47, 30, 5000, 33, 64])
    begin = torch.tensor([256, 261, 10, 47, 30, 4000, 0, 17])
    wl = workloads.make_decode_workload("sink", ctx, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=D, dtype=dtype,
                                        seed=Hq + sink, free_frac=0.2, poison_unused=True)
    out_ref, lse_ref = ref.paged_decode_ref(wl.q, wl.k_pool, wl.v_pool, wl.block_table, wl.ctx_len, 16, wl.scale,
                                            ctx_begin=begin, sink_tokens=sink)
    d = wl.to(DEV)
    # pages that hold neither sink nor window keys are gone: overwrite them with NaN
    kp, vp = d.k_pool.clone(), d.v_pool.clone()
    for s in range(len(ctx)):
        keep = set(range((min(sink, int(begin[s])) + 15) // 16)) | set(range(int(begin[s]) // 16, (int(ctx[s]) + 15) // 16))
        for pidx in range((int(ctx[s]) + 15) // 16):
            if pidx not in keep:
                pg = int(wl.block_table[s, pidx])
                kp[:, :, pg * 16:(pg + 1) * 16] = float("nan")
                vp[:, :, pg * 16:(pg + 1) * 16] = float("nan")
    check_decode(lambda od: iva_b200.paged_decode_attention(
        d.q, kp, vp, d.block_table, d.ctx_len, 16, wl.scale, return_lse=True, check=True, ctx_begin=begin.to(DEV),
        sink_tokens=sink, out_dtype=od), out_ref, lse_ref, dtype)


def test_module_window_with_sinks_on_a_paged_cache():
    """Single-token decode through AttentionB200 with sliding_window and sink_cfg, after the hidden
    pages were evicted (sink pages kept)."""
    torch.manual_seed(2)
    B, H, hd, w, sink = 2, 4, 64, 48, 4
    cfg = SimpleNamespace(d_model=H * hd, n_heads=H, dropout=0.0, causal=False, attn_impl="b200")
    mod = iva_b200.AttentionB200(cfg).to(DEV).eval()
    wts = [p.detach().cpu() for p in (mod.q_proj.weight, mod.k_proj.weight, mod.v_proj.weight, mod.o_proj.weight)]
    cache = iva_b200.PagedKVCache(batch_size=B, n_heads=H, head_dim=hd, device=DEV, dtype=torch.float32,
                                  max_seq_len=256, shuffle_seed=4)
    xs = [torch.randn(B, 150, H * hd)] + [torch.randn(B, 1, H * hd) for _ in range(5)]
    dense_k = dense_v = None
    y, _ = mod(xs[0].to(DEV), kv_cache=cache)
    _, dense_k, dense_v = ref.attention_module_ref(xs[0], *wts, H, None, None)
    for x in xs[1:]:
        L = dense_k.shape[2] + 1
        cache.evict_before([L - w] * B, keep_sink_tokens=sink)
        y, _ = mod(x.to(DEV), kv_cache=cache, sliding_window=w, sink_cfg={"sink_tokens": sink})
        # checker: the module's math on the visible keys only
        q = torch.nn.functional.linear(x, wts[0]).view(B, 1, H, hd).transpose(1, 2)
        kn = torch.nn.functional.linear(x, wts[1]).view(B, 1, H, hd).transpose(1, 2)
        vn = torch.nn.functional.linear(x, wts[2]).view(B, 1, H, hd).transpose(1, 2)
        dense_k, dense_v = torch.cat([dense_k, kn], 2), torch.cat([dense_v, vn], 2)
        vis = list(range(sink)) + list(range(L - w, L))
        o, _ = ref.attention_math_ref(q, dense_k[:, :, vis], dense_v[:, :, vis], hd ** -0.5)
        y_ref = torch.nn.functional.linear(o.transpose(1, 2).reshape(B, 1, H * hd), wts[3])
        assert (y.cpu() - y_ref).abs().max().item() <= 1e-4
    assert cache.free_pages > 0


@pytest.mark.parametrize("dtype,D", [(torch.bfloat16, 128), (torch.float32, 64)])
def test_long_and_short_chunk_lists_merge_in_one_call(dtype, D):
    """One sequence cut into hundreds of chunks beside sequences of a few chunks and of one: the merge
    kernel's CTA-per-slice path, its warp-per-head path and the attention kernel's direct output all
    run in the same call.  Also with an output tensor that is only 2-byte (4-byte) aligned, which
    takes the element-wise store path."""
    ctx = torch.tensor([60000, 3000, 500, 17, 0])
    wl = workloads.make_decode_workload("mixed", ctx, n_q_heads=8, n_kv_heads=2, head_dim=D, dtype=dtype, seed=77,
                                        free_frac=0.05, poison_unused=True)
    _, _, out_ref, lse_ref = ref.decode_step_ref(wl)
    d, out, lse = step_and_check(wl, out_ref, lse_ref)
    B, Hq = 5, 8
    flat = torch.empty(B * Hq * D + 8, device=DEV, dtype=dtype)
    odd = flat[1:1 + B * Hq * D].view(B, Hq, D)
    assert odd.data_ptr() % 8 != 0
    lens = (d.ctx_len + 1).contiguous()
    out2 = iva_b200.paged_decode_attention(d.q, d.k_pool, d.v_pool, d.block_table, lens, 16, wl.scale, out=odd, check=True)
    assert torch.equal(out2, out)


@pytest.mark.parametrize("dtype,Hq,Hkv,D,fp8", [
    (torch.bfloat16, 8, 8, 128, False), (torch.bfloat16, 32, 8, 128, False), (torch.float16, 16, 2, 64, False),
    (torch.float32, 4, 2, 64, False), (torch.bfloat16, 32, 2, 128, False),        # 16 query heads per KV head: two head groups
    (torch.bfloat16, 8, 8, 128, True), (torch.bfloat16, 32, 8, 128, True), (torch.float16, 8, 4, 64, True)])
@pytest.mark.parametrize("batch", [7, 70])
def test_fused_step_equals_append_then_attention(dtype, Hq, Hkv, D, fp8, batch):
    """paged_decode_step (the new token written inside the attention launch) against paged_append followed by
    paged_decode_attention: the pools and the results must agree bit for bit.  New tokens that open a page,
    close one, sit in the middle; sequences cut into several chunks; an empty sequence; batches below and
    above the size that goes through the plan kernel."""
    g = torch.Generator().manual_seed(batch + Hq)
    base = torch.tensor([0, 15, 16, 31, 100, 2500, 7000])
    ctx = base if batch == 7 else torch.cat([base, torch.randint(0, 600, (batch - 7,), generator=g)])
    wl = workloads.make_decode_workload("fused", ctx, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=D, dtype=dtype,
                                        seed=batch + D, free_frac=0.1)
    d = wl.to(DEV)
    kw = {}
    if fp8:
        kw = dict(k_scale=0.02, v_scale=0.03)
        d.k_pool = ref.quantize_fp8_ref(wl.k_pool, 0.02).to(DEV)
        d.v_pool = ref.quantize_fp8_ref(wl.v_pool, 0.03).to(DEV)
    lens = (d.ctx_len + 1).contiguous()
    k2, v2 = d.k_pool.clone(), d.v_pool.clone()
    iva_b200.paged_append(k2, v2, d.slot_mapping, d.k_new, d.v_new, 16, check=True, **kw)
    want, want_lse = iva_b200.paged_decode_attention(d.q, k2, v2, d.block_table, lens, 16, wl.scale, return_lse=True,
                                                     check=True, **kw)
    got, got_lse = iva_b200.paged_decode_step(d.q, d.k_new, d.v_new, d.k_pool, d.v_pool, d.block_table, lens, 16, wl.scale,
                                              return_lse=True, check=True, **kw)
    raw = (lambda t: t.view(torch.uint8)) if fp8 else (lambda t: t)
    assert torch.equal(raw(d.k_pool), raw(k2)) and torch.equal(raw(d.v_pool), raw(v2)), "the fused append differs"
    assert torch.equal(got, want) and torch.equal(got_lse, want_lse)
    if not fp8:                                             # and both are right: the checker on a few sequences
        _, _, out_ref, lse_ref = ref.decode_step_ref(wl, seqs=[0, 1, 2, 5])
        assert_attn_close(got[[0, 1, 2, 5]], out_ref[[0, 1, 2, 5]], dtype, strict=False)
        assert_lse_close(got_lse[[0, 1, 2, 5]], lse_ref[[0, 1, 2, 5]])


def test_fused_step_leaves_an_empty_sequence_alone_and_flags_a_bad_page():
    """ctx_len 0 appends nothing; a block-table entry out of range for the new token's page is flagged and
    nothing is written outside the pool."""
    wl = workloads.make_decode_workload("fz", torch.tensor([20, 0, 33]), n_q_heads=4, n_kv_heads=2, head_dim=128, seed=3)
    d = wl.to(DEV)
    lens = torch.tensor([21, 0, 34], dtype=torch.int32, device=DEV)
    before = d.k_pool.clone()
    out, lse = iva_b200.paged_decode_step(d.q, d.k_new, d.v_new, d.k_pool, d.v_pool, d.block_table, lens, 16,
                                          return_lse=True, check=True)
    changed = (d.k_pool != before).any(-1)[0]               # [H, slots]
    assert int(changed.any(0).sum()) == 2                   # exactly the two new tokens' slots
    assert not out[1].any() and torch.isinf(lse[1]).all()
    bt = d.block_table.clone()
    bt[0, 1] = 1 << 20
    ws = torch.empty(decode_workspace_bytes(3, 4, 2, 128), dtype=torch.uint8, device=DEV)
    iva_b200.paged_decode_step(d.q, d.k_new, d.v_new, d.k_pool, d.v_pool, bt, lens, 16, workspace=ws)
    assert decode_status(ws) & 2
