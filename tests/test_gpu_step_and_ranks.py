"""The graphed decode step (public end-to-end call) and the multi-GPU forms on real GPUs."""

import os
import socket
from types import SimpleNamespace

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import iva_b200
from iva_b200 import workloads
from oracle import paged_ref as ref
from util import OUT_TOL, assert_attn_close, assert_lse_close, check_decode

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("use_graph,direct,zero_copy", [(False, False, False), (True, False, False), (True, True, False),
                                                        (True, True, True), (False, True, True)])
def test_graphed_decode_steps_follow_the_dense_reference(use_graph, direct, zero_copy):
    """Six consecutive decode steps from pinned host buffers; every step is checked against the
    CPU checker on the pool it should have produced."""
    cache = iva_b200.PagedKVCache(batch_size=3, n_heads=2, head_dim=128, device=DEV, dtype=torch.bfloat16,
                                  max_seq_len=96, shuffle_seed=5)
    g = torch.Generator().manual_seed(3)
    prompt_k = torch.randn(3, 40, 2, 128, generator=g).to(torch.bfloat16)
    prompt_v = torch.randn(3, 40, 2, 128, generator=g).to(torch.bfloat16)
    cache.append(prompt_k.to(DEV), prompt_v.to(DEV))
    step = iva_b200.GraphedDecodeStep(cache.k_pool, cache.v_pool, cache.block_table_dev, n_q_heads=8,
                                      return_lse=True, use_graph=use_graph, direct_host_output=direct,
                                      zero_copy_inputs=zero_copy)
    k_ref, v_ref = cache.k_pool.cpu(), cache.v_pool.cpu()
    for t in range(6):
        L = 40 + t
        cache._reserve([L + 1] * 3)                        # host bookkeeping: room for one more token
        cache._sync_device()
        q = torch.randn(3, 8, 128, generator=g).to(torch.bfloat16)
        kn = torch.randn(3, 2, 128, generator=g).to(torch.bfloat16)
        vn = torch.randn(3, 2, 128, generator=g).to(torch.bfloat16)
        slots = torch.tensor([cache.slots(s, L, L + 1)[0] for s in range(3)])
        step.q_host.copy_(q); step.k_new_host.copy_(kn); step.v_new_host.copy_(vn)
        step.slot_mapping_host.copy_(slots); step.ctx_len_host.fill_(L + 1)
        step.run()
        out = step.result().clone()
        lse = step.lse_host.clone()
        k_ref = ref.paged_append_ref(k_ref, slots, kn)
        v_ref = ref.paged_append_ref(v_ref, slots, vn)
        out_ref, lse_ref = ref.paged_decode_ref(q, k_ref, v_ref, cache._bt_host, torch.full((3,), L + 1), 16)
        assert_attn_close(out, out_ref, torch.bfloat16, strict=False)
        assert_lse_close(lse, lse_ref)
    assert torch.equal(cache.k_pool.cpu(), k_ref) and torch.equal(cache.v_pool.cpu(), v_ref)
    assert (step.graph is not None) == use_graph


def test_three_layer_decode_loop_carries_one_cache_across_steps_and_layers():
    """A prompt and eight decode steps through three stacked attention layers that share one
    PagedKVCache (one block table, three pools).  Every layer of every step must match the reference
    module's math on that layer's own dense cache."""
    torch.manual_seed(4)
    B, H, hd, L = 2, 4, 64, 3
    dm = H * hd
    cfg = SimpleNamespace(d_model=dm, n_heads=H, dropout=0.0, causal=False, attn_impl="b200")
    layers = [iva_b200.AttentionB200(cfg).to(DEV).eval() for _ in range(L)]
    wts = [[p.detach().cpu() for p in (m.q_proj.weight, m.k_proj.weight, m.v_proj.weight, m.o_proj.weight)] for m in layers]
    cache = iva_b200.PagedKVCache(batch_size=B, n_heads=H, head_dim=hd, device=DEV, dtype=torch.float32,
                                  max_seq_len=64, shuffle_seed=8, n_layers=L)
    dense = [(None, None)] * L
    xs = [torch.randn(B, 21, dm)] + [torch.randn(B, 1, dm) for _ in range(8)]
    for x in xs:
        h_gpu, h_ref = x.to(DEV), x
        for i, m in enumerate(layers):
            y, view = m(h_gpu, kv_cache=cache.layer(i))
            y_ref, dk, dv = ref.attention_module_ref(h_ref, *wts[i], H, *dense[i])
            dense[i] = (dk, dv)
            assert (y.cpu() - y_ref).abs().max().item() <= 2e-4, (i, x.shape)
            h_gpu, h_ref = h_gpu + y, h_ref + y_ref          # residual stream
    assert cache.lengths == [29, 29] and cache._step is None
    for i in range(L):
        assert torch.allclose(cache.layer(i).k.cpu(), dense[i][0], atol=1e-4)
    # one allocator: the three layers use the same pages
    assert cache.free_pages == cache.num_pages - B * 2
    with pytest.raises(RuntimeError, match="appended twice"):
        k = torch.zeros(B, 1, H, hd, device=DEV)
        cache.layer(0).append(k, k)
        cache.layer(0).append(k, k)


def test_decode_loop_function_matches_the_layer_by_layer_checker():
    """``decode_loop``: a 13-token prompt and six autoregressive steps through two layers on one shared
    cache, each step's input built from the previous step's output, against the checker's dense caches."""
    torch.manual_seed(7)
    B, H, hd, L = 2, 2, 64, 2
    dm = H * hd
    cfg = SimpleNamespace(d_model=dm, n_heads=H, dropout=0.0, causal=False, attn_impl="b200")
    layers = [iva_b200.AttentionB200(cfg).to(DEV).eval() for _ in range(L)]
    wts = [[p.detach().cpu() for p in (m.q_proj.weight, m.k_proj.weight, m.v_proj.weight, m.o_proj.weight)] for m in layers]
    cache = iva_b200.PagedKVCache(batch_size=B, n_heads=H, head_dim=hd, device=DEV, dtype=torch.float32,
                                  max_seq_len=48, shuffle_seed=2, n_layers=L)
    prompt = torch.randn(B, 13, dm)

    def next_x(prev, t):                                  # step t+1 is a function of step t's output
        if t == 0:
            return prompt.to(DEV)
        return torch.tanh(prev[:, -1:, :]) if t <= 6 else None

    outs = iva_b200.decode_loop(layers, cache, next_x)
    assert len(outs) == 7 and cache.lengths == [19, 19]
    dense = [(None, None)] * L
    x = prompt
    for t in range(7):
        h = x
        for i in range(L):
            y, dk, dv = ref.attention_module_ref(h, *wts[i], H, *dense[i])
            dense[i] = (dk, dv)
            h = h + y
        assert (outs[t].cpu() - h).abs().max().item() <= 5e-4, t
        x = torch.tanh(h[:, -1:, :])
    with pytest.raises(ValueError, match="layers"):
        iva_b200.decode_loop(layers[:1], cache, [prompt.to(DEV)])


def test_step_buffers_keep_two_steps_apart():
    """Two steps enqueued back to back from the two staging buffers, then read in order: each result is
    the one of its own inputs (the second step sees the first step's appended token), also with fp32 output."""
    g = torch.Generator().manual_seed(11)
    wl = workloads.make_decode_workload("buf", torch.tensor([70, 31, 300]) + 6, n_q_heads=8, n_kv_heads=2, head_dim=128,
                                        dtype=torch.bfloat16, seed=5, free_frac=0.1)
    d = wl.to(DEV)
    ctx = torch.tensor([70, 31, 300])
    step = iva_b200.GraphedDecodeStep(d.k_pool, d.v_pool, d.block_table, n_q_heads=8, return_lse=True,
                                      out_dtype=torch.float32)
    assert step.n_buffers == 2
    k_ref, v_ref = wl.k_pool.clone(), wl.v_pool.clone()
    for rounds in range(3):                                # eager, capture, replay
        feeds = []
        for b in range(2):
            L = ctx + 2 * rounds + b
            q = torch.randn(3, 8, 128, generator=g).to(torch.bfloat16)
            kn = torch.randn(3, 2, 128, generator=g).to(torch.bfloat16)
            vn = torch.randn(3, 2, 128, generator=g).to(torch.bfloat16)
            slots = torch.tensor([int(wl.block_table[s, int(L[s]) // 16]) * 16 + int(L[s]) % 16 for s in range(3)])
            io = step.inputs(b)
            io.q_host.copy_(q); io.k_new_host.copy_(kn); io.v_new_host.copy_(vn)
            io.slot_mapping_host.copy_(slots); io.ctx_len_host.copy_((L + 1).to(torch.int32))
            step.run(b)                                   # both steps are in flight before either is read
            feeds.append((q, kn, vn, slots, L))
        for b, (q, kn, vn, slots, L) in enumerate(feeds):
            out = step.result(b)
            assert out.dtype == torch.float32
            k_ref = ref.paged_append_ref(k_ref, slots, kn)
            v_ref = ref.paged_append_ref(v_ref, slots, vn)
            out_ref, lse_ref = ref.paged_decode_ref(q, k_ref, v_ref, wl.block_table, L + 1, 16)
            assert_attn_close(out, out_ref, torch.bfloat16, strict=True)      # fp32 output: the plain bar
            assert_lse_close(step.inputs(b).lse_host, lse_ref)
    assert step.graph is not None and step.inputs(1).graph is not None


class _SelfExchange:
    """The exchange buffers of a one-rank "group": the library's all-gather with this GPU as its only peer,
    which exercises the kernels (send, poll, slots, step counter) without a second GPU."""

    SLOTS = 2

    def __init__(self, numel):
        import ctypes
        self.numel = numel
        self.block_bytes = (numel * 4 + 15) // 16 * 16
        self.staging_off = self.SLOTS * self.block_bytes
        self.buf = torch.zeros((self.staging_off + self.SLOTS * 2 * self.block_bytes) // 4, dtype=torch.float32, device=DEV)
        self.peers = (ctypes.c_void_p * 1)(self.buf.data_ptr())
        self.epoch = torch.zeros(1, dtype=torch.int32, device=DEV)
        self.status = torch.zeros(1, dtype=torch.int32, device=DEV)

    def exchange_args(self, block):
        return (block.data_ptr(), self.block_bytes, self.peers, 1, 0, self.SLOTS, self.staging_off,
                self.epoch.data_ptr(), self.status.data_ptr(), 1_000_000_000)

    def row(self, step):
        return self.buf.view(torch.uint8)[(step % 2) * self.block_bytes:(step % 2 + 1) * self.block_bytes].view(torch.float32)[:self.numel]


@pytest.mark.parametrize("ctx", [[3000, 70, 1500], [20, 5, 31], [40000], [37 * (i % 9) + 11 * i + 1 for i in range(40)]],
                         ids=["split", "unsplit", "one_long", "planned_batch_of_40"])
def test_step_that_ends_in_the_all_gather(ctx):
    """``ivab_paged_decode_step_allgather``: the rows of a step are written into one block and exchanged by the
    merge kernel's last CTA (or, when no sequence can be split, by the stand-alone exchange kernel).  One rank:
    the result row must be the block, the block must be the plain fp32 result, over four steps (both slots)."""
    wl = workloads.make_decode_workload("xchg", torch.tensor(ctx), n_q_heads=8, n_kv_heads=2, head_dim=128, seed=31).to(DEV)
    B, Hq, D = wl.q.shape
    flat = torch.zeros(B * Hq * (D + 1), dtype=torch.float32, device=DEV)
    out_view, lse_view = flat[:B * Hq * D].view(B, Hq, D), flat[B * Hq * D:].view(B, Hq)
    xch = _SelfExchange(flat.numel())
    lens = (wl.ctx_len + 1).contiguous()
    ref_pools = (wl.k_pool.clone(), wl.v_pool.clone())
    o_ref, l_ref = iva_b200.paged_decode_step(wl.q, wl.k_new, wl.v_new, ref_pools[0], ref_pools[1], wl.block_table, lens, 16,
                                              return_lse=True, out_dtype=torch.float32, check=True)
    for step in range(4):
        flat.zero_()
        if step % 2 == 0:
            iva_b200.paged_decode_step(wl.q, wl.k_new, wl.v_new, wl.k_pool, wl.v_pool, wl.block_table, lens, 16,
                                       out=out_view, lse=lse_view, out_dtype=torch.float32, check=True, exchange=(xch, flat))
        else:       # attention only (the token is in the pool already)
            iva_b200.paged_decode_attention(wl.q, wl.k_pool, wl.v_pool, wl.block_table, lens, 16,
                                            out=out_view, lse=lse_view, out_dtype=torch.float32, check=True, exchange=(xch, flat))
        torch.cuda.synchronize()
        assert int(xch.status.item()) == 0 and int(xch.epoch.item()) == step + 1
        assert torch.equal(out_view, o_ref) and torch.equal(lse_view, l_ref)
        assert torch.equal(xch.row(step), flat)
    assert torch.equal(wl.k_pool, ref_pools[0]) and torch.equal(wl.v_pool, ref_pools[1])


def test_step_that_ends_in_the_all_gather_on_8bit_pools():
    """The same entry point on e4m3 pools (quantising fused append, 8-bit engine), one rank as its own peer."""
    wl = workloads.make_decode_workload("xchg8", torch.tensor([2500, 90]), n_q_heads=8, n_kv_heads=2, head_dim=128, seed=33).to(DEV)
    ks, vs = 0.03, 0.04
    k8, v8 = ref.quantize_fp8_ref(wl.k_pool, ks), ref.quantize_fp8_ref(wl.v_pool, vs)
    k8r, v8r = k8.clone(), v8.clone()
    B, Hq, D = wl.q.shape
    flat = torch.zeros(B * Hq * (D + 1), dtype=torch.float32, device=DEV)
    out_view, lse_view = flat[:B * Hq * D].view(B, Hq, D), flat[B * Hq * D:].view(B, Hq)
    xch = _SelfExchange(flat.numel())
    lens = (wl.ctx_len + 1).contiguous()
    o_ref, l_ref = iva_b200.paged_decode_step(wl.q, wl.k_new, wl.v_new, k8r, v8r, wl.block_table, lens, 16, return_lse=True,
                                              out_dtype=torch.float32, check=True, k_scale=ks, v_scale=vs)
    for step in range(2):
        iva_b200.paged_decode_step(wl.q, wl.k_new, wl.v_new, k8, v8, wl.block_table, lens, 16, out=out_view, lse=lse_view,
                                   out_dtype=torch.float32, check=True, k_scale=ks, v_scale=vs, exchange=(xch, flat))
        torch.cuda.synchronize()
        assert int(xch.status.item()) == 0 and int(xch.epoch.item()) == step + 1
        assert torch.equal(out_view, o_ref) and torch.equal(lse_view, l_ref) and torch.equal(xch.row(step), flat)
    assert torch.equal(k8.view(torch.uint8), k8r.view(torch.uint8)) and torch.equal(v8.view(torch.uint8), v8r.view(torch.uint8))


def test_fp8_cache_object():
    cache = iva_b200.PagedKVCache(batch_size=2, n_heads=2, head_dim=128, device=DEV, dtype=torch.float8_e4m3fn,
                                  max_seq_len=64, k_scale=0.02, v_scale=0.02)
    g = torch.Generator().manual_seed(1)
    k = torch.randn(2, 40, 2, 128, generator=g).to(torch.bfloat16)
    v = torch.randn(2, 40, 2, 128, generator=g).to(torch.bfloat16)
    cache.append(k.to(DEV), v.to(DEV))
    q = torch.randn(2, 4, 128, generator=g).to(torch.bfloat16)
    qd = q.to(DEV)
    kq = ref.dequantize_fp8_ref(ref.quantize_fp8_ref(k, 0.02), 0.02).permute(0, 2, 1, 3)     # [B,H,L,D]
    vq = ref.dequantize_fp8_ref(ref.quantize_fp8_ref(v, 0.02), 0.02).permute(0, 2, 1, 3)
    want, lse_want = ref.attention_math_ref(q.view(2, 2, 2, 1, 128).reshape(2, 4, 1, 128), kq.repeat_interleave(2, 1),
                                            vq.repeat_interleave(2, 1), 128 ** -0.5)
    check_decode(lambda od: iva_b200.paged_decode_attention(qd, cache.k_pool, cache.v_pool, cache.block_table_dev,
                                                            cache.ctx_len_dev, 16, k_scale=0.02, v_scale=0.02, check=True,
                                                            return_lse=True, out_dtype=od),
                 want.view(2, 4, 128), lse_want.view(2, 4), torch.bfloat16)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _nccl_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from iva_b200.sharding import HeadParallelDecoder, shard_requests

        dev = torch.device("cuda", rank)
        # head-parallel: every rank holds the same inputs, keeps its KV-head slab, all-gathers outputs
        wl = workloads.make_decode_workload("hp", torch.tensor([5000, 77]), n_q_heads=16, n_kv_heads=4, head_dim=128,
                                            dtype=torch.bfloat16, seed=11)
        out_ref, lse_ref = ref.paged_decode_ref(wl.q, wl.k_pool, wl.v_pool, wl.block_table, wl.ctx_len, 16)
        d = wl.to(dev)
        dec = HeadParallelDecoder(16, 4)
        kl, vl = dec.local_pools(d.k_pool, d.v_pool)
        out, lse = dec.decode(d.q, kl.contiguous(), vl.contiguous(), d.block_table, d.ctx_len, 16, wl.scale)
        single = iva_b200.paged_decode_attention(d.q, d.k_pool, d.v_pool, d.block_table, d.ctx_len, 16)
        ok = torch.equal(out, single)                                   # same bits as one GPU
        step = dec.capture_local(d.q, kl.contiguous(), vl.contiguous(), d.block_table, d.ctx_len, 16, wl.scale)
        g_out, g_lse = step()                                            # graph replay + one eager all-gather
        torch.cuda.synchronize()
        ok = ok and torch.equal(g_out.to(single.dtype), single) and torch.equal(g_lse, lse)
        err = (out.float().cpu() - out_ref).abs().max().item()
        lerr = (lse.cpu() - lse_ref).abs().max().item()
        # request sharding: each rank decodes its share on its own pool, nothing is exchanged
        mine = shard_requests(6, world, rank)
        wl2 = workloads.config_c5a(n_seq=6, context=300, rank=rank, world=world)
        _, _, o2_ref, _ = ref.decode_step_ref(wl2)
        d2 = wl2.to(dev)
        iva_b200.paged_append(d2.k_pool, d2.v_pool, d2.slot_mapping, d2.k_new, d2.v_new, 16)
        o2 = iva_b200.paged_decode_attention(d2.q, d2.k_pool, d2.v_pool, d2.block_table, (d2.ctx_len + 1).contiguous(), 16)
        err2 = (o2.float().cpu() - o2_ref).abs().max().item()
        ret[rank] = (bool(ok), err, lerr, err2, len(mine) == wl2.batch)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_head_parallel_and_request_sharding():
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_nccl_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    for r in range(2):
        ok, err, lerr, err2, covered = ret[r]
        # contexts of 5000, 77 and 300 keys: the plain bf16 bar, no allowance for the output's rounding
        assert ok and covered and err <= OUT_TOL[torch.bfloat16] and lerr <= 1e-3 and err2 <= OUT_TOL[torch.bfloat16], ret[r]


def _p2p_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from iva_b200.sharding import HeadParallelDecoder, PeerExchange

        dev = torch.device("cuda", rank)
        # the exchange alone: five steps, every rank contributes a block that names rank and step
        xch = PeerExchange(1000, device=dev)
        ok = True
        checks = []
        for t in range(5):
            block = torch.full((1000,), float(100 * t + rank), device=dev)
            rows = xch.gather(block)
            torch.cuda.synchronize()
            want = torch.tensor([100.0 * t + r for r in range(world)], device=dev).view(world, 1).expand(world, 1000)
            checks.append((f"rows of step {t}", bool(torch.equal(rows, want))))
        checks.append(("status", int(xch.status.item()) == 0))
        # head-parallel decode with the outputs reassembled by that kernel instead of NCCL
        wl = workloads.make_decode_workload("hp", torch.tensor([5000, 77]), n_q_heads=16, n_kv_heads=4, head_dim=128,
                                            dtype=torch.bfloat16, seed=11)
        d = wl.to(dev)
        single, single_lse = iva_b200.paged_decode_attention(d.q, d.k_pool, d.v_pool, d.block_table, d.ctx_len, 16,
                                                             return_lse=True)
        dec = HeadParallelDecoder(16, 4, exchange="p2p")
        kl, vl = dec.local_pools(d.k_pool, d.v_pool)
        kl, vl = kl.contiguous(), vl.contiguous()
        out, lse = dec.decode(d.q, kl, vl, d.block_table, d.ctx_len, 16, wl.scale)
        torch.cuda.synchronize()
        checks.append(("eager out", bool(torch.equal(out, single))))
        checks.append(("eager lse", bool(torch.equal(lse, single_lse))))
        step = dec.capture_local(d.q, kl, vl, d.block_table, d.ctx_len, 16, wl.scale)
        for i in range(4):                                   # both slots, twice: the whole step is one graph replay
            g_out, g_lse = step()
            torch.cuda.synchronize()
            checks.append((f"graph replay {i} out", bool(torch.equal(g_out.to(single.dtype), single))))
            checks.append((f"graph replay {i} lse", bool(torch.equal(g_lse, single_lse))))
        prepared = dec.capture_local(d.q, kl, vl, d.block_table, d.ctx_len, 16, wl.scale, graph=False)
        for i in range(3):                                   # the same step launched eagerly (one library call)
            e_out, e_lse = prepared()
            torch.cuda.synchronize()
            checks.append((f"eager step {i} out", bool(torch.equal(e_out.to(single.dtype), single))))
            checks.append((f"eager step {i} lse", bool(torch.equal(e_lse, single_lse))))
        checks.append(("status at the end", int(dec._peer.status.item()) == 0))
        ret[rank] = checks
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_outputs_reassembled_over_peer_memory():
    """The head-parallel mode with this library's own all-gather kernel (plain peer stores over NVLink, arrival
    counters, bounded wait) in place of the NCCL collective: same bits as one GPU, eager and as one CUDA-graph
    replay per step."""
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_p2p_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    for r in range(2):
        assert ret.get(r), dict(ret)
        failed = [name for name, ok in ret[r] if not ok]
        assert not failed, (r, failed)
