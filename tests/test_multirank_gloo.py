"""world_size-2 runs on CPU (gloo): the multi-GPU forms of the path must give the single-process
result.  The attention itself is injected (the CPU checker) -- what is under test is the
partitioning, the head slicing and the all-gather."""

import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from iva_b200 import workloads
from iva_b200.sharding import HeadParallelDecoder, shard_requests
from oracle import paged_ref as ref


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_attn(q, k_pool, v_pool, block_table, ctx_len, page_size, scale, return_lse=True):
    return ref.paged_decode_ref(q, k_pool, v_pool, block_table, ctx_len, page_size, scale)


def _head_parallel_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        wl = workloads.make_decode_workload("hp", torch.tensor([300, 45]), n_q_heads=8, n_kv_heads=4, head_dim=64,
                                            dtype=torch.float32, seed=5)
        dec = HeadParallelDecoder(8, 4, attn_fn=_oracle_attn)
        kl, vl = dec.local_pools(wl.k_pool, wl.v_pool)
        assert kl.shape[1] == 4 // world
        out, lse = dec.decode(wl.q, kl, vl, wl.block_table, wl.ctx_len, wl.page_size, wl.scale)
        full_out, full_lse = _oracle_attn(wl.q, wl.k_pool, wl.v_pool, wl.block_table, wl.ctx_len, wl.page_size, wl.scale)
        ret[rank] = bool(torch.equal(out, full_out) and torch.equal(lse, full_lse))
    finally:
        dist.destroy_process_group()


def _request_shard_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n_seq = 6
        mine = shard_requests(n_seq, world, rank)
        wl = workloads.config_c5a(n_seq=n_seq, context=40, rank=rank, world=world)
        assert wl.batch == len(mine)
        _, _, out, _ = ref.decode_step_ref(wl)
        # no collective on the data path; the count exchange below only checks coverage
        counts = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(counts, torch.tensor([wl.batch]))
        ret[rank] = bool(sum(int(c) for c in counts) == n_seq and torch.isfinite(out).all())
    finally:
        dist.destroy_process_group()


def _run(worker, world=2):
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert all(ret.get(r) for r in range(world)), dict(ret)


def test_head_parallel_all_gather_equals_single_rank():
    _run(_head_parallel_worker)


def test_request_sharding_covers_all_sequences():
    _run(_request_shard_worker)


def _lonely_rank(port, ret):
    """Rank 0 of a world of 2 whose peer never starts: the rendezvous must fail with an error after
    its timeout instead of hanging."""
    import datetime

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    try:
        dist.init_process_group("gloo", rank=0, world_size=2, timeout=datetime.timedelta(seconds=3))
        ret["outcome"] = "joined"
        dist.destroy_process_group()
    except Exception as e:                                  # noqa: BLE001 - any rendezvous error is the expected outcome
        ret["outcome"] = "error: " + type(e).__name__


def test_missing_peer_is_an_error_not_a_hang():
    mgr = mp.Manager()
    ret = mgr.dict()
    proc = mp.get_context("spawn").Process(target=_lonely_rank, args=(_free_port(), ret))
    proc.start()
    proc.join(60)
    alive = proc.is_alive()
    if alive:
        proc.kill()
    assert not alive, "rendezvous with a missing peer did not time out"
    assert str(ret.get("outcome", "")).startswith("error"), dict(ret)
