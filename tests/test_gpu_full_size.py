"""GPU checks at the benchmark's full sizes, through size-independent properties plus a sampled
comparison against the CPU checker (a few sequences/heads finish in seconds on the host)."""

import pytest
import torch

import iva_b200
from iva_b200 import workloads
from oracle import paged_ref as ref
from util import assert_attn_close, assert_lse_close, check_decode

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _sampled_oracle(wl_gpu, lens, seqs, out, lse):
    """Oracle on a few sequences: copy only their pages' worth of pool to the host."""
    kp, vp = wl_gpu.k_pool.cpu(), wl_gpu.v_pool.cpu()
    out_ref, lse_ref = ref.paged_decode_ref(wl_gpu.q.cpu(), kp, vp, wl_gpu.block_table.cpu(), lens.cpu(),
                                            wl_gpu.page_size, wl_gpu.scale, seqs=seqs)
    assert_attn_close(out[seqs], out_ref[seqs], wl_gpu.dtype, strict=True)
    assert_lse_close(lse[seqs], lse_ref[seqs])


def test_c2_full_size_step():
    """64 x 32 heads x 4096 context, bf16: append then attention; sampled oracle + invariances."""
    wl = workloads.config_c2(device=DEV)
    pos_before = wl.k_pool[0, :, wl.slot_mapping].clone()
    iva_b200.paged_append(wl.k_pool, wl.v_pool, wl.slot_mapping, wl.k_new, wl.v_new, 16, check=True)
    assert torch.equal(wl.k_pool[0, :, wl.slot_mapping], wl.k_new.permute(1, 0, 2))     # append landed, bit-exact
    assert not torch.equal(pos_before, wl.k_new.permute(1, 0, 2))
    lens = (wl.ctx_len + 1).contiguous()
    out, lse = iva_b200.paged_decode_attention(wl.q, wl.k_pool, wl.v_pool, wl.block_table, lens, 16,
                                               return_lse=True, check=True)
    _sampled_oracle(wl, lens, [0, 37, 63], out, lse)
    # linearity in V: doubling V doubles the output exactly (power of two), lse unchanged
    wl.v_pool.mul_(2)
    out2, lse2 = iva_b200.paged_decode_attention(wl.q, wl.k_pool, wl.v_pool, wl.block_table, lens, 16,
                                                 return_lse=True, check=True)
    assert torch.equal(out2.float(), out.float() * 2) and torch.equal(lse2, lse)
    # run-to-run determinism
    out3 = iva_b200.paged_decode_attention(wl.q, wl.k_pool, wl.v_pool, wl.block_table, lens, 16)
    assert torch.equal(out3, out2)


@pytest.mark.parametrize("seed", [0, 1])
def test_c3_full_size_ragged_gqa(seed):
    """128 ragged sequences (log-normal lengths, 16 .. 32768), 32 query / 8 KV heads.  Checked against
    the checker on every sequence shorter than 64 tokens, the eight shortest, the longest, and eight
    more spread over the length order -- with the fp32 output at the plain 2e-3 bar, so that short
    contexts (outputs of order 1) are not excused by the bf16 rounding of the result."""
    wl = workloads.config_c3(device=DEV, seed=seed)
    iva_b200.paged_append(wl.k_pool, wl.v_pool, wl.slot_mapping, wl.k_new, wl.v_new, 16, check=True)
    lens = (wl.ctx_len + 1).contiguous()
    out, lse = iva_b200.paged_decode_attention(wl.q, wl.k_pool, wl.v_pool, wl.block_table, lens, 16,
                                               return_lse=True, check=True)
    out32, lse32 = iva_b200.paged_decode_attention(wl.q, wl.k_pool, wl.v_pool, wl.block_table, lens, 16,
                                                   return_lse=True, check=True, out_dtype=torch.float32)
    assert torch.equal(out32.to(out.dtype), out) and torch.equal(lse32, lse)
    ctx = wl.ctx_len.cpu()
    order = torch.argsort(ctx)
    n = len(order)
    picks = {int(s) for s in torch.nonzero(ctx < 64).flatten()} | {int(s) for s in order[:8]} | {int(order[-1])}
    picks |= {int(order[i]) for i in range(n // 9, n, n // 9)}
    seqs = sorted(picks)
    assert len(seqs) >= 16
    _sampled_oracle(wl, lens, seqs, out32, lse32)        # fp32 output: the plain bar on every sampled sequence
    order_l = [int(order[n // 2]), int(order[-1])]
    _sampled_oracle(wl, lens, order_l, out, lse)          # bf16 output on the median and the longest
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()


def test_c5a_per_gpu_share_at_eight_gpus():
    """The request-sharded configuration at the size one of eight GPUs gets: 128 sequences x 8192
    tokens, 32 query / 8 KV heads (4.3 GB of K/V); append + attention, sampled checker, bit-reproducible."""
    wl = workloads.config_c5a(device=DEV, n_seq=1024, context=8192, rank=3, world=8)
    assert wl.batch == 128
    iva_b200.paged_append(wl.k_pool, wl.v_pool, wl.slot_mapping, wl.k_new, wl.v_new, 16, check=True)
    assert torch.equal(wl.v_pool[0, :, wl.slot_mapping], wl.v_new.permute(1, 0, 2))
    lens = (wl.ctx_len + 1).contiguous()
    out, lse = iva_b200.paged_decode_attention(wl.q, wl.k_pool, wl.v_pool, wl.block_table, lens, 16,
                                               return_lse=True, check=True)
    _sampled_oracle(wl, lens, [0, 61, 127], out, lse)
    out2 = iva_b200.paged_decode_attention(wl.q, wl.k_pool, wl.v_pool, wl.block_table, lens, 16)
    assert torch.equal(out2, out)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_head_parallel_split_on_one_gpu(world):
    """The head-parallel mode's arithmetic without a second GPU: every rank's KV-head slab (and the query
    heads that follow it) goes through the kernels in turn on this device and the results are
    concatenated.  A head's result may not depend on which other heads share its launch beyond the
    split-K summation order (the chunk size follows the number of KV heads in the call), so the
    concatenation must agree with the unsplit call to fp32 rounding noise, and both must meet the
    checker's bar.  The long sequence is cut into many chunks per slab (the single-131072-token
    configuration scaled to 32768 tokens), the short one into none."""
    from iva_b200.sharding import head_slice

    wl = workloads.make_decode_workload("hp1", torch.tensor([32768, 777]), n_q_heads=32, n_kv_heads=8, head_dim=128,
                                        dtype=torch.bfloat16, seed=12, device=DEV)
    lens = wl.ctx_len.contiguous()
    full, full_lse = iva_b200.paged_decode_attention(wl.q, wl.k_pool, wl.v_pool, wl.block_table, lens, 16,
                                                     return_lse=True, check=True, out_dtype=torch.float32)
    parts, parts_lse = [], []
    for rank in range(world):
        qs, kvs = head_slice(32, 8, world, rank)
        o, l = iva_b200.paged_decode_attention(wl.q[:, qs].contiguous(), wl.k_pool[:, kvs].contiguous(),
                                               wl.v_pool[:, kvs].contiguous(), wl.block_table, lens, 16,
                                               return_lse=True, check=True, out_dtype=torch.float32)
        parts.append(o)
        parts_lse.append(l)
    got, got_lse = torch.cat(parts, 1), torch.cat(parts_lse, 1)
    assert (got - full).abs().max().item() <= 1e-5 and (got_lse - full_lse).abs().max().item() <= 1e-5
    out_ref, lse_ref = ref.paged_decode_ref(wl.q.cpu(), wl.k_pool.cpu(), wl.v_pool.cpu(), wl.block_table.cpu(),
                                            lens.cpu(), 16, wl.scale)
    for o, l in ((full, full_lse), (got, got_lse)):
        assert_attn_close(o, out_ref, wl.dtype, strict=True)
        assert_lse_close(l, lse_ref)


def test_c4_full_size_append_gather_roundtrip():
    """256 sequences x 512-token fp16 chunks after priors U[0,8192]: append, then gather every
    sequence; the chunk must come back bit-exact and the priors must be untouched."""
    wl = workloads.config_c4(device=DEV)
    T, chunk = wl.k_new.shape[0], wl.new_tokens_per_seq
    lens = (wl.ctx_len + chunk).contiguous()
    offs = torch.zeros(wl.batch + 1, dtype=torch.int64, device=DEV)
    offs[1:] = torch.cumsum(lens.long(), 0)
    total = int(offs[-1])
    before = iva_b200.paged_gather(wl.k_pool, wl.block_table, wl.ctx_len, 16, layout="token_major", check=True)
    iva_b200.paged_append(wl.k_pool, wl.v_pool, wl.slot_mapping, wl.k_new, wl.v_new, 16, check=True)
    for pool, new in ((wl.k_pool, wl.k_new), (wl.v_pool, wl.v_new)):
        got = iva_b200.paged_gather(pool, wl.block_table, lens, 16, layout="token_major", out_offsets=offs,
                                    total_tokens=total, check=True)
        pos = torch.arange(total, device=DEV)
        seq_of = torch.bucketize(pos, offs[1:], right=True)
        within = pos - offs[seq_of]
        is_new = within >= wl.ctx_len.long()[seq_of]
        assert int(is_new.sum()) == T
        assert torch.equal(got[is_new], new)                                   # round trip of the chunk
        if pool is wl.k_pool:
            assert torch.equal(got[~is_new], before)                            # priors untouched
        del got
    # the reference-signature operator on the same pool: gather the chunk's slots back
    back = iva_b200.kv_ops(wl.v_pool, wl.slot_mapping[:4096], None, "gather", compat=False, check=True)
    assert torch.equal(back[0].permute(1, 0, 2), wl.v_new[:4096])


def test_c5b_single_131072_token_sequence():
    """One sequence of 131072 tokens, 32 query / 8 KV heads: hundreds of chunks per head, merged by
    logsumexp; compared with the checker on the whole sequence."""
    wl = workloads.config_c5b(device=DEV)
    lens = wl.ctx_len.contiguous()
    out, lse = iva_b200.paged_decode_attention(wl.q, wl.k_pool, wl.v_pool, wl.block_table, lens, 16,
                                               return_lse=True, check=True)
    out_ref, lse_ref = ref.paged_decode_ref(wl.q.cpu(), wl.k_pool.cpu(), wl.v_pool.cpu(), wl.block_table.cpu(),
                                            lens.cpu(), 16, wl.scale)
    assert_attn_close(out, out_ref, wl.dtype, strict=True)
    assert_lse_close(lse, lse_ref)
    # sliding window over the last 4096 keys plus 4 sink keys: 257 pages read instead of 8192
    begin = (lens - 4096).clamp(min=0)
    out_w, lse_w = iva_b200.paged_decode_attention(wl.q, wl.k_pool, wl.v_pool, wl.block_table, lens, 16,
                                                   return_lse=True, check=True, ctx_begin=begin, sink_tokens=4)
    ow_ref, lw_ref = ref.paged_decode_ref(wl.q.cpu(), wl.k_pool.cpu(), wl.v_pool.cpu(), wl.block_table.cpu(), lens.cpu(),
                                          16, wl.scale, ctx_begin=begin.cpu(), sink_tokens=4)
    assert_attn_close(out_w, ow_ref, wl.dtype, strict=True)
    assert_lse_close(lse_w, lw_ref)


def test_batch_larger_than_the_planner_tiles():
    """1500 ragged sequences: more than the planner sorts (1024) and more than one scan tile."""
    g = torch.Generator().manual_seed(5)
    ctx = torch.randint(0, 300, (1500,), generator=g)
    ctx[7] = 4000                                            # one long sequence that gets split
    wl = workloads.make_decode_workload("big", ctx, n_q_heads=8, n_kv_heads=2, head_dim=64, dtype=torch.float16,
                                        seed=6)
    _, _, out_ref, lse_ref = ref.decode_step_ref(wl)
    d = wl.to(DEV)
    iva_b200.paged_append(d.k_pool, d.v_pool, d.slot_mapping, d.k_new, d.v_new, 16, check=True)
    lens = (d.ctx_len + 1).contiguous()
    check_decode(lambda od: iva_b200.paged_decode_attention(d.q, d.k_pool, d.v_pool, d.block_table, lens, 16,
                                                            return_lse=True, check=True, out_dtype=od),
                 out_ref, lse_ref, wl.dtype)


@pytest.mark.parametrize("shape", ["uniform", "ragged"])
def test_large_plan_free_batch(shape):
    """Batches of at most 32 sequences are cut into work items inside the attention kernel; from 256 pages
    per CTA on it compares several chunk sizes.  16 x 4096 tokens x 32 heads (uniform) and 24 ragged
    sequences of up to 12000 tokens reach that search: sampled comparison with the checker, the fused step
    against append + attention, bit-identical repeats."""
    if shape == "uniform":
        wl = workloads.config_c2(device=DEV, batch=16)
    else:
        g = torch.Generator().manual_seed(11)
        ctx = torch.randint(1500, 12000, (24,), generator=g)
        ctx[3], ctx[17] = 5, 0
        wl = workloads.make_decode_workload("ragged24", ctx, n_q_heads=32, n_kv_heads=32, head_dim=128,
                                            dtype=torch.bfloat16, seed=12, device=DEV)
    lens = (wl.ctx_len + 1).contiguous()
    out32, lse = iva_b200.paged_decode_step(wl.q, wl.k_new, wl.v_new, wl.k_pool, wl.v_pool, wl.block_table, lens, 16,
                                            return_lse=True, check=True, out_dtype=torch.float32)
    assert torch.equal(wl.k_pool[0, :, wl.slot_mapping], wl.k_new.permute(1, 0, 2))
    assert torch.equal(wl.v_pool[0, :, wl.slot_mapping], wl.v_new.permute(1, 0, 2))
    order = torch.argsort(wl.ctx_len.cpu())
    seqs = sorted({int(order[0]), int(order[1]), int(order[len(order) // 2]), int(order[-1])})
    _sampled_oracle(wl, lens, seqs, out32, lse)       # fp32 output: the plain bar, also for the short sequences
    # the same workspace again (the first call on it assigns items statically, later ones through the work counter)
    for _ in range(3):
        out2, lse2 = iva_b200.paged_decode_attention(wl.q, wl.k_pool, wl.v_pool, wl.block_table, lens, 16,
                                                     return_lse=True, check=True)
        assert torch.equal(out2, out32.to(out2.dtype)) and torch.equal(lse2, lse)


@pytest.mark.parametrize("config", ["c2", "c3"])
def test_full_size_on_fp8_pools(config):
    """The MHA and the ragged GQA benchmark configurations on 8-bit pools: quantising append, decode,
    sampled comparison against the checker on the dequantised pools; doubling v_scale doubles the
    output exactly; repeated calls are bit-identical."""
    wl = workloads.config_c2(device=DEV) if config == "c2" else workloads.config_c3(device=DEV)
    ks, vs = 0.02, 0.03
    k8, v8 = ref.quantize_fp8_ref(wl.k_pool, ks), ref.quantize_fp8_ref(wl.v_pool, vs)   # same definition, run by torch on the GPU
    wl.k_pool = wl.v_pool = None
    iva_b200.paged_append(k8, v8, wl.slot_mapping, wl.k_new, wl.v_new, 16, check=True, k_scale=ks, v_scale=vs)
    assert torch.equal(k8[0, :, wl.slot_mapping].view(torch.uint8),
                       ref.quantize_fp8_ref(wl.k_new, ks).permute(1, 0, 2).view(torch.uint8))
    lens = (wl.ctx_len + 1).contiguous()
    out, lse = iva_b200.paged_decode_attention(wl.q, k8, v8, wl.block_table, lens, 16, wl.scale, return_lse=True,
                                               check=True, k_scale=ks, v_scale=vs)
    order = torch.argsort(wl.ctx_len.cpu())
    seqs = [int(order[0]), int(order[len(order) // 2]), int(order[-1])]
    out_ref, lse_ref = ref.paged_decode_ref(wl.q.cpu(), ref.dequantize_fp8_ref(k8.cpu(), ks),
                                            ref.dequantize_fp8_ref(v8.cpu(), vs), wl.block_table.cpu(), lens.cpu(), 16,
                                            wl.scale, seqs=seqs)
    assert_attn_close(out[seqs], out_ref[seqs], wl.dtype, strict=True)
    assert_lse_close(lse[seqs], lse_ref[seqs])
    out2, lse2 = iva_b200.paged_decode_attention(wl.q, k8, v8, wl.block_table, lens, 16, wl.scale, return_lse=True,
                                                 k_scale=ks, v_scale=2 * vs)
    assert torch.equal(out2.float(), out.float() * 2) and torch.equal(lse2, lse)
    out3 = iva_b200.paged_decode_attention(wl.q, k8, v8, wl.block_table, lens, 16, wl.scale, k_scale=ks, v_scale=2 * vs)
    assert torch.equal(out3, out2)
