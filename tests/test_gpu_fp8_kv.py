"""8-bit (e4m3) KV storage: quantising append is bit-exact against the checker's definition,
decode attention on the stored values meets the 16-bit tolerance against the checker run on the
dequantised pools, and the error of the quantisation itself is bounded."""

import pytest
import torch

import iva_b200
from iva_b200 import workloads
from oracle import paged_ref as ref
from util import assert_attn_close, assert_lse_close, check_decode

pytestmark = pytest.mark.gpu
DEV = "cuda"
F8 = torch.float8_e4m3fn


def _fp8_workload(ctx, Hq, Hkv, D, dtype, seed, k_scale, v_scale, poison=False):
    wl = workloads.make_decode_workload("fp8", ctx, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=D, dtype=dtype, seed=seed,
                                        free_frac=0.2, poison_unused=poison)   # poison: NaN bytes in every unused slot
    k8 = ref.quantize_fp8_ref(wl.k_pool, k_scale)
    v8 = ref.quantize_fp8_ref(wl.v_pool, v_scale)
    return wl, k8, v8


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("D", [64, 128])
def test_quantising_append_is_bit_exact(dtype, D):
    ctx = torch.tensor([0, 15, 16, 100, 257])
    k_scale, v_scale = 0.03125, 0.0123
    wl, k8, v8 = _fp8_workload(ctx, 4, 4, D, dtype, 3, k_scale, v_scale)
    # outliers far beyond the representable range must saturate, not become NaN
    wl.k_new[0, 0, 0] = 1000.0
    wl.v_new[1, 1, 3] = -1000.0
    kd, vd = k8.to(DEV), v8.to(DEV)
    iva_b200.paged_append(kd, vd, wl.slot_mapping.to(DEV), wl.k_new.to(DEV), wl.v_new.to(DEV), 16, check=True,
                          k_scale=k_scale, v_scale=v_scale)
    k_want = k8.clone().view(torch.uint8)
    v_want = v8.clone().view(torch.uint8)
    k_want[0, :, wl.slot_mapping] = ref.quantize_fp8_ref(wl.k_new, k_scale).view(torch.uint8).permute(1, 0, 2)
    v_want[0, :, wl.slot_mapping] = ref.quantize_fp8_ref(wl.v_new, v_scale).view(torch.uint8).permute(1, 0, 2)
    assert torch.equal(kd.cpu().view(torch.uint8), k_want) and torch.equal(vd.cpu().view(torch.uint8), v_want)
    assert torch.isfinite(kd.float()).all()
    # 8-bit pools go through the same gather kernels (raw bytes)
    lens = (wl.ctx_len + 1).to(DEV)
    got = iva_b200.paged_gather(kd, wl.block_table.to(DEV), lens, 16, layout="head_major", check=True)
    want = ref.paged_gather_ref(k_want.view(torch.uint8), wl.block_table, wl.ctx_len + 1, 16)
    for g, w in zip(got, want):
        assert torch.equal(g.cpu().view(torch.uint8), w)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("Hq,Hkv,D", [(4, 4, 128), (8, 2, 128), (8, 4, 64), (16, 2, 128), (32, 8, 128), (16, 8, 128), (16, 4, 64), (16, 2, 64),
                                      (6, 2, 128), (14, 2, 128), (10, 2, 64), (32, 2, 128)])
def test_decode_on_fp8_pools(dtype, Hq, Hkv, D):
    ctx = torch.tensor([0, 1, 15, 16, 17, 100, 700, 3000])
    k_scale, v_scale = 0.02, 0.025
    wl, k8, v8 = _fp8_workload(ctx, Hq, Hkv, D, dtype, Hq + D, k_scale, v_scale, poison=True)
    kd, vd = k8.to(DEV), v8.to(DEV)
    d = wl.to(DEV)
    iva_b200.paged_append(kd, vd, d.slot_mapping, d.k_new, d.v_new, 16, check=True, k_scale=k_scale, v_scale=v_scale)
    lens = (d.ctx_len + 1).contiguous()
    # checker: the same attention on the dequantised pools (what the kernel must reproduce) ...
    kf = ref.dequantize_fp8_ref(kd.cpu(), k_scale)
    vf = ref.dequantize_fp8_ref(vd.cpu(), v_scale)
    out_ref, lse_ref = ref.paged_decode_ref(wl.q, kf, vf, wl.block_table, wl.ctx_len + 1, 16, wl.scale)
    out, lse = check_decode(lambda od: iva_b200.paged_decode_attention(
        d.q, kd, vd, d.block_table, lens, 16, wl.scale, return_lse=True, check=True, k_scale=k_scale, v_scale=v_scale,
        out_dtype=od), out_ref, lse_ref, dtype)
    # ... and, for the record, the cost of storing 8 bits: against the 16-bit pools
    _, _, out16, _ = ref.decode_step_ref(wl)
    rel = (out.float().cpu() - out16).norm() / out16.norm()
    assert rel < 0.08, f"quantisation error {rel:.3f}"


@pytest.mark.parametrize("Hkv,D", [(8, 128), (2, 128), (2, 64)])
def test_fp8_window_and_sinks_and_errors(Hkv, D):
    ctx = torch.tensor([300, 47, 5000])
    wl, k8, v8 = _fp8_workload(ctx, 8, Hkv, D, torch.bfloat16, 9, 0.02, 0.02)
    begin = torch.tensor([261, 10, 4000])
    d = wl.to(DEV)
    out_ref, lse_ref = ref.paged_decode_ref(wl.q, ref.dequantize_fp8_ref(k8, 0.02), ref.dequantize_fp8_ref(v8, 0.02),
                                            wl.block_table, wl.ctx_len, 16, wl.scale, ctx_begin=begin, sink_tokens=4)
    kd8, vd8 = k8.to(DEV), v8.to(DEV)
    check_decode(lambda od: iva_b200.paged_decode_attention(
        d.q, kd8, vd8, d.block_table, d.ctx_len, 16, wl.scale, return_lse=True, check=True, ctx_begin=begin.to(DEV),
        sink_tokens=4, k_scale=0.02, v_scale=0.02, out_dtype=od), out_ref, lse_ref, torch.bfloat16)
    with pytest.raises(ValueError, match="fp16 or bf16"):
        iva_b200.paged_decode_attention(d.q.float(), k8.to(DEV), v8.to(DEV), d.block_table, d.ctx_len, 16)
    with pytest.raises(ValueError, match="positive"):
        iva_b200.paged_decode_attention(d.q, k8.to(DEV), v8.to(DEV), d.block_table, d.ctx_len, 16, k_scale=0.0)


def test_widening_engine_still_passes():
    """IVAB_FP8_REG=0 (read once per process): grouped-query decode on 8-bit pools goes through the
    engine that widens each page to fp16 tiles in shared memory; the same cases pass."""
    import os, subprocess, sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, IVAB_FP8_REG="0")
    res = subprocess.run([sys.executable, "-m", "pytest", os.path.join(root, "tests", "test_gpu_fp8_kv.py"), "-q", "-x",
                          "-m", "gpu", "-k", "decode_on_fp8_pools or window_and_sinks", "-p", "no:cacheprovider"],
                         env=env, capture_output=True, text=True, timeout=900, cwd=root)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-2000:]


def test_graphed_step_on_fp8_pools():
    """GraphedDecodeStep with e4m3 pools: quantising append + attention replayed from pinned host
    buffers, three steps, each against the checker on the dequantised pools it should have produced."""
    ks, vs = 0.02, 0.03
    B, Hq, Hkv, D = 3, 8, 2, 128
    ctx = torch.tensor([40, 17, 300])
    # pools and block tables with room for three more tokens per sequence
    wl3 = workloads.make_decode_workload("fp8step", ctx + 3, n_q_heads=Hq, n_kv_heads=Hkv, head_dim=D,
                                         dtype=torch.bfloat16, seed=21, free_frac=0.2)
    k8, v8 = ref.quantize_fp8_ref(wl3.k_pool, ks), ref.quantize_fp8_ref(wl3.v_pool, vs)
    kd, vd = k8.to(DEV), v8.to(DEV)
    bt = wl3.block_table.to(DEV)
    step = iva_b200.GraphedDecodeStep(kd, vd, bt, n_q_heads=Hq, return_lse=True, token_dtype=torch.bfloat16,
                                      k_scale=ks, v_scale=vs)
    g = torch.Generator().manual_seed(5)
    k_ref, v_ref = k8.clone(), v8.clone()
    for t in range(3):
        L = ctx + t
        q = torch.randn(B, Hq, D, generator=g).to(torch.bfloat16)
        kn = torch.randn(B, Hkv, D, generator=g).to(torch.bfloat16)
        vn = torch.randn(B, Hkv, D, generator=g).to(torch.bfloat16)
        slots = torch.tensor([int(wl3.block_table[s, int(L[s]) // 16]) * 16 + int(L[s]) % 16 for s in range(B)])
        step.q_host.copy_(q); step.k_new_host.copy_(kn); step.v_new_host.copy_(vn)
        step.slot_mapping_host.copy_(slots); step.ctx_len_host.copy_((L + 1).to(torch.int32))
        step.run()
        out = step.result().clone()
        lse = step.lse_host.clone()
        k_ref[0, :, slots] = ref.quantize_fp8_ref(kn, ks).permute(1, 0, 2)
        v_ref[0, :, slots] = ref.quantize_fp8_ref(vn, vs).permute(1, 0, 2)
        out_ref, lse_ref = ref.paged_decode_ref(q, ref.dequantize_fp8_ref(k_ref, ks), ref.dequantize_fp8_ref(v_ref, vs),
                                                wl3.block_table, L + 1, 16, wl3.scale)
        assert_attn_close(out, out_ref, torch.bfloat16, strict=False)
        assert_lse_close(lse, lse_ref)
    assert torch.equal(kd.cpu().view(torch.uint8), k_ref.view(torch.uint8))
    assert step.graph is not None
