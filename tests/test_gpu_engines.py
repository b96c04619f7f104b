"""Both page engines of the decode kernel on the same inputs.  The engine is chosen per call from
the head-group size; IVAB_TC_MIN_GROUP (read once per process) moves the threshold, so each
setting runs in a child process."""

import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import sys, torch
sys.path.insert(0, {root!r}); sys.path.insert(0, {root!r} + "/tests")
import iva_b200
from iva_b200 import workloads
from oracle import paged_ref as ref
from util import check_decode
for dtype in (torch.bfloat16, torch.float16):
    for hq, hkv, D in ((4, 4, 128), (8, 2, 128), (16, 2, 64), (8, 4, 256), (8, 2, 256), (16, 2, 256)):
        ctx = torch.tensor([0, 1, 15, 16, 17, 100, 333, 2500])
        wl = workloads.make_decode_workload("eng", ctx, n_q_heads=hq, n_kv_heads=hkv, head_dim=D, dtype=dtype,
                                            seed=hq + D, free_frac=0.3, poison_unused=True)
        _, _, out_ref, lse_ref = ref.decode_step_ref(wl)
        d = wl.to("cuda")
        iva_b200.paged_append(d.k_pool, d.v_pool, d.slot_mapping, d.k_new, d.v_new, 16, check=True)
        lens = (d.ctx_len + 1).contiguous()
        check_decode(lambda od: iva_b200.paged_decode_attention(d.q, d.k_pool, d.v_pool, d.block_table, lens, 16,
                                                                return_lse=True, check=True, out_dtype=od),
                     out_ref, lse_ref, dtype)
# 8-bit pools: the same thresholds move these between the CUDA-core and the tensor-core engines
for hq, hkv, D in ((4, 4, 128), (8, 2, 128), (4, 4, 64)):
    ctx = torch.tensor([0, 1, 15, 16, 17, 100, 333, 2500])
    wl = workloads.make_decode_workload("eng8", ctx, n_q_heads=hq, n_kv_heads=hkv, head_dim=D, dtype=torch.bfloat16,
                                        seed=hq + D, free_frac=0.3, poison_unused=True)
    k8, v8 = ref.quantize_fp8_ref(wl.k_pool, 0.02).cuda(), ref.quantize_fp8_ref(wl.v_pool, 0.03).cuda()
    d = wl.to("cuda")
    out_ref, lse_ref = ref.paged_decode_ref(wl.q, ref.dequantize_fp8_ref(k8.cpu(), 0.02),
                                            ref.dequantize_fp8_ref(v8.cpu(), 0.03), wl.block_table, wl.ctx_len, 16, wl.scale)
    check_decode(lambda od: iva_b200.paged_decode_attention(d.q, k8, v8, d.block_table, d.ctx_len, 16, wl.scale,
                                                            return_lse=True, check=True, k_scale=0.02, v_scale=0.03,
                                                            out_dtype=od), out_ref, lse_ref, torch.bfloat16)
print("engines ok")
"""


@pytest.mark.parametrize("min_group", ["1", "2", "99"])
def test_engine_threshold(min_group):
    """1: tensor-core engine even for multi-head attention; 2: the default split; 99: CUDA cores only."""
    env = dict(os.environ, IVAB_TC_MIN_GROUP=min_group)
    res = subprocess.run([sys.executable, "-c", CHILD.format(root=ROOT)], env=env, capture_output=True, text=True,
                         timeout=600)
    assert res.returncode == 0 and "engines ok" in res.stdout, res.stdout[-2000:] + res.stderr[-4000:]


def test_plain_stream_order_launches():
    """IVAB_PDL=0: the attention and merge kernels are launched in plain stream order instead of
    as programmatic dependents; the same cases pass."""
    env = dict(os.environ, IVAB_PDL="0")
    res = subprocess.run([sys.executable, "-c", CHILD.format(root=ROOT)], env=env, capture_output=True, text=True,
                         timeout=600)
    assert res.returncode == 0 and "engines ok" in res.stdout, res.stdout[-2000:] + res.stderr[-4000:]
