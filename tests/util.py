"""Helpers shared by the GPU parity tests."""

import torch

# Tolerances of the decode-attention parity bar: max-abs 2e-3 (bf16), 1e-3 (fp16), and 1e-3 on the
# per-head logsumexp.  fp32 inputs are held to 2e-5.
OUT_TOL = {torch.bfloat16: 2e-3, torch.float16: 1e-3, torch.float32: 2e-5}
LSE_TOL = 1e-3
# One unit in the last place of the storage dtype, relative: the kernel's fp32 result is rounded
# once to the output dtype, which for |out| of order 1 (contexts of a few tokens) is itself larger
# than the absolute bar.  Tests on such short contexts allow abs + one rounding step.
ULP = {torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11, torch.float32: 0.0}


def assert_attn_close(got, ref32, dtype, strict=True, what="out"):
    got32 = got.float().cpu()
    ref32 = ref32.float().cpu()
    assert torch.isfinite(got32).all(), f"{what}: non-finite values"
    err = (got32 - ref32).abs()
    if strict:
        assert err.max().item() <= OUT_TOL[dtype], f"{what}: max-abs {err.max().item():.3e} > {OUT_TOL[dtype]}"
    else:
        bound = OUT_TOL[dtype] + ULP[dtype] * ref32.abs()
        bad = err > bound
        assert not bad.any(), f"{what}: max-abs {err.max().item():.3e} beyond abs+1ulp bound"


def assert_lse_close(got, ref):
    got, ref = got.float().cpu(), ref.float().cpu()
    inf = torch.isinf(ref)
    assert torch.equal(torch.isinf(got), inf)
    err = (got[~inf] - ref[~inf]).abs()
    if err.numel():
        assert err.max().item() <= LSE_TOL, f"lse: max-abs {err.max().item():.3e} > {LSE_TOL}"


def check_decode(call, out_ref, lse_ref, dtype):
    """``call(out_dtype) -> (out, lse)`` runs one decode-attention call.  The fp32 output is held to
    the plain bar (2e-3 for bf16 inputs, 1e-3 for fp16, 2e-5 for fp32; logsumexp 1e-3), i.e. the
    kernels' arithmetic is checked BEFORE the final rounding; the output in q's own 16-bit type may
    differ from the checker by that bar plus one rounding step of the stored value, and must be
    exactly the fp32 output rounded to that type."""
    out, lse = call(None)
    assert out.dtype == dtype
    assert_attn_close(out, out_ref, dtype, strict=False)
    assert_lse_close(lse, lse_ref)
    if dtype == torch.float32:
        assert_attn_close(out, out_ref, dtype, strict=True)
        return out, lse
    out32, lse32 = call(torch.float32)
    assert out32.dtype == torch.float32
    assert_attn_close(out32, out_ref, dtype, strict=True, what="fp32 out")
    assert_lse_close(lse32, lse_ref)
    assert torch.equal(out32.to(dtype), out), "the 16-bit output is not the rounded fp32 output"
    assert torch.equal(lse32, lse)
    return out, lse
