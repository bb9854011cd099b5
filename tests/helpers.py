"""Comparison helpers shared by the parity tests."""
import torch

# Stated tolerances: bf16/fp16 outputs and gradients within 2e-2 (relative, with an absolute floor of
# 2e-2 of the tensor's typical magnitude); fp32 paths 2e-4; AdamW state 1e-5; loss 1e-3 relative.
TOL = {torch.bfloat16: 2e-2, torch.float16: 4e-3, torch.float32: 2e-4}


def close(actual, expected, dtype=None, scale=None, what="", atol_mult=2.0):
    """|actual - expected| <= tol * |expected| + tol * atol_mult * scale, scale = mean |expected| by default
    (with a floor of 1e-5 so an exactly-zero expectation admits rounding noise)."""
    dtype = dtype or actual.dtype
    tol = TOL[dtype]
    expected = expected.detach().float().cpu()
    actual = actual.detach().float().cpu()
    assert actual.shape == expected.shape, (what, actual.shape, expected.shape)
    assert torch.isfinite(actual).all(), what
    s = float(expected.abs().mean()) if scale is None else scale
    torch.testing.assert_close(actual, expected, rtol=tol, atol=max(tol * s * atol_mult, 1e-5),
                               msg=lambda m: f"{what}: {m}")


def rel_l2(actual, expected):
    a, e = actual.detach().float().cpu(), expected.detach().float().cpu()
    return float((a - e).norm() / e.norm().clamp_min(1e-30))


def randn(shape, seed, dtype=torch.float32, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)
