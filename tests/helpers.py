"""Comparison helpers shared by the parity tests."""
import os

import torch

# Stated tolerances. Elementwise: bf16/fp16 outputs and gradients within 2e-2 relative, with an absolute floor of
# 2e-2 of the tensor's typical magnitude (sums of products legitimately land near zero, where a relative bound means
# nothing); fp32 paths 2e-4; AdamW state 1e-5; loss 1e-3 relative. Per tensor: the relative L2 distance
# |actual - expected| / |expected| must also stay under L2 below - a whole wrong tile passes an elementwise floor
# when its values are small, but not this.
TOL = {torch.bfloat16: 2e-2, torch.float16: 4e-3, torch.float32: 2e-4}
L2 = {torch.bfloat16: 5e-3, torch.float16: 1.5e-3, torch.float32: 1e-4}
L2_ATTENTION_GRAD = {torch.bfloat16: 1e-2, torch.float16: 3e-3, torch.float32: 2e-4}

# (what, relative L2) of every comparison of the current test; tests/conftest.py appends the per-test maximum to the
# file named by Q3_TEST_L2_LOG when that variable is set.
l2_seen = []


def close(actual, expected, dtype=None, scale=None, what="", atol_mult=2.0, l2=None):
    """|actual - expected| <= tol * |expected| + tol * atol_mult * scale, scale = mean |expected| by default, or the
    mean of each last-dimension row with scale='row' (floor 1e-5 so an exactly-zero expectation admits rounding
    noise), and
    |actual - expected|_2 <= l2 * |expected|_2 (l2 = L2[dtype] by default; pass False to skip)."""
    dtype = dtype or actual.dtype
    tol = TOL[dtype]
    expected = expected.detach().float().cpu()
    actual = actual.detach().float().cpu()
    assert actual.shape == expected.shape, (what, actual.shape, expected.shape)
    assert torch.isfinite(actual).all(), what
    if isinstance(scale, str) and scale == 'row':
        # absolute floor per row of the last dimension: rows of one tensor can differ in magnitude by orders (the
        # attention output of query 1 averages two values, that of query 8000 thousands), and a rounding error scales
        # with the row's terms, not with the tensor's mean
        floor = (expected.abs().mean(dim=-1, keepdim=True) * (tol * atol_mult)).clamp_min(1e-5)
        excess = (actual - expected).abs() - tol * expected.abs() - floor
        worst = float(excess.max())
        assert worst <= 0, (f"{what}: {int((excess > 0).sum())} of {excess.numel()} elements outside "
                            f"{tol:g} * |expected| + {tol * atol_mult:g} * mean|expected row|, worst by {worst:.3e}")
    else:
        s = float(expected.abs().mean()) if scale is None else scale
        torch.testing.assert_close(actual, expected, rtol=tol, atol=max(tol * s * atol_mult, 1e-5),
                                   msg=lambda m: f"{what}: {m}")
    if l2 is False:
        return
    bound = L2[dtype] if l2 is None else l2
    norm = float(expected.norm())
    if norm > 0:
        r = float((actual - expected).norm()) / norm
        l2_seen.append((what, r))
        if not os.environ.get("Q3_TEST_L2_SOFT"):   # set to only record the distances (see conftest.py)
            assert r <= bound, f"{what}: relative L2 error {r:.3e} > {bound:.1e}"
        elif r > bound:
            l2_seen.append((what + " OVER " + format(bound, ".1e"), r))


def rel_l2(actual, expected):
    a, e = actual.detach().float().cpu(), expected.detach().float().cpu()
    return float((a - e).norm() / e.norm().clamp_min(1e-30))


def randn(shape, seed, dtype=torch.float32, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def l2_log_path():
    return os.environ.get("Q3_TEST_L2_LOG")
