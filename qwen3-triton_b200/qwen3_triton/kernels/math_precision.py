"""The operator names the 8B training graph imports (reference qwen3_triton/kernels/math_precision.py:
rms_norm :37, norm_rope :64, swiglu :96). The reference keeps a second set of Triton kernels there that
reproduce PyTorch's summation order; here both sets of names share one set of kernels (fp32 math, one
rounding), which is what ops/reference computes."""
from .activation import _SwiGLU
from .norm import _RMSNorm
from .norm_rope import _NormRoPE


def rms_norm(x, w, eps=1e-6):
    return _RMSNorm.apply(x, w, eps, False)


def norm_rope(x, w, cos, sin, eps=1e-6):
    return _NormRoPE.apply(x, w, cos, sin, eps)


def swiglu(g, u, *, fma=True):
    return _SwiGLU.apply(g, u)
