"""SwiGLU y = silu(gate) * up with explicit forward/backward kernels
(reference qwen3_triton/kernels/activation.py:22-36; math of ops/reference/swiglu.py:9-21)."""
import torch

from .. import _abi


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, g, u):
        if (not g.is_cuda or g.device != u.device or g.shape != u.shape or g.dtype != u.dtype
                or not g.is_contiguous() or not u.is_contiguous() or g.numel() < 1):
            raise ValueError('Matching contiguous nonempty CUDA inputs required')
        if g.dtype not in _abi.FLOAT_DTYPES:
            raise TypeError('Floating point required')
        y = torch.empty_like(g)
        _abi.call('q3_swiglu_fwd', g.data_ptr(), u.data_ptr(), y.data_ptr(), g.numel(), _abi.dt(g.dtype),
                  _abi.stream())
        ctx.save_for_backward(g, u)
        return y

    @staticmethod
    def backward(ctx, dy):
        g, u = ctx.saved_tensors
        dy = dy.contiguous()
        dg = torch.empty_like(g)
        du = torch.empty_like(u)
        _abi.call('q3_swiglu_bwd', g.data_ptr(), u.data_ptr(), dy.data_ptr(), dg.data_ptr(), du.data_ptr(),
                  g.numel(), _abi.dt(g.dtype), _abi.stream())
        return dg, du


def swiglu(gate, up):
    return _SwiGLU.apply(gate, up)
