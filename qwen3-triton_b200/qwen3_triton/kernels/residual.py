"""Residual addition (reference qwen3_triton/kernels/residual.py:13-30)."""
import torch

from .. import _abi


class _Residual(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b):
        if not a.is_cuda or a.device != b.device or a.shape != b.shape or a.dtype != b.dtype:
            raise ValueError('Matching same-device CUDA tensors required; no fallback')
        if not a.is_contiguous() or not b.is_contiguous() or a.numel() < 1:
            raise ValueError('Contiguous nonempty residual inputs required')
        if a.dtype not in _abi.FLOAT_DTYPES:
            raise TypeError('Floating point inputs required')
        out = torch.empty_like(a)
        _abi.call('q3_residual_add', a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), _abi.dt(a.dtype),
                  _abi.stream())
        return out

    @staticmethod
    def backward(ctx, dy):
        return dy, dy


def residual_add(a, b):
    return _Residual.apply(a, b)
