"""Split-half rotary tables and application (reference qwen3_triton/kernels/rotary.py:36-66;
math of ops/reference/rope.py:6-55)."""
import torch

from .. import _abi


def rotary_tables(position_ids, inv_freq, dtype):
    if not position_ids.is_cuda or inv_freq.device != position_ids.device:
        raise ValueError('Same CUDA device required')
    if position_ids.ndim != 2 or not position_ids.is_contiguous() or position_ids.dtype not in (torch.int32, torch.int64):
        raise ValueError('Contiguous integer [B,S] position IDs required')
    if inv_freq.dtype != torch.float32 or inv_freq.ndim != 1 or not inv_freq.is_contiguous():
        raise ValueError('Contiguous FP32 frequency buffer required')
    if dtype not in _abi.FLOAT_DTYPES:
        raise TypeError('Floating point output required')
    d = inv_freq.numel() * 2
    if position_ids.numel() < 1 or d < 2:
        raise ValueError('Nonempty positions/frequencies required')
    cos = torch.empty((*position_ids.shape, d), device=position_ids.device, dtype=dtype)
    sin = torch.empty_like(cos)
    _abi.call('q3_rope_tables', position_ids.data_ptr(), int(position_ids.dtype == torch.int64), inv_freq.data_ptr(),
              cos.data_ptr(), sin.data_ptr(), position_ids.numel(), d, _abi.dt(dtype), _abi.stream())
    return cos, sin


def _apply(x, cos, sin, backward, layout):
    y = torch.empty_like(x)
    if layout == 0:
        b, s, h, d = x.shape
    else:
        b, h, s, d = x.shape
    _abi.call('q3_rope_apply', x.data_ptr(), cos.data_ptr(), sin.data_ptr(), y.data_ptr(), b, s, h, d, int(backward),
              layout, _abi.dt(x.dtype), _abi.stream())
    return y


class _Rotary(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin):
        if x.ndim != 4 or cos.shape != sin.shape or cos.shape != (x.shape[0], x.shape[1], x.shape[3]) or x.shape[-1] % 2:
            raise ValueError('Expected [B,S,H,D] and matching [B,S,D], even D')
        if not x.is_cuda or any(t.device != x.device or t.dtype != x.dtype or not t.is_contiguous() for t in (x, cos, sin)):
            raise ValueError('Same-device/dtype contiguous CUDA tensors required')
        if cos.requires_grad or sin.requires_grad:
            raise ValueError('Fixed frequency buffers only')
        ctx.save_for_backward(cos, sin)
        return _apply(x, cos, sin, False, 0)

    @staticmethod
    def backward(ctx, dy):
        cos, sin = ctx.saved_tensors
        return _apply(dy.contiguous(), cos, sin, True, 0), None, None


def apply_rotary(x, cos, sin):
    return _Rotary.apply(x, cos, sin)
