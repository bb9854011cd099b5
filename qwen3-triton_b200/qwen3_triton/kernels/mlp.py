"""Fused gate/up projections + SwiGLU forward with saved gate/up tensors and a full backward
(reference qwen3_triton/kernels/mlp.py:34-57 and kernels/mlp_precision.py:37-66)."""
import torch

from .. import _abi
from .linear import matmul
from .residual import residual_add


class _GateUp(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, wg, wu, optimized):
        if not x.is_cuda or x.ndim < 2 or wg.ndim != 2 or wg.shape != wu.shape or x.shape[-1] != wg.shape[1]:
            raise ValueError('Expected CUDA X[...,K] and matching [N,K] gate/up weights')
        if x.dtype not in _abi.FLOAT_DTYPES or any(
                t.device != x.device or t.dtype != x.dtype or not t.is_contiguous() for t in (x, wg, wu)):
            raise ValueError('Matching contiguous floating point CUDA inputs required')
        k = x.shape[-1]
        m = x.numel() // k
        n = wg.shape[0]
        if min(m, k, n) < 1:
            raise ValueError('Nonempty inputs required')
        shape = (*x.shape[:-1], n)
        g = torch.empty(shape, device=x.device, dtype=x.dtype)
        u = torch.empty_like(g)
        y = torch.empty_like(g)
        _abi.call('q3_gate_up_swiglu_fwd', x.data_ptr(), wg.data_ptr(), wu.data_ptr(), g.data_ptr(), u.data_ptr(),
                  y.data_ptr(), m, n, k, _abi.dt(x.dtype), _abi.status_word(x.device).data_ptr(), _abi.stream())
        ctx.save_for_backward(x, wg, wu, g, u)
        ctx.optimized = optimized
        return y

    @staticmethod
    def backward(ctx, dy):
        x, wg, wu, g, u = ctx.saved_tensors
        dy = dy.contiguous()
        k = x.shape[-1]
        m = x.numel() // k
        n = wg.shape[0]
        dg = torch.empty_like(g)
        du = torch.empty_like(u)
        _abi.call('q3_swiglu_bwd', g.data_ptr(), u.data_ptr(), dy.data_ptr(), dg.data_ptr(), du.data_ptr(), g.numel(),
                  _abi.dt(g.dtype), _abi.stream())
        dg = dg.view(m, n)
        du = du.view(m, n)
        flat = x.view(m, k)
        dx = None
        if ctx.needs_input_grad[0]:
            dx = residual_add(matmul(dg, wg, optimized=ctx.optimized), matmul(du, wu, optimized=ctx.optimized)).view(x.shape)
        dwg = matmul(dg.t(), flat, optimized=ctx.optimized) if ctx.needs_input_grad[1] else None
        dwu = matmul(du.t(), flat, optimized=ctx.optimized) if ctx.needs_input_grad[2] else None
        return dx, dwg, dwu, None


def gate_up_swiglu(x, gate_weight, up_weight, *, optimized=False):
    return _GateUp.apply(x, gate_weight, up_weight, optimized)
