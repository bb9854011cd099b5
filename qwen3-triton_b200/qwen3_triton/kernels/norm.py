"""RMSNorm with saved inverse RMS and a deterministic weight gradient
(reference qwen3_triton/kernels/norm.py:39-66; math of ops/reference/rms_norm.py:6-13), plus the fused
residual-add + RMSNorm operator the bandwidth-bound sweep measures."""
import torch

from .. import _abi


def _validate(x, weight, eps):
    if not x.is_cuda or x.device != weight.device or x.dtype != weight.dtype:
        raise ValueError('Same-device/dtype CUDA input and weight required; no fallback')
    if x.dtype not in _abi.FLOAT_DTYPES:
        raise TypeError('Floating point required')
    if (weight.ndim != 1 or not x.is_contiguous() or not weight.is_contiguous()
            or x.shape[-1] != weight.numel() or x.numel() < 1):
        raise ValueError('Contiguous [...,H] input and [H] weight required')
    if weight.numel() > 8192 or eps <= 0:
        raise ValueError('Supported H<=8192 and positive epsilon required')


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps, optimized):
        _validate(x, weight, eps)
        h = weight.numel()
        rows = x.numel() // h
        y = torch.empty_like(x)
        inv = torch.empty(rows, device=x.device, dtype=torch.float32)
        _abi.call('q3_rmsnorm_fwd', x.data_ptr(), weight.data_ptr(), y.data_ptr(), inv.data_ptr(), rows, h,
                  float(eps), _abi.dt(x.dtype), _abi.stream())
        ctx.save_for_backward(x, weight, inv)
        ctx.optimized = optimized
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, inv = ctx.saved_tensors
        dy = dy.contiguous()
        h = w.numel()
        rows = inv.numel()
        dx = torch.empty_like(x)
        dw = torch.empty_like(w)
        nbytes = _abi.lib().q3_rmsnorm_bwd_workspace_bytes(rows, h)
        ws = _abi.workspace(nbytes, x.device)
        _abi.call('q3_rmsnorm_bwd', x.data_ptr(), w.data_ptr(), dy.data_ptr(), inv.data_ptr(), dx.data_ptr(),
                  dw.data_ptr(), ws.data_ptr(), ws.numel(), rows, h, _abi.dt(x.dtype), _abi.stream())
        return dx, dw, None, None


def rms_norm(x, weight, eps=1e-6, *, optimized=False):
    return _RMSNorm.apply(x, weight, eps, optimized)


class _AddRMSNorm(torch.autograd.Function):
    """(y, residual_out) = (RMSNorm(x + residual) * weight, x + residual) in one pass over HBM."""

    @staticmethod
    def forward(ctx, x, residual, weight, eps):
        _validate(x, weight, eps)
        if residual.shape != x.shape or residual.dtype != x.dtype or residual.device != x.device or not residual.is_contiguous():
            raise ValueError('Residual must match the input in shape, dtype, device and be contiguous')
        h = weight.numel()
        rows = x.numel() // h
        y = torch.empty_like(x)
        res_out = torch.empty_like(x)
        inv = torch.empty(rows, device=x.device, dtype=torch.float32)
        _abi.call('q3_add_rmsnorm_fwd', x.data_ptr(), residual.data_ptr(), weight.data_ptr(), y.data_ptr(),
                  res_out.data_ptr(), inv.data_ptr(), rows, h, float(eps), _abi.dt(x.dtype), _abi.stream())
        ctx.save_for_backward(res_out, weight, inv)
        return y, res_out

    @staticmethod
    def backward(ctx, dy, dres):
        res_out, w, inv = ctx.saved_tensors
        h = w.numel()
        rows = inv.numel()
        dy = dy.contiguous() if dy is not None else torch.zeros_like(res_out)
        dres = dres.contiguous() if dres is not None else None
        dx = torch.empty_like(res_out)
        dw = torch.empty_like(w)
        nbytes = _abi.lib().q3_rmsnorm_bwd_workspace_bytes(rows, h)
        ws = _abi.workspace(nbytes, res_out.device)
        _abi.call('q3_add_rmsnorm_bwd', res_out.data_ptr(), w.data_ptr(), dy.data_ptr(), _abi.ptr(dres),
                  inv.data_ptr(), dx.data_ptr(), dw.data_ptr(), ws.data_ptr(), ws.numel(), rows, h,
                  _abi.dt(res_out.dtype), _abi.stream())
        return dx, dx, dw, None


def add_rms_norm(x, residual, weight, eps=1e-6):
    return _AddRMSNorm.apply(x, residual, weight, eps)
