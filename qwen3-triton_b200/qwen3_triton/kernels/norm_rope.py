"""Fused per-head RMSNorm + split-half RoPE (reference qwen3_triton/kernels/norm_rope.py:52-71;
math of ops/reference/fused_qk_norm_rope.py:9-80)."""
import torch

from .. import _abi


class _NormRoPE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, cos, sin, eps):
        if (x.ndim != 4 or w.shape != (x.shape[-1],) or cos.shape != sin.shape
                or cos.shape != (x.shape[0], x.shape[1], x.shape[-1])):
            raise ValueError('Expected [B,S,heads,D], [D] and [B,S,D]')
        if not x.is_cuda or any(t.device != x.device or t.dtype != x.dtype or not t.is_contiguous() for t in (x, w, cos, sin)):
            raise ValueError('Matching contiguous CUDA tensors required')
        if x.dtype not in _abi.FLOAT_DTYPES or x.shape[-1] % 2 or x.numel() < 1 or eps <= 0:
            raise ValueError('Floating point, even nonempty D and positive epsilon required')
        if cos.requires_grad or sin.requires_grad:
            raise ValueError('Fixed rotary buffers only')
        b, s, heads, d = x.shape
        y = torch.empty_like(x)
        inv = torch.empty(b * s * heads, device=x.device, dtype=torch.float32)
        _abi.call('q3_norm_rope_fwd', x.data_ptr(), w.data_ptr(), cos.data_ptr(), sin.data_ptr(), y.data_ptr(),
                  inv.data_ptr(), b * s, heads, d, float(eps), _abi.dt(x.dtype), _abi.stream())
        ctx.save_for_backward(x, w, cos, sin, inv)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, cos, sin, inv = ctx.saved_tensors
        dy = dy.contiguous()
        b, s, heads, d = x.shape
        dx = torch.empty_like(x)
        dw = torch.empty_like(w)
        ws = _abi.workspace(_abi.lib().q3_norm_rope_bwd_workspace_bytes(b * s, heads, d), x.device)
        _abi.call('q3_norm_rope_bwd', x.data_ptr(), w.data_ptr(), cos.data_ptr(), sin.data_ptr(), dy.data_ptr(),
                  inv.data_ptr(), dx.data_ptr(), dw.data_ptr(), ws.data_ptr(), ws.numel(), b * s, heads, d,
                  _abi.dt(x.dtype), _abi.stream())
        return dx, dw, None, None, None


def norm_rope(x, weight, cos, sin, eps=1e-6):
    return _NormRoPE.apply(x, weight, cos, sin, eps)
