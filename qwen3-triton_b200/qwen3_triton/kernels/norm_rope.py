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


class _QKNormRoPE(torch.autograd.Function):
    """q [B,S,Hq,D] and k [B,S,Hk,D] through per-head RMSNorm + RoPE in one launch per direction
    (reference ops/triton/fused_qk_norm_rope.py:`_FusedQKNormRoPEFunction`)."""

    @staticmethod
    def forward(ctx, q, k, qw, kw, cos, sin, eps):
        for x, w in ((q, qw), (k, kw)):
            if (x.ndim != 4 or w.shape != (x.shape[-1],) or cos.shape != sin.shape
                    or cos.shape != (x.shape[0], x.shape[1], x.shape[-1])):
                raise ValueError('Expected [B,S,heads,D], [D] and [B,S,D]')
        if not q.is_cuda or any(t.device != q.device or t.dtype != q.dtype or not t.is_contiguous()
                                for t in (q, k, qw, kw, cos, sin)):
            raise ValueError('Matching contiguous CUDA tensors required')
        if q.dtype not in _abi.FLOAT_DTYPES or q.shape[-1] % 2 or q.numel() < 1 or k.numel() < 1 or eps <= 0:
            raise ValueError('Floating point, even nonempty D and positive epsilon required')
        if cos.requires_grad or sin.requires_grad:
            raise ValueError('Fixed rotary buffers only')
        b, s, hq, d = q.shape
        hk = k.shape[2]
        yq, yk = torch.empty_like(q), torch.empty_like(k)
        invq = torch.empty(b * s * hq, device=q.device, dtype=torch.float32)
        invk = torch.empty(b * s * hk, device=q.device, dtype=torch.float32)
        _abi.call('q3_qk_norm_rope_fwd', q.data_ptr(), k.data_ptr(), qw.data_ptr(), kw.data_ptr(), cos.data_ptr(),
                  sin.data_ptr(), yq.data_ptr(), yk.data_ptr(), invq.data_ptr(), invk.data_ptr(), b * s, hq, hk, d,
                  float(eps), _abi.dt(q.dtype), _abi.stream())
        ctx.save_for_backward(q, k, qw, kw, cos, sin, invq, invk)
        return yq, yk

    @staticmethod
    def backward(ctx, dyq, dyk):
        q, k, qw, kw, cos, sin, invq, invk = ctx.saved_tensors
        dyq, dyk = dyq.contiguous(), dyk.contiguous()
        b, s, hq, d = q.shape
        hk = k.shape[2]
        dq, dk, dqw, dkw = torch.empty_like(q), torch.empty_like(k), torch.empty_like(qw), torch.empty_like(kw)
        ws = _abi.workspace(_abi.lib().q3_qk_norm_rope_bwd_workspace_bytes(b * s, hq, hk, d), q.device)
        _abi.call('q3_qk_norm_rope_bwd', q.data_ptr(), k.data_ptr(), qw.data_ptr(), kw.data_ptr(), cos.data_ptr(),
                  sin.data_ptr(), dyq.data_ptr(), dyk.data_ptr(), invq.data_ptr(), invk.data_ptr(), dq.data_ptr(),
                  dk.data_ptr(), dqw.data_ptr(), dkw.data_ptr(), ws.data_ptr(), ws.numel(), b * s, hq, hk, d,
                  _abi.dt(q.dtype), _abi.stream())
        return dq, dk, dqw, dkw, None, None, None


def qk_norm_rope(q, k, q_weight, k_weight, cos, sin, eps=1e-6):
    return _QKNormRoPE.apply(q, k, q_weight, k_weight, cos, sin, eps)
