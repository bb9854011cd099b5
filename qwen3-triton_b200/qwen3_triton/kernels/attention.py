"""Dense causal grouped-query attention, forward and backward, and the dtype cast helper
(reference qwen3_triton/kernels/attention.py:14-50; math of ops/reference/attention.py:10-124)."""
import math

import torch

from .. import _abi


def cast_tensor(x, dtype):
    if not x.is_cuda or not x.is_contiguous():
        raise ValueError('Contiguous CUDA tensor required')
    out = torch.empty(x.shape, device=x.device, dtype=dtype)
    if x.numel():
        _abi.call('q3_cast', x.data_ptr(), _abi.dt(x.dtype), out.data_ptr(), _abi.dt(dtype), x.numel(), _abi.stream())
    return out


def attention_forward(q, k, v, scale):
    """(out, lse) for contiguous q [B,Hq,S,D], k/v [B,Hkv,S,D]."""
    b, hq, s, d = q.shape
    hk = k.shape[1]
    out = torch.empty_like(q)
    lse = torch.empty((b, hq, s), device=q.device, dtype=torch.float32)
    _abi.call('q3_attn_fwd', q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), b, hq, hk, s, d,
              float(scale), _abi.dt(q.dtype), _abi.status_word(q.device).data_ptr(), _abi.stream())
    return out, lse


def attention_backward(q, k, v, out, dout, lse, scale):
    """(dq, dk, dv); dk/dv are already summed over the query heads of each group."""
    b, hq, s, d = q.shape
    hk = k.shape[1]
    dq = torch.empty_like(q)
    dk = torch.empty_like(k)
    dv = torch.empty_like(v)
    ws = _abi.workspace(_abi.lib().q3_attn_bwd_workspace_bytes(b, hq, hk, s, d), q.device)
    _abi.call('q3_attn_bwd', q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(),
              lse.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), ws.data_ptr(), ws.numel(), b, hq, hk, s, d,
              float(scale), _abi.dt(q.dtype), _abi.status_word(q.device).data_ptr(), _abi.stream())
    return dq, dk, dv


def attention_path(q, k, v):
    """'tcgen05' or 'simt': which kernels `causal_attention(q, k, v)` runs."""
    tc = _abi.lib().q3_attn_path(q.data_ptr(), k.data_ptr(), v.data_ptr(), q.data_ptr(), q.shape[-1], _abi.dt(q.dtype))
    return 'tcgen05' if tc else 'simt'


def validate_qkv(q, k, v):
    if q.ndim != 4 or k.ndim != 4 or v.shape != k.shape or q.shape[0] != k.shape[0] or q.shape[2:] != k.shape[2:]:
        raise ValueError('Expected equal-length [B,H,S,D] Q and grouped K/V')
    if not q.is_cuda or any(t.device != q.device or t.dtype != q.dtype or not t.is_contiguous() for t in (q, k, v)):
        raise ValueError('Same-device/dtype contiguous CUDA QKV required; no fallback')
    if q.dtype not in _abi.FLOAT_DTYPES:
        raise TypeError('Floating point QKV required')
    b, hq, s, d = q.shape
    hk = k.shape[1]
    if min(b, hq, hk, s, d) < 1 or hq % hk or d > 256 or d % 2:
        raise ValueError('Nonempty supported GQA with even D<=256 required')


class _Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, optimized):
        validate_qkv(q, k, v)
        out, lse = attention_forward(q, k, v, scale)
        ctx.save_for_backward(q, k, v, lse, out)
        ctx.scale = scale
        return out

    @staticmethod
    def backward(ctx, dy):
        q, k, v, lse, out = ctx.saved_tensors
        dq, dk, dv = attention_backward(q, k, v, out, dy.contiguous(), lse, ctx.scale)
        return dq, dk, dv, None, None


def causal_attention(q, k, v, *, scale=None, optimized=False):
    return _Attention.apply(q, k, v, scale if scale is not None else 1. / math.sqrt(q.shape[-1]), optimized)
