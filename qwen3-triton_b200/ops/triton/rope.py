"""`apply_rope_triton(q, k, cos, sin)` on [B, H, S, D] tensors with cos/sin [B, S, D]
(reference ops/triton/rope.py:150-170; math of ops/reference/rope.py:13-55)."""
import torch

from qwen3_triton.kernels.rotary import _apply


def _check(x, cos, sin):
    if x.ndim != 4 or cos.shape != sin.shape or cos.shape != (x.shape[0], x.shape[2], x.shape[3]) or x.shape[-1] % 2:
        raise ValueError("expected [B,H,S,D] tensors and [B,S,D] cos/sin with even D")
    if not x.is_cuda:
        raise ValueError("apply_rope_triton requires CUDA tensors")


class _RoPEFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, cos, sin):
        _check(q, cos, sin)
        _check(k, cos, sin)
        cos = cos.to(q.dtype).contiguous()
        sin = sin.to(q.dtype).contiguous()
        ctx.save_for_backward(cos, sin)
        return _apply(q.contiguous(), cos, sin, False, 1), _apply(k.contiguous(), cos, sin, False, 1)

    @staticmethod
    def backward(ctx, grad_q, grad_k):
        cos, sin = ctx.saved_tensors
        return _apply(grad_q.contiguous(), cos, sin, True, 1), _apply(grad_k.contiguous(), cos, sin, True, 1), None, None


def apply_rope_triton(q, k, cos, sin):
    return _RoPEFunction.apply(q, k, cos, sin)
