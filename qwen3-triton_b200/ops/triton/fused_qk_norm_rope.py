"""`fused_qk_norm_rope_triton(q, k, q_weight, k_weight, cos, sin, eps)` on [B, S, heads, D] tensors
(reference ops/triton/fused_qk_norm_rope.py:237-273; math of ops/reference/fused_qk_norm_rope.py:9-80)."""
import torch

from qwen3_triton.kernels.norm_rope import _QKNormRoPE


def fused_qk_norm_rope_triton(q, k, q_weight, k_weight, cos, sin, eps: float = 1e-6):
    if not q.is_cuda:
        raise ValueError("fused_qk_norm_rope_triton requires CUDA tensors")
    cos = cos.detach().to(q.dtype).contiguous()
    sin = sin.detach().to(q.dtype).contiguous()
    return _QKNormRoPE.apply(q.contiguous(), k.contiguous(), q_weight.contiguous(), k_weight.contiguous(), cos, sin, eps)
