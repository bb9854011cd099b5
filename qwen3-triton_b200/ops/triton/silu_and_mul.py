"""`silu_and_mul_triton(gate, up)` (reference ops/triton/silu_and_mul.py:111-121)."""
import torch

from qwen3_triton.kernels.activation import _SwiGLU


def silu_and_mul_triton(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    if gate.shape != up.shape:
        raise ValueError(f"gate and up must have the same shape, got {gate.shape} and {up.shape}")
    if not (gate.is_cuda and up.is_cuda):
        raise ValueError("silu_and_mul_triton requires CUDA tensors")
    if not (gate.is_floating_point() and up.is_floating_point()):
        raise TypeError("SwiGLU inputs must be floating-point tensors")
    return _SwiGLU.apply(gate.contiguous(), up.contiguous())
