"""`rms_norm_triton(x, weight, eps)` (reference ops/triton/rms_norm.py:136-138)."""
import torch

from qwen3_triton.kernels.norm import _RMSNorm


def rms_norm_triton(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    if not x.is_cuda:
        raise ValueError("rms_norm_triton requires CUDA tensors")
    return _RMSNorm.apply(x.contiguous(), weight.contiguous(), eps, False)
