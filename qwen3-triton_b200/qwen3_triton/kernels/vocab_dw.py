"""Per-data-rank weight-gradient GEMMs of the vocab-parallel head, each rounded to BF16 and averaged in
FP32 in rank order (reference qwen3_triton/kernels/vocab_dw.py:33-44). Any world size and row count."""
import torch

from .linear import matmul
from .vocab_ce import accumulate_weight_gradient


def weight_gradient_mean(dz, hidden, rows_per_rank, world, config=None):
    if (dz.dtype != torch.bfloat16 or hidden.dtype != torch.bfloat16 or not dz.is_cuda
            or dz.device != hidden.device or not dz.is_contiguous() or not hidden.is_contiguous()
            or dz.shape[0] != hidden.shape[0] or dz.shape[0] != rows_per_rank * world):
        raise ValueError('Contiguous same-device BF16 [world*R,V] dZ and [world*R,H] hidden required')
    v, k = dz.shape[1], hidden.shape[1]
    out = torch.empty((v, k), device=dz.device, dtype=torch.float32)
    for source in range(world):
        rows = slice(source * rows_per_rank, (source + 1) * rows_per_rank)
        partial = matmul(dz[rows].t(), hidden[rows], optimized=True)
        accumulate_weight_gradient(partial, out, world, source == 0)
    return out
