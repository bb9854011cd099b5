"""Stand-alone causal GQA attention entry points (reference ops/triton/attention.py:136-292)."""
import math

import torch

from qwen3_triton.kernels.attention import _Attention, attention_forward


def _validate(q, k, v, is_causal):
    if not all(t.is_cuda for t in (q, k, v)):
        raise ValueError("attention_triton requires CUDA tensors")
    if not (q.ndim == k.ndim == v.ndim == 4):
        raise ValueError("q, k, and v must be rank-4 tensors")
    batch, q_heads, q_len, head_dim = q.shape
    k_batch, kv_heads, k_len, k_dim = k.shape
    if (k_batch, k_len, k_dim) != (batch, q_len, head_dim):
        raise ValueError("q/k sequence and head_dim shapes must match")
    if v.shape != (batch, kv_heads, q_len, head_dim):
        raise ValueError("v must have shape [batch, kv_heads, seq_len, head_dim]")
    if q_heads % kv_heads != 0:
        raise ValueError("q_heads must be divisible by kv_heads for GQA")
    if not is_causal:
        raise NotImplementedError("only causal attention is supported")
    if head_dim <= 0 or head_dim % 2 != 0 or head_dim > 256:
        raise ValueError("head_dim must be a positive even number <= 256")


def attention_triton(q, k, v, *, is_causal: bool = True, scale: float | None = None, return_lse: bool = False):
    _validate(q, k, v, is_causal)
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    out, lse = attention_forward(q.contiguous(), k.contiguous(), v.contiguous(), scale)
    return (out, lse) if return_lse else out


def attention_triton_with_lse(q, k, v, *, scale: float | None = None):
    return attention_triton(q, k, v, scale=scale, return_lse=True)


def attention_triton_autograd(q, k, v, *, scale: float | None = None):
    _validate(q, k, v, True)
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    return _Attention.apply(q.contiguous(), k.contiguous(), v.contiguous(), scale, True)
