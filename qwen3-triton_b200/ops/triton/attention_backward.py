"""`attention_backward_triton(q, k, v, grad_out, *, scale, lse)` (reference ops/triton/attention_backward.py:196-236)."""
import math

from qwen3_triton.kernels.attention import attention_backward, attention_forward


def attention_backward_triton(q, k, v, grad_out, *, scale: float | None = None, lse=None):
    if q.ndim != 4 or k.ndim != 4 or v.shape != k.shape or grad_out.shape != q.shape:
        raise ValueError("invalid attention or grad_out shapes")
    if not all(t.is_cuda for t in (q, k, v, grad_out)):
        raise ValueError("attention_backward_triton requires CUDA tensors")
    q, k, v, grad_out = (t.contiguous() for t in (q, k, v, grad_out))
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    # the output (for delta = rowsum(dO*O)) and, if not given, the log-sum-exp come from one forward pass
    out, fresh_lse = attention_forward(q, k, v, scale)
    return attention_backward(q, k, v, out, grad_out, lse.contiguous() if lse is not None else fresh_lse, scale)
