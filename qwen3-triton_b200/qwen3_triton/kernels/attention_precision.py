"""`candidate`: the attention entry the 8B training graph calls
(reference qwen3_triton/kernels/attention_precision.py:147-182). The keyword switches select between
Triton kernel variants in the reference; they are accepted and ignored here: there is one kernel family,
deterministic, with fp32 softmax statistics."""
import torch

from .attention import attention_backward, attention_forward, validate_qkv


class _NativePrecision(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, fusion, lane_sum, round_kv, reciprocal, stages, lse_fma, native_delta, xor_sum,
                native_dq, sum_fma):
        validate_qkv(q, k, v)
        if q.shape[-1] != 128 or q.dtype != torch.bfloat16:
            raise ValueError('BF16 head_dim 128 required on this entry point')
        scale = q.shape[-1] ** -0.5
        out, lse = attention_forward(q, k, v, scale)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.scale = scale
        return out

    @staticmethod
    def backward(ctx, g):
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = attention_backward(q, k, v, out, g.contiguous(), lse, ctx.scale)
        return (dq, dk, dv) + (None,) * 10


def candidate(q, k, v, *, fusion=False, lane_sum=True, round_kv=True, reciprocal=1, stages=1, lse_fma=False,
              native_delta=False, xor_sum=True, native_dq=False, sum_fma=False):
    return _NativePrecision.apply(q, k, v, fusion, lane_sum, round_kv, reciprocal, stages, lse_fma, native_delta,
                                  xor_sum, native_dq, sum_fma)
