"""Causal token-mean cross-entropy over materialised logits: the shift, log-sum-exp, count, mean and
backward all run in CUDA kernels (reference qwen3_triton/kernels/loss.py:46-71; semantics of
model/qwen_tiny.py:224-227)."""
import torch

from .. import _abi


class _CausalCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, labels, ignore_index, optimized):
        if not logits.is_cuda or logits.device != labels.device or logits.ndim != 3 or labels.shape != logits.shape[:2]:
            raise ValueError('CUDA [B,S,V] logits and same-device [B,S] labels required')
        if labels.dtype != torch.int64 or not logits.is_contiguous() or not labels.is_contiguous():
            raise ValueError('Contiguous logits/int64 labels required')
        if logits.dtype not in _abi.FLOAT_DTYPES:
            raise TypeError('Floating point logits required')
        b, s, v = logits.shape
        if b < 1 or s < 2 or v < 1:
            raise ValueError('Nonempty batch/vocabulary and at least 2 tokens required')
        n = b * (s - 1)
        dev = logits.device
        lse = torch.empty(n, device=dev, dtype=torch.float32)
        target = torch.empty_like(lse)
        losses = torch.empty_like(lse)
        count = torch.empty((), device=dev, dtype=torch.int32)
        loss = torch.empty((), device=dev, dtype=torch.float32)
        _abi.call('q3_ce_fwd', logits.data_ptr(), labels.data_ptr(), lse.data_ptr(), target.data_ptr(),
                  losses.data_ptr(), loss.data_ptr(), count.data_ptr(), b, s, v, ignore_index, _abi.dt(logits.dtype),
                  _abi.status_word(dev).data_ptr(), _abi.stream())
        ctx.save_for_backward(logits, labels, lse, count)
        ctx.ignore = ignore_index
        return loss

    @staticmethod
    def backward(ctx, dy):
        x, labels, lse, count = ctx.saved_tensors
        b, s, v = x.shape
        dx = torch.empty_like(x)
        up = dy.contiguous().float().view(1)
        _abi.call('q3_ce_grad', x.data_ptr(), labels.data_ptr(), lse.data_ptr(), count.data_ptr(), up.data_ptr(),
                  dx.data_ptr(), b * s, b * s, s, v, 0, v, ctx.ignore, _abi.dt(x.dtype), _abi.stream())
        return dx, None, None, None


def causal_cross_entropy(logits, labels, *, ignore_index=-100, optimized=False):
    return _CausalCE.apply(logits, labels, ignore_index, optimized)
