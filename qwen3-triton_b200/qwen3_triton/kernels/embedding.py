"""Token embedding with a dense deterministic weight gradient
(reference qwen3_triton/kernels/embedding.py:49-81)."""
import torch

from .. import _abi


class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight):
        if not ids.is_cuda or not weight.is_cuda or ids.device != weight.device:
            raise ValueError('Same-device CUDA inputs required; no fallback')
        if ids.dtype not in (torch.int32, torch.int64) or weight.dtype not in _abi.FLOAT_DTYPES:
            raise TypeError('Integer IDs and floating point weight required')
        if not ids.is_contiguous() or not weight.is_contiguous() or weight.ndim != 2 or ids.numel() < 1:
            raise ValueError('Contiguous nonempty IDs and matrix weight required')
        v, h = weight.shape
        if min(v, h) < 1:
            raise ValueError('Nonempty vocabulary and hidden dimension required')
        y = torch.empty((*ids.shape, h), device=weight.device, dtype=weight.dtype)
        _abi.call('q3_embedding_fwd', ids.data_ptr(), int(ids.dtype == torch.int64), weight.data_ptr(), y.data_ptr(),
                  ids.numel(), h, v, _abi.dt(weight.dtype), _abi.status_word(ids.device).data_ptr(), _abi.stream())
        ctx.save_for_backward(ids)
        ctx.weight_shape = weight.shape
        ctx.weight_dtype = weight.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        ids, = ctx.saved_tensors
        v, h = ctx.weight_shape
        dy = dy.contiguous()
        dw = torch.empty((v, h), device=dy.device, dtype=ctx.weight_dtype)
        _abi.call('q3_embedding_bwd', ids.data_ptr(), int(ids.dtype == torch.int64), dy.data_ptr(), dw.data_ptr(),
                  ids.numel(), h, v, _abi.dt(ctx.weight_dtype), _abi.stream())
        return None, dw


def embedding(ids, weight):
    return _Embedding.apply(ids, weight)
