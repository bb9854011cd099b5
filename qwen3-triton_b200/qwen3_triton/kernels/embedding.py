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
        ws = _abi.workspace(_abi.lib().q3_embedding_bwd_workspace_bytes(ids.numel()), dy.device)
        _abi.call('q3_embedding_bwd', ids.data_ptr(), int(ids.dtype == torch.int64), dy.data_ptr(), dw.data_ptr(),
                  ws.data_ptr(), ws.numel(), ids.numel(), h, v, _abi.dt(ctx.weight_dtype), _abi.stream())
        return None, dw


def embedding(ids, weight):
    return _Embedding.apply(ids, weight)


def shard_lookup(ids, weight_shard, row_lo, vocab, dtype):
    """Rows of one vocabulary shard (`weight_shard` = table rows [row_lo, row_lo + rows), fp32 master or `dtype`)
    for every id in `ids`, zeros where another shard owns the id. No autograd: the vocabulary-parallel embedding
    (training/vocab_parallel.py) owns the graph."""
    if not ids.is_cuda or ids.device != weight_shard.device or ids.dtype not in (torch.int32, torch.int64):
        raise ValueError('Same-device CUDA integer IDs required; no fallback')
    if weight_shard.ndim != 2 or not weight_shard.is_contiguous() or not ids.is_contiguous() or weight_shard.shape[1] % 8:
        raise ValueError('Contiguous [rows, H] shard with H % 8 == 0 required')
    rows, h = weight_shard.shape
    y = torch.empty((ids.numel(), h), device=ids.device, dtype=dtype)
    _abi.call('q3_embedding_shard_fwd', ids.data_ptr(), int(ids.dtype == torch.int64), weight_shard.data_ptr(),
              _abi.dt(weight_shard.dtype), y.data_ptr(), _abi.dt(dtype), ids.numel(), h, vocab, row_lo, rows,
              _abi.status_word(ids.device).data_ptr(), _abi.stream())
    return y


def shard_weight_gradient(ids, dy, row_lo, rows, scale):
    """fp32 gradient [rows, H] of one vocabulary shard: scale * sum of the dy rows of the positions it owns."""
    if not dy.is_cuda or dy.device != ids.device or dy.ndim != 2 or dy.shape[0] != ids.numel() or not dy.is_contiguous():
        raise ValueError('Contiguous [tokens, H] CUDA gradient required; no fallback')
    h = dy.shape[1]
    dw = torch.empty((rows, h), device=dy.device, dtype=torch.float32)
    ws = _abi.workspace(_abi.lib().q3_embedding_bwd_workspace_bytes(ids.numel()), dy.device)
    _abi.call('q3_embedding_shard_bwd', ids.data_ptr(), int(ids.dtype == torch.int64), dy.data_ptr(), _abi.dt(dy.dtype),
              dw.data_ptr(), ws.data_ptr(), ws.numel(), ids.numel(), h, row_lo, rows, float(scale), _abi.stream())
    return dw
