"""lm_head projection + causal token-mean cross-entropy without the logits ever being written to memory.

`fused_linear_cross_entropy(hidden, weight, labels)` equals
`causal_cross_entropy(linear(hidden, weight), labels)` (reference qwen3_triton/kernels/loss.py:70-71 on the output
of kernels/linear.py:104-105), including the rounding of the logits to the activation dtype before the loss. The
forward runs one tensor-core GEMM whose epilogue reduces every 128x256 logit tile to softmax statistics; the
backward walks the vocabulary in chunks: a GEMM whose epilogue turns the recomputed logits of the chunk into dZ,
then dX += dZ W_chunk (fp32 accumulation) and dW_chunk = dZ^T hidden. Peak extra memory is one [tokens, chunk] dZ
buffer instead of two [tokens, vocab] tensors (5 GB each at 16384 tokens).
"""
import torch

from .. import _abi
from .linear import matmul

DEFAULT_CHUNK = 16384


def shifted_labels(labels, ignore_index, vocab_total):
    eff = torch.empty(labels.numel(), device=labels.device, dtype=torch.int64)
    _abi.call('q3_shift_labels', labels.data_ptr(), eff.data_ptr(), labels.numel(), labels.shape[-1], ignore_index,
              vocab_total, _abi.status_word(labels.device).data_ptr(), _abi.stream())
    return eff


def local_lse_and_target(hidden2d, weight, labels_eff, vocab_start, ignore_index):
    """Per physical row: log-sum-exp over this weight's vocabulary rows and the target logit if owned."""
    m, k = hidden2d.shape
    v = weight.shape[0]
    tiles = _abi.lib().q3_linear_ce_tiles(v)
    dev = hidden2d.device
    part_max = torch.empty((m, tiles), device=dev, dtype=torch.float32)
    part_sum = torch.empty((m, tiles), device=dev, dtype=torch.float32)
    target = torch.empty(m, device=dev, dtype=torch.float32)
    lse = torch.empty(m, device=dev, dtype=torch.float32)
    _abi.call('q3_linear_ce_stats', hidden2d.data_ptr(), weight.data_ptr(), labels_eff.data_ptr(), part_max.data_ptr(),
              part_sum.data_ptr(), target.data_ptr(), m, v, k, vocab_start, ignore_index, _abi.dt(hidden2d.dtype),
              _abi.status_word(dev).data_ptr(), _abi.stream())
    _abi.call('q3_linear_ce_combine', part_max.data_ptr(), part_sum.data_ptr(), lse.data_ptr(), m, tiles, _abi.stream())
    return lse, target


def finish(lse, target, labels_eff, rows_per_rank, ignore_index, maximum=None, pack=None):
    """(losses, counts, means) per data rank; with maximum/pack given, lse is first set to maximum + log(pack[0])."""
    rows = lse.numel()
    world = rows // rows_per_rank
    dev = lse.device
    losses = torch.empty(rows, device=dev, dtype=torch.float32)
    counts = torch.empty(world, device=dev, dtype=torch.int32)
    means = torch.empty(world, device=dev, dtype=torch.float32)
    _abi.call('q3_linear_ce_finish', _abi.ptr(maximum), _abi.ptr(pack), lse.data_ptr(), target.data_ptr(),
              labels_eff.data_ptr(), losses.data_ptr(), counts.data_ptr(), means.data_ptr(), rows, rows_per_rank,
              ignore_index, _abi.status_word(dev).data_ptr(), _abi.stream())
    return losses, counts, means


def head_backward(hidden2d, weight, labels_eff, lse, ups, counts, rows_per_rank, vocab_start, ignore_index, chunk,
                  dw_dtype, need_dx=True, need_dw=True):
    """(dx fp32 [M,K] or None, dw [V,K] in dw_dtype or None) of the projection + loss, one vocabulary chunk at a time."""
    m, k = hidden2d.shape
    v = weight.shape[0]
    dev = hidden2d.device
    chunk = max(256, min(chunk, v) // 8 * 8)
    dx = torch.zeros((m, k), device=dev, dtype=torch.float32) if need_dx else None
    dw = torch.empty((v, k), device=dev, dtype=dw_dtype) if need_dw else None
    dz_buf = torch.empty((m, chunk), device=dev, dtype=hidden2d.dtype)
    ups = ups.contiguous().float()
    status = _abi.status_word(dev).data_ptr()
    for start in range(0, v, chunk):
        width = min(chunk, v - start)
        if width % 8:
            raise ValueError('Vocabulary slice widths must be multiples of 8')
        w_chunk = weight[start:start + width]
        dz = dz_buf.view(-1)[:m * width].view(m, width)
        _abi.call('q3_linear_ce_grad', hidden2d.data_ptr(), w_chunk.data_ptr(), labels_eff.data_ptr(), lse.data_ptr(),
                  ups.data_ptr(), counts.data_ptr(), dz.data_ptr(), m, width, k, vocab_start + start, rows_per_rank,
                  ignore_index, _abi.dt(hidden2d.dtype), status, _abi.stream())
        if need_dx:
            _abi.call('q3_gemm_acc_f32', dz.data_ptr(), width, 1, w_chunk.data_ptr(), k, 1, dx.data_ptr(), m, k, width,
                      _abi.dt(dz.dtype), status, _abi.stream())
        if need_dw:
            _abi.call('q3_gemm', dz.data_ptr(), 1, width, hidden2d.data_ptr(), k, 1, dw[start:start + width].data_ptr(),
                      width, k, m, _abi.dt(dz.dtype), _abi.dt(dw_dtype), status, _abi.stream())
    return dx, dw


class _FusedLinearCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, labels, ignore_index, chunk):
        if hidden.ndim != 3 or weight.ndim != 2 or hidden.shape[-1] != weight.shape[1] or labels.shape != hidden.shape[:2]:
            raise ValueError('Expected hidden [B,S,H], weight [V,H] and labels [B,S]')
        if (not hidden.is_cuda or hidden.device != weight.device or hidden.device != labels.device
                or hidden.dtype != weight.dtype or hidden.dtype not in (torch.bfloat16, torch.float16)
                or labels.dtype != torch.int64 or not hidden.is_contiguous() or not weight.is_contiguous()
                or not labels.is_contiguous()):
            raise ValueError('Matching contiguous BF16/FP16 CUDA hidden/weight and int64 labels required; no fallback')
        b, s, k = hidden.shape
        if s < 2 or k % 8:
            raise ValueError('At least 2 tokens per sequence and a hidden size that is a multiple of 8 required')
        v = weight.shape[0]
        h2 = hidden.view(b * s, k)
        eff = shifted_labels(labels, ignore_index, v)
        lse, target = local_lse_and_target(h2, weight, eff, 0, ignore_index)
        _, counts, means = finish(lse, target, eff, b * s, ignore_index)
        ctx.save_for_backward(h2, weight, eff, lse, counts)
        ctx.ignore, ctx.chunk, ctx.shape = ignore_index, chunk, hidden.shape
        return means[0].clone()

    @staticmethod
    def backward(ctx, dy):
        h2, weight, eff, lse, counts = ctx.saved_tensors
        dx, dw = head_backward(h2, weight, eff, lse, dy.reshape(1), counts, h2.shape[0], 0, ctx.ignore, ctx.chunk,
                               weight.dtype, ctx.needs_input_grad[0], ctx.needs_input_grad[1])
        if dx is not None:
            from .attention import cast_tensor
            dx = cast_tensor(dx, h2.dtype).view(ctx.shape)
        return dx, dw, None, None, None


def fused_linear_cross_entropy(hidden, weight, labels, *, ignore_index=-100, chunk=DEFAULT_CHUNK):
    return _FusedLinearCE.apply(hidden, weight, labels, ignore_index, chunk)
