"""Vocabulary-shard-local cross-entropy pieces of the vocab-parallel head
(reference qwen3_triton/kernels/vocab_ce.py:78-114). Collectives live in training/vocab_parallel.py."""
import torch

from .. import _abi


def local_statistics(logits, labels, sequence, start, *, vocab_total=None, ignore=-100):
    """Per shifted row: log-sum-exp over this shard's columns and the target logit if the shard owns it."""
    rows, v = logits.shape
    n = labels.numel() // sequence * (sequence - 1)
    lse = torch.empty(n, device=logits.device, dtype=torch.float32)
    target = torch.empty_like(lse)
    total = vocab_total if vocab_total is not None else (1 << 62)
    _abi.call('q3_ce_local_rows', logits.data_ptr(), labels.data_ptr(), lse.data_ptr(), target.data_ptr(), rows,
              sequence, v, start, total, ignore, _abi.dt(logits.dtype), _abi.status_word(logits.device).data_ptr(),
              _abi.stream())
    return lse, target


def packed_statistics(local_lse, maximum, target):
    pack = torch.empty((2, local_lse.numel()), device=local_lse.device, dtype=torch.float32)
    _abi.call('q3_vce_pack', local_lse.data_ptr(), maximum.data_ptr(), target.data_ptr(), pack.data_ptr(),
              local_lse.numel(), _abi.stream())
    return pack


def finish_statistics(maximum, pack, labels, rows_per_rank, sequence, world, ignore):
    n = maximum.numel()
    lse = torch.empty_like(maximum)
    losses = torch.empty_like(maximum)
    counts = torch.empty(world, device=maximum.device, dtype=torch.int32)
    means = torch.empty(world, device=maximum.device, dtype=torch.float32)
    _abi.call('q3_vce_finish', maximum.data_ptr(), pack.data_ptr(), labels.data_ptr(), lse.data_ptr(),
              losses.data_ptr(), counts.data_ptr(), means.data_ptr(), n, rows_per_rank, sequence, world, ignore,
              _abi.status_word(maximum.device).data_ptr(), _abi.stream())
    return lse, counts, means


def logit_gradient(logits, labels, lse, counts, up, rows_per_rank, sequence, start, ignore, *, vocab_total=None):
    dz = torch.empty_like(logits)
    total = vocab_total if vocab_total is not None else (1 << 62)
    up = up.contiguous().float()
    _abi.call('q3_ce_grad', logits.data_ptr(), labels.data_ptr(), lse.data_ptr(), counts.data_ptr(), up.data_ptr(),
              dz.data_ptr(), logits.shape[0], rows_per_rank, sequence, logits.shape[1], start, total, ignore,
              _abi.dt(logits.dtype), _abi.stream())
    return dz


def accumulate_weight_gradient(partial, out, world, first):
    _abi.call('q3_vce_accumulate', partial.data_ptr(), _abi.dt(partial.dtype), out.data_ptr(), out.numel(), world,
              int(bool(first)), _abi.stream())
