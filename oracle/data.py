"""CPU restatement of the reference's data path and validation arithmetic. TEST INFRASTRUCTURE ONLY: imported by
tests/ (and nothing in the product), it is the checker for training/data.py, training/evaluation.py and
qwen3_triton/runtime/metrics.py of the package.

Restates, with plain Python integers and numpy / torch CPU ops:
  * training/data.py:9-28   - block count (tail dropped), coprime stride search from 104729 in steps of 2, the
                               training permutation ((i + offset) * stride + seed) mod n, uint32 -> int64 widening;
  * training/evaluation.py:7-26 - the round-robin validation partition with padded (masked) tail and the shifted,
                               summed NLL with its token count;
  * qwen3_triton/runtime/metrics.py:8-17 - totals += (loss * tokens, tokens) in fp64 with separate roundings.
Pinned by tests/golden/data.npz, which tests/golden/make_golden.py generates by importing the reference itself.
"""
import math

import numpy as np
import torch


def stride_for(n):
    stride = 104729
    while math.gcd(stride, n) != 1:
        stride += 2
    return stride


def block_order(n, count, *, seed, offset=0, training=True, first=0):
    stride = stride_for(n)
    return [((first + i + offset) * stride + seed) % n if training else first + i for i in range(count)]


def read_block(tokens_u32, seq, index):
    """tokens_u32: 1-D numpy array of dtype '<u4'."""
    return torch.from_numpy(tokens_u32[index * seq:(index + 1) * seq].astype(np.int64))


def partition(size, rank, world, batch):
    """[(block indices with None for padding)] per forward of this rank."""
    width = world * batch
    out = []
    for start in range(0, size, width):
        idx = [start + rank * batch + j for j in range(batch)]
        out.append([i if i < size else None for i in idx])
    return out


def shifted_nll(logits, ids, valid):
    labels = ids[:, 1:].clone()
    labels[~valid] = -100
    total = torch.nn.functional.cross_entropy(logits[:, :-1].double().reshape(-1, logits.shape[-1]), labels.reshape(-1),
                                              ignore_index=-100, reduction='sum')
    return float(total), int(valid.sum()) * (ids.shape[1] - 1)


def accumulate(totals, loss_f32, tokens):
    """totals: [nll, count] Python floats (fp64)."""
    return [totals[0] + float(np.float64(np.float32(loss_f32)) * np.float64(tokens)), totals[1] + float(tokens)]
