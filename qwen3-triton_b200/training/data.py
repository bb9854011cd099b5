"""Pre-tokenised corpus as fixed-length blocks, on the host and resident on the GPU.

A corpus file is a flat array of little-endian uint32 token ids; block b is tokens [b*seq, (b+1)*seq) and the tail that
does not fill a block is dropped. Evaluation visits blocks in file order; training visits block
((i + offset) * stride + seed) mod n, where stride is the first odd number >= 104729 coprime to n - a full-period
permutation that needs no shuffle buffer and is reproducible from (seed, offset) alone. Same class name, arguments and
indexing as the reference's training/data.py:9-28, so a run can be resumed or compared block for block.

`DeviceBlocks` is the B200 form: the corpus is uploaded once (4 bytes per token; a 10-billion-token corpus takes 40 of
the 180 GB) and every batch is produced by two small kernels of the CUDA library - the block order
(q3_block_order) and the gather that widens uint32 to the int64 ids the embedding takes (q3_token_blocks) - so a
training step has no host indexing and no host-to-device copy.
"""
import math

import numpy as np
import torch

FIRST_STRIDE = 104729      # the 10000th prime; only its coprimality to the block count matters


def coprime_stride(blocks, start=FIRST_STRIDE):
    """Smallest stride of the form start + 2k that shares no factor with the number of blocks."""
    stride = start
    while math.gcd(stride, blocks) != 1:
        stride += 2
    return stride


def block_for(i, *, blocks, stride, seed, offset, training):
    """Index of the block served at position i."""
    return ((i + offset) * stride + seed) % blocks if training else i


class Blocks(torch.utils.data.Dataset):
    """Host view: `dataset[i]` is an int64 tensor of `seq` token ids read through a memory map."""

    def __init__(self, path, seq, offset=0, training=False, seed=20261102):
        if type(seq) is not int or seq < 2:
            raise ValueError('Sequence length must be an integer >= 2')
        self.data = np.memmap(path, dtype='<u4', mode='r')
        self.seq, self.offset, self.training, self.seed = seq, offset, training, seed
        self.n = self.data.shape[0] // seq
        if self.n < 1:
            raise ValueError('Corpus shorter than one sequence')
        self.stride = coprime_stride(self.n)

    def __len__(self):
        return self.n

    def block_index(self, i):
        return block_for(i, blocks=self.n, stride=self.stride, seed=self.seed, offset=self.offset,
                         training=self.training)

    def __getitem__(self, i):
        first = self.block_index(i) * self.seq
        return torch.from_numpy(self.data[first:first + self.seq].astype(np.int64))


class DeviceBlocks:
    """The same blocks served from a copy of the corpus in GPU memory. `batch(first, count)` returns the int64 ids
    [count, seq] of positions first .. first+count-1, bit-identical to stacking `Blocks[i]` for those positions."""

    def __init__(self, blocks, device='cuda'):
        from qwen3_triton import _abi
        self._abi = _abi
        self.source = blocks
        self.device = torch.device(device)
        usable = blocks.n * blocks.seq
        # uint32 has no arithmetic in torch; the buffer is only ever read by the gather kernel, so carry it as int32
        host = torch.from_numpy(np.ascontiguousarray(blocks.data[:usable]).view(np.int32))
        self.corpus = host.to(self.device)
        self.tokens = usable

    def __len__(self):
        return self.source.n

    def order(self, first, count):
        """Block indices of positions first .. first+count-1 (int64 on the device)."""
        src, abi = self.source, self._abi
        out = torch.empty(count, device=self.device, dtype=torch.int64)
        with torch.cuda.device(self.device):
            abi.call('q3_block_order', out.data_ptr(), first, count, src.offset, src.stride, src.seed, src.n,
                     int(bool(src.training)), abi.stream())
        return out

    def batch(self, first, count):
        if count < 1 or first < 0 or (not self.source.training and first + count > self.source.n):
            raise IndexError('Positions outside the corpus')
        abi = self._abi
        index = self.order(first, count)
        ids = torch.empty((count, self.source.seq), device=self.device, dtype=torch.int64)
        with torch.cuda.device(self.device):
            abi.call('q3_token_blocks', self.corpus.data_ptr(), self.tokens, index.data_ptr(), ids.data_ptr(), count,
                     self.source.seq, abi.status_word(self.device).data_ptr(), abi.stream())
        return ids
