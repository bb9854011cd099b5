"""Validation statistics kept on the GPU in fp64 (reference qwen3_triton/runtime/metrics.py:8-17): the running pair
(summed NLL, token count) never visits the host between batches, and the update is one tiny kernel of the CUDA
library with the multiply and the add rounded separately, as the host arithmetic it replaces."""
import torch

from .. import _abi


def accumulate_validation(totals, loss, tokens):
    """totals[0] += loss * tokens; totals[1] += tokens. `totals`: two fp64 values on the GPU; `loss`: this rank's
    token-mean loss (a one-element fp32 CUDA tensor); `tokens`: how many tokens that mean covers (0 = nothing to add)."""
    if (totals.numel() != 2 or not totals.is_cuda or totals.dtype != torch.float64 or totals.device != loss.device
            or loss.numel() != 1):
        raise ValueError('Two GPU FP64 totals and a local scalar loss required')
    if tokens < 0:
        raise ValueError('Nonnegative token count required')
    if tokens:
        value = loss.detach().reshape(1)
        value = value if value.dtype == torch.float32 else value.float()
        with torch.cuda.device(totals.device):
            _abi.call('q3_validation_accumulate', value.data_ptr(), totals.data_ptr(), int(tokens), _abi.stream())
