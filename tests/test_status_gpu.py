"""The device status word and the bounded waits. Kernels of this library never trap: a wait that runs out raises a
CTA-wide flag, the CTA leaves in an orderly way and Q3_STATUS_WAIT_TIMEOUT appears in the caller's status word.
The self-test entry makes that happen harmlessly (a barrier nothing arrives at, a 1 ms limit); afterwards the
context must be intact and the tensor-core kernels must still work."""
import pytest
import torch

from helpers import close, randn

pytestmark = pytest.mark.gpu


def test_wait_that_runs_out_sets_the_status_bit_and_returns():
    from qwen3_triton import _abi
    from qwen3_triton.kernels.linear import matmul
    status = torch.zeros(1, dtype=torch.int32, device='cuda')
    outcome = torch.full((2,), -1, dtype=torch.int32, device='cuda')
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    _abi.call('q3_selftest_wait_timeout', 1_000_000, status.data_ptr(), outcome.data_ptr(), _abi.stream())
    end.record()
    torch.cuda.synchronize()                      # returns: the kernel did not hang
    assert int(status.item()) == _abi.STATUS_WAIT_TIMEOUT
    assert outcome.tolist() == [0, 0]             # warp 0 by its limit, warp 1 through the abort flag
    assert 0.5 < start.elapsed_time(end) < 500.0  # about the 1 ms limit, nowhere near the 2 s default
    # the context is intact: a tensor-core GEMM right after gives the right answer and a clean status
    a, b = randn((256, 512), 1, torch.bfloat16), randn((512, 384), 2, torch.bfloat16)
    close(matmul(a.cuda(), b.cuda()), (a.float() @ b.float()).to(torch.bfloat16), what='gemm after timeout')
    assert _abi.read_status() == 0


def test_selftest_rejects_unbounded_limits():
    from qwen3_triton import _abi
    status = torch.zeros(1, dtype=torch.int32, device='cuda')
    assert _abi.lib().q3_selftest_wait_timeout(10 ** 10, status.data_ptr(), None, _abi.stream()) != 0
    assert _abi.lib().q3_selftest_wait_timeout(1_000_000, None, None, _abi.stream()) != 0


def test_raise_on_status_names_the_violation():
    from qwen3_triton import _abi
    word = _abi.status_word('cuda')
    word.fill_(_abi.STATUS_WAIT_TIMEOUT | _abi.STATUS_LABEL_RANGE)
    with pytest.raises(_abi.Q3Error, match='wait timed out'):
        _abi.raise_on_status()
    assert _abi.read_status() == 0                # reading clears
