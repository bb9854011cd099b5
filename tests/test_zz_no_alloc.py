"""q3_rmsnorm_bwd_noalloc: the RMSNorm backward for callers that must not allocate device memory at call time
(allocator callbacks, hosts with a fixed HBM plan, latency-critical loops). Its scratch is a fixed device
array inside the library, so this test drives it straight through the C ABI with caller-owned inputs and
outputs only, and compares it with the workspace-taking entry point on two consecutive calls (the second
call re-uses the scratch the first one left behind). Collected last on purpose."""
import pytest
import torch

from helpers import randn

pytestmark = pytest.mark.gpu


def run_pair(rows, H, dtype, seed):
    from qwen3_triton import _abi
    lib = _abi.lib()
    x, w, dy = (randn(s, seed + i, dtype).cuda() for i, s in enumerate([(rows, H), (H,), (rows, H)]))
    y = torch.empty_like(x)
    inv = torch.empty(rows, device='cuda', dtype=torch.float32)
    _abi.call('q3_rmsnorm_fwd', x.data_ptr(), w.data_ptr(), y.data_ptr(), inv.data_ptr(), rows, H, 1e-6,
              _abi.dt(dtype), _abi.stream())
    dx_ref, dw_ref = torch.empty_like(x), torch.empty_like(w)
    ws = _abi.workspace(lib.q3_rmsnorm_bwd_workspace_bytes(rows, H), 'cuda')
    _abi.call('q3_rmsnorm_bwd', x.data_ptr(), w.data_ptr(), dy.data_ptr(), inv.data_ptr(), dx_ref.data_ptr(),
              dw_ref.data_ptr(), ws.data_ptr(), ws.numel(), rows, H, _abi.dt(dtype), _abi.stream())
    dx = torch.full_like(x, float('nan'))
    dw = torch.full_like(w, float('nan'))
    args = (x.data_ptr(), w.data_ptr(), dy.data_ptr(), inv.data_ptr(), dx.data_ptr(), dw.data_ptr(), rows, H,
            _abi.dt(dtype), _abi.stream())
    # First call of this shape: the driver may load the kernel (and, on a device's very first call, the module
    # that holds the scratch array) - set-up that belongs outside a caller's no-allocation region.
    _abi.call('q3_rmsnorm_bwd_noalloc', *args)
    torch.cuda.synchronize()
    dx.fill_(float('nan'))
    dw.fill_(float('nan'))
    torch.cuda.synchronize()
    # Steady state: neither torch's allocator nor the driver (cudaMalloc inside the library would show here)
    # hands out a byte during the call.
    before, free_before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
    _abi.call('q3_rmsnorm_bwd_noalloc', *args)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    assert torch.cuda.mem_get_info()[0] == free_before
    tol = 2e-2 if dtype != torch.float32 else 2e-4
    torch.testing.assert_close(dx, dx_ref, rtol=0, atol=0)           # same kernel, same per-row math
    torch.testing.assert_close(dw.float(), dw_ref.float(), rtol=tol, atol=tol * float(dw_ref.float().abs().mean()))


def test_two_calls_in_a_row_match_the_workspace_entry_point():
    run_pair(4096, 4096, torch.bfloat16, 100)     # fills many partial rows of the shared scratch
    run_pair(37, 256, torch.bfloat16, 200)        # smaller call right after: stale scratch must not leak in
    run_pair(513, 1000, torch.float32, 300)


def test_rejects_rows_wider_than_the_fixed_scratch():
    from qwen3_triton import _abi
    lib = _abi.lib()
    x = torch.zeros(2, 8192, device='cuda', dtype=torch.bfloat16)
    w = torch.zeros(8192, device='cuda', dtype=torch.bfloat16)
    inv = torch.zeros(2, device='cuda')
    rc = lib.q3_rmsnorm_bwd_noalloc(x.data_ptr(), w.data_ptr(), x.data_ptr(), inv.data_ptr(), x.data_ptr(),
                                    w.data_ptr(), 2, 8192, _abi.Q3_BF16, _abi.stream())
    assert rc == -8
    assert b"no-allocation" in lib.q3_error_string(rc)
