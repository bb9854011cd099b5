"""q3_reduce_scatter_pull on one GPU: the kernel takes one pointer per rank, and nothing in it cares which GPU a
pointer lives on, so `world` local buffers stand in for the peers' staging buffers. Checked against the fp32 sum in
rank order computed by torch (bit-exact: same upcast, same order, one multiplication by the scale), for every world
size the entry point takes, ragged counts, both 16-bit types, and its argument checks. The two-rank run over real
peer mappings is in test_multi_gpu.py."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _pull(buffers, first, count, scale, dtype):
    from qwen3_triton import _abi
    table = (ctypes.c_void_p * len(buffers))(*[b.data_ptr() for b in buffers])
    out = torch.full((count,), float('nan'), device='cuda')
    _abi.call('q3_reduce_scatter_pull', table, len(buffers), out.data_ptr(), first, count, scale, _abi.dt(dtype),
              _abi.stream())
    return out


def _expected(buffers, first, count, scale):
    total = buffers[0][first:first + count].float()
    for b in buffers[1:]:
        total = total + b[first:first + count].float()
    return total * scale


@pytest.mark.parametrize('world', [2, 4, 8])
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16])
@pytest.mark.parametrize('count', [5, 8, 4096 + 11, 3 * 1024 * 1024 + 64])
def test_pull_equals_ordered_fp32_sum(world, dtype, count):
    g = torch.Generator(device='cuda').manual_seed(world * 1000 + count % 997)
    pitch = (count + 7) // 8 * 8                    # a rank's rows start on a 16-byte boundary
    buffers = [(torch.randn(world * pitch, device='cuda', generator=g) * (r + 1)).to(dtype) for r in range(world)]
    for rank in (0, world - 1):
        got = _pull(buffers, rank * pitch, count, 1.0 / world, dtype)
        assert torch.equal(got, _expected(buffers, rank * pitch, count, 1.0 / world))
    got = _pull(buffers, pitch, count, 1.0, dtype)
    assert torch.equal(got, _expected(buffers, pitch, count, 1.0))


def test_pull_rejects_bad_arguments():
    from qwen3_triton import _abi
    a = torch.zeros(64, device='cuda', dtype=torch.bfloat16)
    out = torch.zeros(64, device='cuda')
    table3 = (ctypes.c_void_p * 3)(a.data_ptr(), a.data_ptr(), a.data_ptr())
    table2 = (ctypes.c_void_p * 2)(a.data_ptr(), a.data_ptr())
    lib = _abi.lib()
    s = _abi.stream()
    assert lib.q3_reduce_scatter_pull(table3, 3, out.data_ptr(), 0, 64, 1.0, _abi.dt(torch.bfloat16), s) < 0   # world
    assert lib.q3_reduce_scatter_pull(table2, 2, out.data_ptr(), 0, 64, 1.0, _abi.dt(torch.float32), s) < 0    # dtype
    assert lib.q3_reduce_scatter_pull(table2, 2, out.data_ptr(), 3, 64, 1.0, _abi.dt(torch.bfloat16), s) < 0   # alignment
    assert lib.q3_reduce_scatter_pull(table2, 2, None, 0, 64, 1.0, _abi.dt(torch.bfloat16), s) < 0             # null
    assert lib.q3_reduce_scatter_pull(table2, 2, out.data_ptr(), 0, 0, 1.0, _abi.dt(torch.bfloat16), s) == 0   # empty
    torch.cuda.synchronize()
