"""FSDP pack/unpack kernels (q3_multi_copy) against torch's own copy-in, split_with_sizes_copy and _chunk_cat:
bit-exact, including ragged chunk padding, unaligned sizes and the routed torch.ops.fsdp.* entry points."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device('cuda', 0)


@pytest.mark.parametrize('src_dtype', [torch.float32, torch.bfloat16])
@pytest.mark.parametrize('numels', [[4096 * 3, 128, 4096 * 1024 + 4], [5, 12, 1, 4099]])
def test_copy_in_matches_foreach_copy(src_dtype, numels):
    from qwen3_triton.runtime import ops
    g = torch.Generator(device='cuda').manual_seed(1)
    world, rank = 4, 3
    shards = [torch.randn(n, device=_dev(), generator=g).to(src_dtype) for n in numels]
    total = sum(numels)
    out = torch.zeros(world * total, device=_dev(), dtype=torch.bfloat16)
    ref = torch.zeros_like(out)
    torch._foreach_copy_(list(torch.split(ref.narrow(0, total * rank, total), numels)), shards)
    inp, whole = ops.all_gather_copy_in(shards, out, numels, total, rank)
    assert whole.data_ptr() == out.data_ptr() and inp.data_ptr() == out.data_ptr() + total * rank * 2
    assert torch.equal(out, ref)


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float32])
@pytest.mark.parametrize('sizes', [[4096 * 512, 128, 4096 * 128], [5, 12, 1, 4099]])
def test_split_copy_matches_aten(dtype, sizes):
    from qwen3_triton.runtime import ops
    g = torch.Generator(device='cuda').manual_seed(2)
    world = 8
    gathered = torch.randn(world, sum(sizes), device=_dev(), generator=g).to(dtype)
    outs = [torch.full((world, n), 7.0, device=_dev(), dtype=dtype) for n in sizes]
    refs = [torch.empty_like(o) for o in outs]
    torch.split_with_sizes_copy(gathered, sizes, dim=1, out=refs)
    ops.split_with_sizes_copy(gathered, sizes, dim=1, out=outs)
    for o, r in zip(outs, refs):
        assert torch.equal(o, r)


@pytest.mark.parametrize('shapes', [[(4096, 1024), (128,), (4096, 512), (1024, 4096)],
                                    [(6, 3), (5, 2), (9,), (1, 4), (151, 7)]])
@pytest.mark.parametrize('world', [2, 8])
def test_chunk_cat_matches_aten(shapes, world):
    from qwen3_triton.runtime import ops
    g = torch.Generator(device='cuda').manual_seed(3)
    grads = [torch.randn(s, device=_dev(), generator=g).to(torch.bfloat16) for s in shapes]
    _, cols = ops.plan_chunk_cat(shapes, [0] * len(shapes), 0, 4, world)
    ref = torch.empty(world, cols, device=_dev(), dtype=torch.float32)
    torch._chunk_cat(grads, 0, world, out=ref)
    got = torch.full((world, cols), float('nan'), device=_dev(), dtype=torch.float32)
    ops.chunk_cat(grads, 0, world, got)
    assert torch.equal(got, ref)


def test_routed_fsdp_ops_use_the_kernel():
    from qwen3_triton import _abi
    from qwen3_triton.runtime import ops
    ops.install_fsdp_pack_kernels()
    ops.install_fsdp_pack_kernels()
    seen = []
    real = _abi.call

    def spy(name, *a):
        seen.append(name)
        return real(name, *a)

    _abi.call = spy
    try:
        g = torch.Generator(device='cuda').manual_seed(4)
        grads = [torch.randn(64, 32, device=_dev(), generator=g).to(torch.bfloat16) for _ in range(3)]
        out = torch.empty(4, 3 * 16 * 32, device=_dev())
        torch.ops.fsdp.chunk_cat(grads, dim=0, num_chunks=4, out=out)
        ref = torch.empty_like(out)
        torch._chunk_cat(grads, 0, 4, out=ref)
        assert torch.equal(out, ref)
        shards = [torch.randn(n, device=_dev(), generator=g) for n in (256, 100)]
        buf = torch.zeros(2 * 356, device=_dev(), dtype=torch.bfloat16)
        inp, _ = torch.ops.fsdp.all_gather_copy_in(shards, buf, [256, 100], 356, 1)
        assert torch.equal(inp, torch.cat(shards).to(torch.bfloat16))
        outs = [torch.empty(2, 256, device=_dev(), dtype=torch.bfloat16), torch.empty(2, 100, device=_dev(), dtype=torch.bfloat16)]
        torch.ops.fsdp.split_with_sizes_copy(buf.view(2, -1), [256, 100], dim=1, out=outs)
        assert torch.equal(outs[1], buf.view(2, -1)[:, 256:])
    finally:
        _abi.call = real
    assert seen.count('q3_multi_copy') == 3
