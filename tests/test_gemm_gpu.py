"""GEMM parity: the tcgen05 tensor-core kernel in all three operand layouts (forward X*W^T, input gradient
dY*W, weight gradient dY^T*X), tails in M, N and K, fp32 output, the fused gate/up+SwiGLU kernel, and the
CUDA-core fallback; all against fp32 torch.mm on the same bf16-quantised inputs."""
import pytest
import torch

from helpers import close, randn, rel_l2
from oracle import ops as O

pytestmark = pytest.mark.gpu


def ref_mm(a, b):
    return a.float().cpu() @ b.float().cpu()


SHAPES = [(128, 256, 64), (256, 512, 128), (200, 264, 72), (1, 8, 8), (129, 1000, 520), (512, 4096, 4096), (300, 136, 1024)]


@pytest.mark.parametrize('M,N,K', SHAPES)
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16])
def test_forward_layout_tensor_cores(M, N, K, dtype):
    from qwen3_triton.kernels.linear import gemm_path, matmul
    x, w = randn((M, K), 1, dtype).cuda(), randn((N, K), 2, dtype).cuda()
    assert gemm_path(x, w.t()) == 'tcgen05'
    y = matmul(x, w.t())
    close(y, ref_mm(x, w.t()).to(dtype), scale=K ** 0.5, what='X*W^T')


@pytest.mark.parametrize('M,N,K', SHAPES)
def test_input_gradient_layout_tensor_cores(M, N, K):
    from qwen3_triton.kernels.linear import gemm_path, matmul
    dy, w = randn((M, K), 3, torch.bfloat16).cuda(), randn((K, N), 4, torch.bfloat16).cuda()   # B row-major [K,N]
    assert gemm_path(dy, w) == 'tcgen05'
    close(matmul(dy, w), ref_mm(dy, w).to(torch.bfloat16), scale=K ** 0.5, what='dY*W')


@pytest.mark.parametrize('M,N,K', SHAPES)
def test_weight_gradient_layout_tensor_cores(M, N, K):
    from qwen3_triton.kernels.linear import gemm_path, matmul
    # C[M,N] = A^T-view [M,K] * B [K,N] with both stored token-major, as dY^T * X
    dy, x = randn((K, M), 5, torch.bfloat16).cuda(), randn((K, N), 6, torch.bfloat16).cuda()
    if M % 8 == 0:
        assert gemm_path(dy.t(), x) == 'tcgen05'
    close(matmul(dy.t(), x), ref_mm(dy.t(), x).to(torch.bfloat16), scale=K ** 0.5, what='dY^T*X')


def test_fp32_output_and_determinism():
    from qwen3_triton.kernels.linear import matmul
    a, b = randn((384, 1536), 7, torch.bfloat16).cuda(), randn((1536, 520), 8, torch.bfloat16).cuda()
    c = matmul(a, b, output_dtype=torch.float32)
    assert c.dtype == torch.float32
    torch.testing.assert_close(c.cpu(), ref_mm(a, b), rtol=1e-4, atol=1e-2)
    assert torch.equal(c, matmul(a, b, output_dtype=torch.float32))


@pytest.mark.parametrize('M,N,K', [(128, 256, 64), (2048, 12288, 4096), (4096, 4096, 12288), (300, 1000, 520)])
def test_tile_hand_out_policies_agree_bit_for_bit(M, N, K):
    """Tiles drawn from the device counter (default) or taken with a fixed stride: every tile is computed whole by
    one CTA, so the result cannot depend on the policy; and the counters must come back to zero, launch after launch
    (forty launches in a row, then a different grid size)."""
    from qwen3_triton import _abi
    from qwen3_triton.kernels.linear import matmul
    a, b = randn((M, K), 11, torch.bfloat16).cuda(), randn((K, N), 12, torch.bfloat16).cuda()
    assert _abi.lib().q3_gemm_tile_schedule(-1) == 1
    drawn = [matmul(a, b) for _ in range(40)]
    small = matmul(a[:128], b)
    previous = _abi.lib().q3_gemm_tile_schedule(0)
    try:
        assert previous == 1
        strided, small_strided = matmul(a, b), matmul(a[:128], b)
    finally:
        _abi.lib().q3_gemm_tile_schedule(previous)
    assert all(torch.equal(d, strided) for d in drawn)
    assert torch.equal(small, small_strided)
    close(strided, ref_mm(a, b).to(torch.bfloat16), scale=K ** 0.5, what='A*B')
    assert _abi.read_status() == 0


@pytest.mark.parametrize('M,N,K', [(256, 256, 64), (2048, 4096, 4096), (384, 1000, 520), (129, 264, 72), (4096, 12288, 512)])
def test_cta_pairs_and_single_ctas_agree_bit_for_bit(M, N, K):
    """Two CTAs per 256-row tile (the default wherever there are two row tiles) against one CTA per 128-row tile: the
    same products accumulated over k in the same order, so all three layouts of a linear layer, the fp32 output, the
    fused gate/up kernel and the accumulating epilogue must agree exactly - odd row-tile counts (the second CTA of
    the last pair has no rows) and ragged N and K included."""
    from qwen3_triton import _abi
    from qwen3_triton.kernels.linear import matmul
    x, w = randn((M, K), 21, torch.bfloat16).cuda(), randn((N, K), 22, torch.bfloat16).cuda()
    dy = randn((M, N), 23, torch.bfloat16).cuda()

    def products():
        return [matmul(x, w.t()), matmul(dy, w), matmul(dy.t(), x), matmul(x, w.t(), output_dtype=torch.float32)]

    assert _abi.lib().q3_gemm_cta_pairs(-1) == 1
    paired = products()
    previous = _abi.lib().q3_gemm_cta_pairs(0)
    try:
        single = products()
    finally:
        _abi.lib().q3_gemm_cta_pairs(previous)
    for a, b in zip(paired, single):
        assert torch.equal(a, b), float((a.float() - b.float()).abs().max())
    close(paired[0], ref_mm(x, w.t()).to(torch.bfloat16), scale=K ** 0.5, what='X*W^T by pairs')
    close(paired[2], ref_mm(dy.t(), x).to(torch.bfloat16), scale=M ** 0.5, what='dY^T*X by pairs')
    assert _abi.read_status() == 0


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16])
@pytest.mark.parametrize('M,K,sizes', [(2048, 4096, (4096, 1024, 1024)), (300, 520, (192, 64, 320)), (129, 136, (448, 64)),
                                       (2048, 1024, (3072, 3072)), (2048, 4096, (12288, 12288)),
                                       (8192, 4096, (4096, 1024, 1024))])
def test_grouped_linear_layers_equal_separate_gemms(dtype, M, K, sizes):
    """q/k/v- and gate/up-style groups in one launch: forward outputs and weight gradients bit-identical to the
    single GEMMs (same tiles, same k order), the summed input gradient equal to fp32 math on the same operands."""
    from qwen3_triton import _abi
    from qwen3_triton.fused import linear_group_dgrad, linear_group_fwd, linear_group_wgrad, mm_nn, mm_nt, mm_tn
    x = randn((M, K), 41, dtype).cuda()
    ws = [randn((n, K), 42 + i, dtype, scale=0.05).cuda() for i, n in enumerate(sizes)]
    dys = [randn((M, n), 52 + i, dtype).cuda() for i, n in enumerate(sizes)]
    ys = linear_group_fwd(x, ws)
    for y, w in zip(ys, ws):
        assert torch.equal(y, mm_nt(x, w))
        close(y, ref_mm(x, w.t()).to(dtype), scale=K ** 0.5 * 0.05, what='grouped fwd')
    dws = linear_group_wgrad(dys, x)
    for dw, dy in zip(dws, dys):
        assert torch.equal(dw, mm_tn(dy, x))
    dx = linear_group_dgrad(dys, ws)
    ref = sum(ref_mm(dy, w) for dy, w in zip(dys, ws))
    close(dx, ref.to(dtype), scale=float(ref.abs().mean()) / 2, what='grouped dgrad')
    assert torch.equal(dx, linear_group_dgrad(dys, ws))
    assert _abi.read_status() == 0


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16])
@pytest.mark.parametrize('M,I,H', [(256, 512, 128), (200, 264, 72), (2048, 3072, 1024), (2048, 12288, 4096)])
def test_down_proj_input_gradient_fused_with_swiglu_backward(dtype, M, I, H):
    """dG, dU from the GEMM epilogue (dY never stored) against q3_gemm followed by q3_swiglu_bwd on the same
    operands: the epilogue rounds dY to the storage type first, so the two agree to the last bit or, where the
    compiler fuses the multiplies differently, to one unit in the last place; and against fp32 math."""
    from qwen3_triton import _abi
    from qwen3_triton.fused import mm_nn
    dm = randn((M, H), 91, dtype).cuda()
    wd = randn((H, I), 92, dtype, scale=0.05).cuda()
    g, u = randn((M, I), 93, dtype).cuda(), randn((M, I), 94, dtype).cuda()
    dg, du = torch.full_like(g, float('nan')), torch.full_like(u, float('nan'))
    _abi.call('q3_down_dgrad_swiglu_bwd', dm.data_ptr(), wd.data_ptr(), g.data_ptr(), u.data_ptr(), dg.data_ptr(),
              du.data_ptr(), M, I, H, _abi.dt(dtype), _abi.status_word(dm.device).data_ptr(), _abi.stream())
    dy = mm_nn(dm, wd)
    dg2, du2 = torch.empty_like(g), torch.empty_like(u)
    _abi.call('q3_swiglu_bwd', g.data_ptr(), u.data_ptr(), dy.data_ptr(), dg2.data_ptr(), du2.data_ptr(), g.numel(),
              _abi.dt(dtype), _abi.stream())
    ulp = 2 ** -7 if dtype == torch.bfloat16 else 2 ** -10
    for a, b in ((dg, dg2), (du, du2)):
        assert torch.isfinite(a).all()
        assert float(((a.float() - b.float()).abs() / (b.float().abs() + 1e-6)).max()) <= 2 * ulp
    dy32 = ref_mm(dm, wd).to(dtype).float()
    gf, uf = g.float().cpu(), u.float().cpu()
    sg = torch.sigmoid(gf)
    close(dg, (dy32 * uf * sg * (1 + gf * (1 - sg))).to(dtype), scale=H ** 0.5 * 0.05, what='dG')
    close(du, (dy32 * gf * sg).to(dtype), scale=H ** 0.5 * 0.05, what='dU')
    assert _abi.read_status() == 0


@pytest.mark.parametrize('out', [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize('M,N,K', [(256, 512, 128), (200, 264, 72), (2048, 4096, 1024)])
def test_accumulating_epilogue(out, M, N, K):
    """C += A*B with C in the input type (read, add in fp32, round once) or in fp32: against fp32 math on the same
    operands, in the input-gradient layout it is used for."""
    from qwen3_triton import _abi
    dtype = torch.float16 if out == torch.float16 else torch.bfloat16
    dy, w = randn((M, K), 31, dtype).cuda(), randn((K, N), 32, dtype).cuda()
    c0 = randn((M, N), 33, out, scale=K ** 0.5)
    c = c0.cuda().clone()
    _abi.call('q3_gemm_acc', dy.data_ptr(), K, 1, w.data_ptr(), N, 1, c.data_ptr(), M, N, K, _abi.dt(dtype), _abi.dt(out),
              _abi.status_word(c.device).data_ptr(), _abi.stream())
    ref = c0.float() + ref_mm(dy, w)
    if out == torch.float32:
        torch.testing.assert_close(c.cpu(), ref, rtol=1e-4, atol=2e-2)
    else:
        close(c, ref.to(out), scale=K ** 0.5, what='C += A*B')


@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16])
@pytest.mark.parametrize('M,N,K', [(1, 1, 1), (17, 129, 33), (65, 7, 257)])
def test_fallback_path_odd_shapes_and_fp32(dtype, M, N, K):
    from qwen3_triton.kernels.linear import gemm_path, matmul
    a, b = randn((M, K), 9, dtype).cuda(), randn((K, N), 10, dtype).cuda()
    assert gemm_path(a, b) == 'simt'
    close(matmul(a, b), ref_mm(a, b).to(dtype), scale=K ** 0.5)
    close(matmul(a.t().contiguous().t(), b.t().contiguous().t()), ref_mm(a, b).to(dtype), scale=K ** 0.5)


def test_tensor_core_and_fallback_agree():
    from qwen3_triton import _abi
    from qwen3_triton.kernels.linear import matmul
    a, b = randn((256, 512), 11, torch.bfloat16).cuda(), randn((512, 384), 12, torch.bfloat16).cuda()
    tc = matmul(a, b, output_dtype=torch.float32)
    a32, b32 = a.float(), b.float()
    simt = matmul(a32, b32)                 # fp32 operands take the CUDA-core kernel
    torch.testing.assert_close(tc, simt, rtol=1e-4, atol=1e-3)


@pytest.mark.parametrize('shape', [(2, 17, 256), (4, 128, 1024)])
def test_linear_autograd(shape):
    from qwen3_triton.kernels.linear import linear
    K, N = shape[-1], 520
    x, w, dy = randn(shape, 13, torch.bfloat16), randn((N, K), 14, torch.bfloat16, 0.05), randn((*shape[:-1], N), 15, torch.bfloat16)
    xg, wg = x.cuda().requires_grad_(True), w.cuda().requires_grad_(True)
    y = linear(xg, wg)
    y.backward(dy.cuda())
    close(y, O.linear(x, w).to(torch.bfloat16), what='y')
    close(xg.grad, (dy.float().reshape(-1, N) @ w.float()).reshape(shape).to(torch.bfloat16), what='dx')
    close(wg.grad, (dy.float().reshape(-1, N).t() @ x.float().reshape(-1, K)).to(torch.bfloat16), what='dw')
    with pytest.raises(ValueError):
        linear(xg.transpose(0, 1), wg)


@pytest.mark.parametrize('M,N,K', [(128, 128, 64), (200, 344, 256), (512, 1536, 1024), (64, 688, 256), (2048, 12288, 4096)])
def test_fused_gate_up_swiglu(M, N, K):
    from qwen3_triton import _abi
    from qwen3_triton.kernels.mlp import gate_up_swiglu
    from ops.triton.gate_up_swiglu import gate_up_swiglu_triton
    dt = torch.bfloat16
    x, wg, wu, dy = randn((M, K), 16, dt), randn((N, K), 17, dt, 0.05), randn((N, K), 18, dt, 0.05), randn((M, N), 19, dt)
    xg, g_, u_ = x.cuda().requires_grad_(True), wg.cuda().requires_grad_(True), wu.cuda().requires_grad_(True)
    assert _abi.lib().q3_gate_up_path(xg.data_ptr(), g_.data_ptr(), u_.data_ptr(), xg.data_ptr(), xg.data_ptr(),
                                      xg.data_ptr(), M, N, K, _abi.Q3_BF16) == 1
    y = gate_up_swiglu(xg, g_, u_)
    y.backward(dy.cuda())
    gate, up = O.linear(x, wg), O.linear(x, wu)
    close(y, O.swiglu(gate.to(dt), up.to(dt)).to(dt), what='y')
    xr, gr, ur = x.float().requires_grad_(True), wg.float().requires_grad_(True), wu.float().requires_grad_(True)
    (torch.nn.functional.silu(xr @ gr.t()) * (xr @ ur.t())).backward(dy.float())
    close(xg.grad, xr.grad.to(dt), what='dx')
    close(g_.grad, gr.grad.to(dt), what='dWg')
    close(u_.grad, ur.grad.to(dt), what='dWu')
    close(gate_up_swiglu_triton(x.cuda(), wg.cuda(), wu.cuda()), y, what='ops.triton')


# ------------------------------------------------------------------------------------------------------------------
# The GEMM shapes of the Qwen3-8B training step (tokens M = 2048 per GPU, or 8192 for the 4-layer slice):
# attention projections 4096 x 4096, gate/up 12288 x 4096, down 4096 x 12288 and the vocabulary head 151936 x 4096
# (593.5 tiles of 256 columns: the half-full last tile; 2374 k-blocks as a contraction). The GPU computes the whole
# product; the fp32 CPU reference is taken on every 37th output row (three or more rows of every 128-row tile, all
# columns, so every output tile is touched) plus the last row.
LAYER_SHAPES = [(2048, 4096, 4096), (2048, 12288, 4096), (2048, 4096, 12288), (2048, 151936, 4096),
                (8192, 4096, 4096), (8192, 12288, 4096), (8192, 4096, 12288), (8192, 151936, 4096)]
_operands = {}


def _operand(shape, seed, scale=1.0):
    """bf16 operand, generated once per (shape, seed) on the CPU and kept on both sides."""
    key = (shape, seed)
    if key not in _operands:
        if len(_operands) > 6:
            _operands.clear()
        host = randn(shape, seed, torch.bfloat16, scale)
        _operands[key] = (host, host.cuda())
    return _operands[key]


def _rows(n):
    idx = torch.arange(0, n, 37)
    return torch.cat([idx, torch.tensor([n - 1])]) if idx[-1] != n - 1 else idx


@pytest.mark.parametrize('M,N,K', LAYER_SHAPES)
def test_layer_shapes_forward(M, N, K):
    from qwen3_triton.kernels.linear import gemm_path, matmul
    (x, xd), (w, wd) = _operand((M, K), 61), _operand((N, K), 62, 0.02)
    assert gemm_path(xd, wd.t()) == 'tcgen05'
    y = matmul(xd, wd.t())
    r = _rows(M)
    close(y[r.cuda()], (x[r].float() @ w.float().t()).to(torch.bfloat16), what='X*W^T')


@pytest.mark.parametrize('M,N,K', LAYER_SHAPES)
def test_layer_shapes_input_gradient(M, N, K):
    """dX [M,K] = dY [M,N] * W [N,K]: the contraction runs over the layer's output width N."""
    from qwen3_triton.kernels.linear import gemm_path, matmul
    (dy, dyd), (w, wd) = _operand((M, N), 63), _operand((N, K), 62, 0.02)
    assert gemm_path(dyd, wd) == 'tcgen05'
    dx = matmul(dyd, wd)
    r = _rows(M)
    close(dx[r.cuda()], (dy[r].float() @ w.float()).to(torch.bfloat16), what='dY*W')


@pytest.mark.parametrize('M,N,K', LAYER_SHAPES)
@pytest.mark.parametrize('out', [torch.bfloat16, torch.float32])
def test_layer_shapes_weight_gradient(M, N, K, out):
    """dW [N,K] = dY [M,N]^T * X [M,K]: both operands token-major, contraction over the tokens; bf16 result as the
    training step stores it and fp32 result as the vocabulary head accumulates it."""
    from qwen3_triton.kernels.linear import gemm_path, matmul
    if out == torch.float32 and N != 151936:
        pytest.skip('fp32 weight gradients are used for the vocabulary head only')
    (dy, dyd), (x, xd) = _operand((M, N), 63), _operand((M, K), 61)
    assert gemm_path(dyd.t(), xd) == 'tcgen05'
    dw = matmul(dyd.t(), xd, output_dtype=out)
    r = _rows(N)
    ref = dy[:, r].float().t() @ x.float()
    if out == torch.float32:
        torch.testing.assert_close(dw[r.cuda()].cpu(), ref, rtol=1e-3, atol=1e-3 * float(ref.abs().mean()))
        assert rel_l2(dw[r.cuda()], ref) < 1e-4
    else:
        close(dw[r.cuda()], ref.to(torch.bfloat16), what='dY^T*X')
