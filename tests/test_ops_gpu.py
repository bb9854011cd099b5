"""Parity of the bandwidth-bound CUDA operators with the oracle (and, at the fixture shapes, with the
reference's own outputs), through the public operator API -> C ABI. Shapes include odd tails (17, 129)
and widths that force the scalar path."""
import pytest
import torch

import recipe
from helpers import close, randn
from oracle import ops as O

pytestmark = pytest.mark.gpu
DTYPES = [torch.bfloat16, torch.float16, torch.float32]


def dev(t, dtype=None):
    t = t.to(dtype) if dtype is not None else t
    return t.cuda().contiguous()


@pytest.mark.parametrize('dtype', DTYPES)
@pytest.mark.parametrize('shape', [(1, 1, 128), (2, 17, 2048), (1, 129, 96), (3, 5, 4096), (2, 3, 33), (1, 2, 8192)])
def test_rms_norm(dtype, shape):
    from qwen3_triton.kernels.norm import rms_norm
    from ops.triton.rms_norm import rms_norm_triton
    x = randn(shape, 1, dtype)
    w = (1 + 0.1 * randn(shape[-1:], 2)).to(dtype)
    dy = randn(shape, 3, dtype)
    xg, wg = dev(x).requires_grad_(True), dev(w).requires_grad_(True)
    snapshot = xg.detach().clone()
    y = rms_norm(xg, wg, 1e-6)
    y.backward(dev(dy))
    close(y, O.rms_norm(x, w).to(dtype), what='y')
    dx, dw = O.rms_norm_backward(x, w, dy)
    close(xg.grad, dx.to(dtype), what='dx')
    close(wg.grad, dw.to(dtype), scale=float(dw.abs().mean()), what='dw')
    assert torch.equal(xg.detach(), snapshot)
    close(rms_norm_triton(dev(x), dev(w), 1e-6), O.rms_norm(x, w).to(dtype), what='ops.triton')


def test_rms_norm_golden(golden_ops):
    from qwen3_triton.kernels.norm import rms_norm
    d = recipe.op_inputs()
    x, w = dev(d['norm_x']).requires_grad_(True), dev(d['norm_w']).requires_grad_(True)
    y = rms_norm(x, w, 1e-6)
    y.backward(dev(d['norm_dy']))
    close(y, golden_ops['rms_norm'])
    close(x.grad, golden_ops['rms_norm_dx'])
    close(w.grad, golden_ops['rms_norm_dw'])


def test_rms_norm_dweight_is_deterministic():
    from qwen3_triton.kernels.norm import rms_norm
    x, w, dy = randn((4096, 1024), 4, torch.bfloat16), randn((1024,), 5, torch.bfloat16), randn((4096, 1024), 6, torch.bfloat16)
    grads = []
    for _ in range(3):
        xg, wg = dev(x).requires_grad_(True), dev(w).requires_grad_(True)
        rms_norm(xg, wg).backward(dev(dy))
        grads.append(wg.grad.clone())
    assert torch.equal(grads[0], grads[1]) and torch.equal(grads[0], grads[2])


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16])
@pytest.mark.parametrize('H', [2048, 4096, 5120, 8192])
@pytest.mark.parametrize('rows', [1, 300, 3001])
def test_wide_rows_through_the_shared_memory_ring(dtype, H, rows):
    """Rows of 2048..8192 elements go through the bulk-copy ring kernels: fewer rows than CTAs, and enough rows that
    every CTA wraps its ring several times (3001 rows over 296 CTAs = 10-11 rows each, 2-8 slots). Plain and
    add+norm forms, backward with and without an incoming residual gradient; no wait may time out."""
    from qwen3_triton import _abi
    from qwen3_triton.kernels.norm import add_rms_norm, rms_norm
    shape = (rows, H)
    x, r = randn(shape, 21, dtype), randn(shape, 22, dtype)
    w = (1 + 0.1 * randn((H,), 23)).to(dtype)
    dy, dr = randn(shape, 24, dtype), randn(shape, 25, dtype)
    xg, wg = dev(x).requires_grad_(True), dev(w).requires_grad_(True)
    y = rms_norm(xg, wg, 1e-6)
    y.backward(dev(dy))
    close(y, O.rms_norm(x, w).to(dtype), what='y')
    dx, dw = O.rms_norm_backward(x, w, dy)
    close(xg.grad, dx.to(dtype), what='dx')
    close(wg.grad, dw.to(dtype), scale=float(dw.abs().mean()), what='dw')
    xg, rg, wg = dev(x).requires_grad_(True), dev(r).requires_grad_(True), dev(w).requires_grad_(True)
    y, res = add_rms_norm(xg, rg, wg, 1e-6)
    torch.autograd.backward([y, res], [dev(dy), dev(dr)])
    y_ref, res_ref = O.add_rms_norm(x, r, w, 1e-6, round_dtype=dtype)
    close(res, res_ref.to(dtype), what='residual_out')
    close(y, y_ref.to(dtype), what='add y')
    dx_ref, dw_ref = O.rms_norm_backward(res_ref, w, dy)
    close(xg.grad, (dx_ref + dr.float()).to(dtype), what='add dx')
    close(wg.grad, dw_ref.to(dtype), scale=float(dw_ref.abs().mean()), what='add dw')
    assert _abi.read_status() == 0


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float32])
@pytest.mark.parametrize('shape', [(2, 17, 256), (1, 64, 4096), (3, 3, 50)])
def test_add_rms_norm(dtype, shape):
    from qwen3_triton.kernels.norm import add_rms_norm
    x, r = randn(shape, 11, dtype), randn(shape, 12, dtype)
    w = (1 + 0.1 * randn(shape[-1:], 13)).to(dtype)
    dy, dr = randn(shape, 14, dtype), randn(shape, 15, dtype)
    xg, rg, wg = dev(x).requires_grad_(True), dev(r).requires_grad_(True), dev(w).requires_grad_(True)
    y, res = add_rms_norm(xg, rg, wg, 1e-6)
    torch.autograd.backward([y, res], [dev(dy), dev(dr)])
    y_ref, res_ref = O.add_rms_norm(x, r, w, 1e-6, round_dtype=dtype)
    close(res, res_ref.to(dtype), what='residual_out')
    close(y, y_ref.to(dtype), what='y')
    dx_ref, dw_ref = O.rms_norm_backward(res_ref, w, dy)
    dx_ref = dx_ref + dr.float()
    close(xg.grad, dx_ref.to(dtype), what='dx')
    close(rg.grad, dx_ref.to(dtype), what='dresidual')
    close(wg.grad, dw_ref.to(dtype), scale=float(dw_ref.abs().mean()), what='dw')


@pytest.mark.parametrize('dtype', DTYPES)
@pytest.mark.parametrize('n', [1, 17, 1031, 4099, 1 << 20])
def test_residual_and_swiglu(dtype, n):
    from qwen3_triton.kernels.activation import swiglu
    from qwen3_triton.kernels.math_precision import swiglu as swiglu_hf
    from qwen3_triton.kernels.residual import residual_add
    from ops.triton.silu_and_mul import silu_and_mul_triton
    a, b, dy = randn((n,), 21, dtype), randn((n,), 22, dtype), randn((n,), 23, dtype)
    close(residual_add(dev(a), dev(b)), (a.float() + b.float()).to(dtype), what='add')
    g, u = dev(a).requires_grad_(True), dev(b).requires_grad_(True)
    y = swiglu(g, u)
    y.backward(dev(dy))
    close(y, O.swiglu(a, b).to(dtype), what='swiglu')
    dg, du = O.swiglu_backward(a, b, dy)
    close(g.grad, dg.to(dtype), what='dg')
    close(u.grad, du.to(dtype), what='du')
    close(swiglu_hf(dev(a), dev(b)), O.swiglu(a, b).to(dtype), what='hf name')
    close(silu_and_mul_triton(dev(a), dev(b)), O.swiglu(a, b).to(dtype), what='ops.triton')


def test_swiglu_golden(golden_ops):
    from qwen3_triton.kernels.activation import swiglu
    d = recipe.op_inputs()
    g, u = dev(d['gate']).requires_grad_(True), dev(d['up']).requires_grad_(True)
    y = swiglu(g, u)
    y.backward(dev(d['dy_act']))
    close(y, golden_ops['swiglu'])
    close(g.grad, golden_ops['swiglu_dg'])
    close(u.grad, golden_ops['swiglu_du'])


@pytest.mark.parametrize('src', DTYPES)
@pytest.mark.parametrize('dst', DTYPES)
def test_cast(src, dst):
    from qwen3_triton.kernels.attention import cast_tensor
    for n in (1, 7, 1031, 4099, 65536):
        x = randn((n,), 31, src)
        assert torch.equal(cast_tensor(dev(x), dst).cpu(), x.to(dst))
    # a misaligned view still casts correctly
    x = randn((4100,), 32, src)
    assert torch.equal(cast_tensor(dev(x)[1:], dst).cpu(), x[1:].to(dst))


@pytest.mark.parametrize('dtype', DTYPES)
@pytest.mark.parametrize('B,S,H,D', [(1, 1, 4, 64), (2, 17, 4, 128), (1, 129, 2, 64), (2, 5, 3, 6)])
def test_rope_both_layouts(dtype, B, S, H, D):
    from qwen3_triton.kernels.rotary import apply_rotary
    from ops.triton.rope import apply_rope_triton
    cos, sin = randn((B, S, D), 41, dtype), randn((B, S, D), 42, dtype)   # independent halves on purpose
    x, dy = randn((B, S, H, D), 43, dtype), randn((B, S, H, D), 44, dtype)
    xg = dev(x).requires_grad_(True)
    y = apply_rotary(xg, dev(cos), dev(sin))
    y.backward(dev(dy))
    close(y, O.apply_rope(x, cos, sin, 2).to(dtype), what='fwd [B,S,H,D]')
    close(xg.grad, O.apply_rope_backward(dy, cos, sin, 2).to(dtype), what='bwd [B,S,H,D]')
    q, k = randn((B, H, S, D), 45, dtype), randn((B, max(H // 2, 1), S, D), 46, dtype)
    qg, kg = dev(q).requires_grad_(True), dev(k).requires_grad_(True)
    yq, yk = apply_rope_triton(qg, kg, dev(cos), dev(sin))
    torch.autograd.backward([yq, yk], [torch.ones_like(yq), torch.ones_like(yk)])
    close(yq, O.apply_rope(q, cos, sin, 1).to(dtype), what='fwd q [B,H,S,D]')
    close(yk, O.apply_rope(k, cos, sin, 1).to(dtype), what='fwd k [B,H,S,D]')
    close(qg.grad, O.apply_rope_backward(torch.ones_like(q), cos, sin, 1).to(dtype), what='bwd q')


def test_rope_golden(golden_ops):
    from ops.triton.rope import apply_rope_triton
    d = recipe.op_inputs()
    yq, yk = apply_rope_triton(dev(d['q']), dev(d['k']), dev(d['cos']), dev(d['sin']))
    close(yq, golden_ops['rope_q'])
    close(yk, golden_ops['rope_k'])


def test_rotary_tables_and_positions_bit_exact_indexing():
    from qwen3_triton._model import position_ids_for
    from qwen3_triton.kernels.rotary import rotary_tables
    ids = torch.zeros(4, 4096, dtype=torch.int64, device='cuda')
    pos = position_ids_for(ids)
    assert torch.equal(pos.cpu(), torch.arange(4096).repeat(4, 1))          # integer work: bit-exact
    freq = O.inv_freq(128)
    for pdtype in (torch.int64, torch.int32):
        cos, sin = rotary_tables(pos.to(pdtype), freq.cuda(), torch.float32)
        c_ref, s_ref = O.rope_tables(pos.cpu(), freq)
        # fp32 sincos of angles up to ~4e3 rad: a few ulp of the argument
        torch.testing.assert_close(cos.cpu(), c_ref, rtol=0, atol=2e-4)
        torch.testing.assert_close(sin.cpu(), s_ref, rtol=0, atol=2e-4)
        assert torch.equal(cos[..., :64], cos[..., 64:])                      # duplicated halves
    cb, sb = rotary_tables(pos, freq.cuda(), torch.bfloat16)
    close(cb, c_ref.to(torch.bfloat16), scale=1.0)


@pytest.mark.parametrize('dtype', DTYPES)
@pytest.mark.parametrize('B,S,H,D', [(1, 1, 1, 64), (2, 17, 4, 128), (1, 129, 8, 128), (2, 3, 2, 32), (1, 4, 3, 10)])
def test_norm_rope(dtype, B, S, H, D):
    from qwen3_triton.kernels.norm_rope import norm_rope
    x, dy = randn((B, S, H, D), 51, dtype), randn((B, S, H, D), 52, dtype)
    w = (1 + 0.1 * randn((D,), 53)).to(dtype)
    cos, sin = randn((B, S, D), 54, dtype), randn((B, S, D), 55, dtype)
    xg, wg = dev(x).requires_grad_(True), dev(w).requires_grad_(True)
    y = norm_rope(xg, wg, dev(cos), dev(sin), 1e-6)
    y.backward(dev(dy))
    close(y, O.norm_rope(x, w, cos, sin).to(dtype), what='y')
    dx, dw = O.norm_rope_backward(x, w, cos, sin, dy)
    close(xg.grad, dx.to(dtype), what='dx')
    close(wg.grad, dw.to(dtype), scale=float(dw.abs().mean()), what='dw')


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16])
@pytest.mark.parametrize('B,S,H,D', [(1, 5000, 32, 128), (1, 5001, 8, 128), (3, 1667, 16, 64), (2, 301, 1, 256)])
def test_norm_rope_through_the_shared_memory_ring(dtype, B, S, H, D):
    """Token-major norm+RoPE at sizes where every CTA wraps its ring many times, with a ragged last slot
    (5001 tokens in slots of 4) and one to several tokens per slot; no wait may time out."""
    from qwen3_triton import _abi
    from qwen3_triton.kernels.norm_rope import norm_rope
    x, dy = randn((B, S, H, D), 61, dtype), randn((B, S, H, D), 62, dtype)
    w = (1 + 0.1 * randn((D,), 63)).to(dtype)
    cos, sin = randn((B, S, D), 64, dtype), randn((B, S, D), 65, dtype)
    xg, wg = dev(x).requires_grad_(True), dev(w).requires_grad_(True)
    y = norm_rope(xg, wg, dev(cos), dev(sin), 1e-6)
    y.backward(dev(dy))
    close(y, O.norm_rope(x, w, cos, sin).to(dtype), what='y')
    dx, dw = O.norm_rope_backward(x, w, cos, sin, dy)
    close(xg.grad, dx.to(dtype), what='dx')
    close(wg.grad, dw.to(dtype), scale=float(dw.abs().mean()), what='dw')
    assert _abi.read_status() == 0


@pytest.mark.parametrize('T,hq,hk,D', [(4100, 32, 8, 128), (333, 4, 4, 64), (50, 3, 1, 10)])
def test_q_and_k_in_one_launch_equal_two_launches(T, hq, hk, D):
    """q3_qk_norm_rope_* share one grid between q and k (or fall back to two launches for shapes the wide-row kernels
    do not take): outputs, input gradients and inverse norms bit-identical to the single-tensor entry points, weight
    gradients equal up to the fp32 order of the per-CTA partial sums."""
    from qwen3_triton import _abi
    from qwen3_triton.fused import _norm_rope_bwd, _norm_rope_fwd, _qk_norm_rope_bwd, _qk_norm_rope_fwd
    bf = torch.bfloat16
    q, k = randn((T, hq, D), 81, bf).cuda(), randn((T, hk, D), 82, bf).cuda()
    wq, wk = (1 + 0.1 * randn((D,), 83)).to(bf).cuda(), (1 + 0.1 * randn((D,), 84)).to(bf).cuda()
    cos, sin = randn((T, D), 85, bf).cuda(), randn((T, D), 86, bf).cuda()
    dq, dk = randn((T, hq, D), 87, bf).cuda(), randn((T, hk, D), 88, bf).cuda()
    yq, iq, yk, ik = _qk_norm_rope_fwd(q, k, wq, wk, cos, sin, T, hq, hk, D, 1e-6)
    yq1, iq1 = _norm_rope_fwd(q, wq, cos, sin, T, hq, D, 1e-6)
    yk1, ik1 = _norm_rope_fwd(k, wk, cos, sin, T, hk, D, 1e-6)
    assert torch.equal(yq, yq1) and torch.equal(yk, yk1) and torch.equal(iq, iq1) and torch.equal(ik, ik1)
    gq, gwq, gk, gwk = _qk_norm_rope_bwd(q, k, wq, wk, cos, sin, dq, dk, iq, ik, T, hq, hk, D)
    gq1, gwq1 = _norm_rope_bwd(q, wq, cos, sin, dq, iq, T, hq, D)
    gk1, gwk1 = _norm_rope_bwd(k, wk, cos, sin, dk, ik, T, hk, D)
    assert torch.equal(gq, gq1) and torch.equal(gk, gk1)
    close(gwq, gwq1, scale=float(gwq1.float().abs().mean()), what='dwq')
    close(gwk, gwk1, scale=float(gwk1.float().abs().mean()), what='dwk')
    assert _abi.read_status() == 0


def test_fused_qk_norm_rope_golden(golden_ops):
    from ops.triton.fused_qk_norm_rope import fused_qk_norm_rope_triton
    d = recipe.op_inputs()
    q, k = dev(d['qn']).requires_grad_(True), dev(d['kn']).requires_grad_(True)
    qw, kw = dev(d['qw']).requires_grad_(True), dev(d['kw']).requires_grad_(True)
    yq, yk = fused_qk_norm_rope_triton(q, k, qw, kw, dev(d['cos']), dev(d['sin']), 1e-6)
    torch.autograd.backward([yq, yk], [dev(d['dqn']), dev(d['dkn'])])
    close(yq, golden_ops['fused_q'])
    close(yk, golden_ops['fused_k'])
    close(q.grad, golden_ops['fused_dq'])
    close(k.grad, golden_ops['fused_dk'])
    close(qw.grad, golden_ops['fused_dqw'])
    close(kw.grad, golden_ops['fused_dkw'])


@pytest.mark.parametrize('dtype', DTYPES)
@pytest.mark.parametrize('idtype', [torch.int64, torch.int32])
def test_embedding_gather_bit_exact_and_dense_gradient(dtype, idtype):
    from qwen3_triton.kernels.embedding import embedding
    V, H = 997, 136
    w = randn((V, H), 61, dtype)
    g = torch.Generator().manual_seed(62)
    ids = torch.randint(0, V, (3, 129), generator=g)
    ids[0, :40] = 5                     # heavy repetition of one token
    ids[1, 7] = V - 1
    wg = dev(w).requires_grad_(True)
    y = embedding(ids.to(idtype).cuda(), wg)
    assert torch.equal(y.cpu(), w[ids])                                    # gather: bit-exact
    dy = randn((3, 129, H), 63, dtype)
    y.backward(dev(dy))
    close(wg.grad, O.embedding_backward(ids, dy, V).to(dtype), scale=1.0, what='dW')
    untouched = torch.ones(V, dtype=torch.bool)
    untouched[ids.reshape(-1)] = False
    assert wg.grad[untouched.cuda()].abs().max() == 0                      # dense, zero-filled rows
    y2 = embedding(ids.to(idtype).cuda(), wg)
    wg.grad = None
    y2.backward(dev(dy))
    g1 = wg.grad.clone()
    wg.grad = None
    embedding(ids.to(idtype).cuda(), wg).backward(dev(dy))
    assert torch.equal(g1, wg.grad)                                        # deterministic


@pytest.mark.parametrize('world', [1, 4])
def test_embedding_vocabulary_shards_sum_to_the_full_lookup_and_gradient(world):
    """Each of `world` row shards (fp32 master) looks up the tokens it owns and zeros elsewhere: the sum over
    shards is the bf16-cast full lookup bit for bit; the shard gradients, stacked, are the full fp32 gradient
    times the scale; long chains of one repeated token and ids at the shard edges included."""
    from qwen3_triton.kernels.embedding import shard_lookup, shard_weight_gradient
    V, H, T = 1024, 264, 5000
    w = randn((V, H), 66, torch.float32)
    g = torch.Generator().manual_seed(67)
    ids = torch.randint(0, V, (T,), generator=g)
    ids[100:1300] = 255                 # one chain of 1200 positions, on a shard edge for world 4
    ids[0], ids[1], ids[-1] = 0, V - 1, 256
    dy = randn((T, H), 68, torch.bfloat16)
    rows = V // world
    total = torch.zeros(T, H)
    grads = []
    for r in range(world):
        shard = w[r * rows:(r + 1) * rows].cuda().contiguous()
        part = shard_lookup(ids.cuda(), shard, r * rows, V, torch.bfloat16)
        own = (ids >= r * rows) & (ids < (r + 1) * rows)
        assert part[~own.cuda()].abs().sum() == 0
        total += part.float().cpu()
        grads.append(shard_weight_gradient(ids.cuda(), dev(dy), r * rows, rows, 0.25).cpu())
        assert torch.equal(grads[-1], shard_weight_gradient(ids.cuda(), dev(dy), r * rows, rows, 0.25).cpu())
    assert torch.equal(total, w.to(torch.bfloat16)[ids].float())
    ref = torch.zeros(V, H, dtype=torch.float64).index_add_(0, ids, dy.double()) * 0.25
    torch.testing.assert_close(torch.cat(grads).double(), ref, rtol=1e-5, atol=1e-5)


def test_vocab_parallel_embedding_module_world_1():
    from qwen3_triton.training.vocab_parallel import VocabParallelEmbedding
    V, H = 512, 128
    w = randn((V, H), 69, torch.float32)
    emb = VocabParallelEmbedding(w)
    g = torch.Generator().manual_seed(70)
    ids = torch.randint(0, V, (2, 300), generator=g)
    y = emb(ids.cuda())
    assert y.dtype == torch.bfloat16 and torch.equal(y.cpu(), w.to(torch.bfloat16)[ids])
    dy = randn((2, 300, H), 71, torch.bfloat16)
    y.backward(dev(dy))
    ref = torch.zeros(V, H).index_add_(0, ids.view(-1), dy.float().view(-1, H))
    torch.testing.assert_close(emb.weight.grad.cpu(), ref, rtol=1e-5, atol=1e-5)
    assert emb.forward_calls == 1 and emb.backward_calls == 1
    with pytest.raises(TypeError):
        emb(ids.int().cuda())


def test_embedding_out_of_range_id_sets_status_not_trap():
    from qwen3_triton import _abi
    from qwen3_triton.kernels.embedding import embedding
    w = randn((16, 8), 64, torch.float32).cuda()
    ids = torch.tensor([[1, 99, 3]], device='cuda')
    y = embedding(ids, w)
    assert _abi.read_status() & _abi.STATUS_ID_RANGE
    assert y[0, 1].abs().max() == 0 and torch.equal(y[0, 0], w[1])


@pytest.mark.parametrize('dtype', DTYPES)
@pytest.mark.parametrize('B,S,V', [(1, 2, 5), (2, 17, 1031), (1, 129, 2048), (2, 9, 4099)])
def test_cross_entropy(dtype, B, S, V):
    from qwen3_triton.kernels.loss import causal_cross_entropy
    logits = randn((B, S, V), 71, dtype, scale=3.0)
    g = torch.Generator().manual_seed(72)
    labels = torch.randint(0, V, (B, S), generator=g)
    if S > 4:
        labels[0, 3] = -100
    xg = dev(logits).requires_grad_(True)
    loss = causal_cross_entropy(xg, labels.cuda())
    (loss * 1.5).backward()
    ref = O.causal_cross_entropy(logits, labels)
    assert loss.dtype == torch.float32
    torch.testing.assert_close(loss.cpu(), ref, rtol=1e-3, atol=1e-5)     # loss within 1e-3 relative
    gref = O.causal_cross_entropy_backward(logits, labels, upstream=1.5)
    close(xg.grad, gref.to(dtype), scale=float(gref.abs().max()) / 10, what='dlogits')
    assert xg.grad[:, -1].abs().max() == 0                                 # last position is never scored


def test_cross_entropy_bad_label_sets_status():
    from qwen3_triton import _abi
    from qwen3_triton.kernels.loss import causal_cross_entropy
    logits = randn((1, 4, 10), 73, torch.float32).cuda()
    labels = torch.tensor([[1, 2, 77, 3]], device='cuda')
    causal_cross_entropy(logits, labels)
    assert _abi.read_status() & _abi.STATUS_LABEL_RANGE


def test_outputs_fully_overwritten_poison():
    """NaN-poisoned output buffers: every element must be written (reference scripts/check_overwrite_outputs_v13.py)."""
    from qwen3_triton import _abi
    n = 4099
    a, b = randn((n,), 81, torch.bfloat16).cuda(), randn((n,), 82, torch.bfloat16).cuda()
    out = torch.full((n,), float('nan'), dtype=torch.bfloat16, device='cuda')
    _abi.call('q3_residual_add', a.data_ptr(), b.data_ptr(), out.data_ptr(), n, _abi.Q3_BF16, _abi.stream())
    assert torch.isfinite(out).all()
    x, w = randn((7, 2048), 83, torch.bfloat16).cuda(), randn((2048,), 84, torch.bfloat16).cuda()
    y = torch.full_like(x, float('nan'))
    inv = torch.full((7,), float('nan'), device='cuda')
    _abi.call('q3_rmsnorm_fwd', x.data_ptr(), w.data_ptr(), y.data_ptr(), inv.data_ptr(), 7, 2048, 1e-6, _abi.Q3_BF16, _abi.stream())
    assert torch.isfinite(y).all() and torch.isfinite(inv).all()
