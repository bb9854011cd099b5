"""Causal GQA attention forward/backward against the oracle (ops/reference math) and the reference's own
outputs at the fixture shape; GQA head mapping and the log-sum-exp definition are checked explicitly."""
import pytest
import torch

import recipe
from helpers import L2, L2_ATTENTION_GRAD, close, randn, rel_l2
from oracle import ops as O

pytestmark = pytest.mark.gpu

CASES = [  # B, Hq, Hkv, S, D
    (1, 1, 1, 1, 64), (2, 4, 2, 17, 64), (1, 4, 2, 129, 128), (1, 8, 2, 257, 128), (2, 4, 4, 64, 32),
    (1, 2, 1, 33, 96), (1, 4, 1, 200, 256), (2, 8, 2, 512, 128),
]


@pytest.mark.parametrize('B,Hq,Hkv,S,D', CASES)
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float32, torch.float16])
def test_attention_forward_backward(B, Hq, Hkv, S, D, dtype):
    from qwen3_triton.kernels.attention import causal_attention
    q, k, v = randn((B, Hq, S, D), 1, dtype), randn((B, Hkv, S, D), 2, dtype), randn((B, Hkv, S, D), 3, dtype)
    do = randn((B, Hq, S, D), 4, dtype)
    qg, kg, vg = (t.cuda().requires_grad_(True) for t in (q, k, v))
    out = causal_attention(qg, kg, vg)
    out.backward(do.cuda())
    ref, _ = O.attention(q, k, v)
    close(out, ref.to(dtype), what='out')
    dq, dk, dv = O.attention_backward(q, k, v, do)
    # The saved output is rounded to `dtype`, so delta = rowsum(dO*O) carries that rounding into dS; a handful
    # of near-zero gradient elements then sit a few percent of the tensor scale away (the reference's own
    # attention-gradient tolerance is 8e-2 absolute). Relative term stays at the stated 2e-2.
    close(qg.grad, dq.to(dtype), what='dq', atol_mult=5.0, l2=L2_ATTENTION_GRAD[dtype])
    close(kg.grad, dk.to(dtype), what='dk', atol_mult=5.0, l2=L2_ATTENTION_GRAD[dtype])
    close(vg.grad, dv.to(dtype), what='dv', atol_mult=5.0, l2=L2_ATTENTION_GRAD[dtype])


def test_attention_golden_and_lse(golden_ops):
    from ops.triton.attention import attention_triton, attention_triton_autograd
    from ops.triton.attention_backward import attention_backward_triton
    d = recipe.op_inputs()
    q, k, v, do = (d[n].cuda() for n in ('q', 'k', 'v', 'do'))
    out, lse = attention_triton(q, k, v, return_lse=True)
    close(out, golden_ops['attn'])
    _, lse_ref = O.attention(d['q'], d['k'], d['v'])
    torch.testing.assert_close(lse.cpu(), lse_ref, rtol=1e-4, atol=1e-4)
    dq, dk, dv = attention_backward_triton(q, k, v, do, lse=lse)
    close(dq, golden_ops['attn_dq'], l2=L2_ATTENTION_GRAD[dq.dtype])
    close(dk, golden_ops['attn_dk'], l2=L2_ATTENTION_GRAD[dk.dtype])
    close(dv, golden_ops['attn_dv'], l2=L2_ATTENTION_GRAD[dv.dtype])
    qg = q.clone().requires_grad_(True)
    attention_triton_autograd(qg, k, v).backward(do)
    close(qg.grad, golden_ops['attn_dq'], l2=L2_ATTENTION_GRAD[qg.grad.dtype])


def test_gqa_head_mapping_is_exact():
    """Query head h must read kv head h // (Hq/Hkv): make every kv head's V a distinct constant."""
    from qwen3_triton.kernels.attention import causal_attention
    B, Hq, Hkv, S, D = 1, 8, 2, 40, 64
    q, k = randn((B, Hq, S, D), 5, torch.float32).cuda(), randn((B, Hkv, S, D), 6, torch.float32).cuda()
    v = torch.stack([torch.full((S, D), float(i + 1)) for i in range(Hkv)])[None].cuda().contiguous()
    out = causal_attention(q, k, v)
    for h in range(Hq):
        assert torch.allclose(out[0, h], torch.full((S, D), float(h // (Hq // Hkv) + 1), device='cuda'), atol=1e-5)


def test_candidate_entry_matches_causal_attention():
    from qwen3_triton.kernels.attention import causal_attention
    from qwen3_triton.kernels.attention_precision import candidate
    q, k, v = randn((1, 8, 256, 128), 7, torch.bfloat16).cuda(), randn((1, 2, 256, 128), 8, torch.bfloat16).cuda(), randn((1, 2, 256, 128), 9, torch.bfloat16).cuda()
    a = candidate(q, k, v, fusion=False, lane_sum=True, round_kv=True, reciprocal=1, stages=2, xor_sum=True,
                  lse_fma=True, native_delta=True, native_dq=True, sum_fma=True)
    assert torch.equal(a, causal_attention(q, k, v))


@pytest.mark.parametrize('B,Hq,Hkv,S', [(1, 4, 2, 128), (2, 8, 2, 300), (1, 4, 1, 513)])
def test_token_major_layout_matches_head_major(B, Hq, Hkv, S):
    """q3_attn_fwd_bshd / q3_attn_bwd_bshd read and write [B,S,H,128] directly; results must equal the
    [B,H,S,128] entry points on transposed copies, bit for bit (same kernels, different TMA strides)."""
    from qwen3_triton import _abi
    from qwen3_triton.kernels.attention import attention_backward, attention_forward
    dt = torch.bfloat16
    q, k, v, do = (randn(s, i, dt).cuda() for i, s in enumerate([(B, S, Hq, 128), (B, S, Hkv, 128), (B, S, Hkv, 128), (B, S, Hq, 128)]))
    out = torch.empty_like(q)
    lse = torch.empty(B, Hq, S, device='cuda')
    st = _abi.status_word('cuda').data_ptr()
    _abi.call('q3_attn_fwd_bshd', q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), B, S, Hq, Hkv,
              128, 128 ** -0.5, _abi.Q3_BF16, st, _abi.stream())
    qh, kh, vh, doh = (t.transpose(1, 2).contiguous() for t in (q, k, v, do))
    out_h, lse_h = attention_forward(qh, kh, vh, 128 ** -0.5)
    assert torch.equal(out.transpose(1, 2), out_h) and torch.equal(lse, lse_h)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    ws = _abi.workspace(_abi.lib().q3_attn_bwd_workspace_bytes(B, Hq, Hkv, S, 128), 'cuda')
    _abi.call('q3_attn_bwd_bshd', q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), do.data_ptr(), lse.data_ptr(),
              dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), ws.data_ptr(), ws.numel(), B, S, Hq, Hkv, 128, 128 ** -0.5,
              _abi.Q3_BF16, st, _abi.stream())
    dqh, dkh, dvh = attention_backward(qh, kh, vh, out_h, doh, lse_h, 128 ** -0.5)
    assert torch.equal(dq.transpose(1, 2), dqh) and torch.equal(dk.transpose(1, 2), dkh) and torch.equal(dv.transpose(1, 2), dvh)


# ------------------------------------------------------------------------------------------------------------------
# The two dK/dV schedules at head_dim 128. Small grids (fewer than two CTAs per SM) run one CTA per query head and a
# fixed-order reduction; the shapes the training step and the attention benchmark use (batch x kv heads x key tiles
# >= 296) run one CTA per key tile that accumulates the whole query-head group in tensor memory. Both are compared
# with the oracle here, on long sequences (16 - 64 key tiles), and the test asserts which schedule ran.
def _oracle_by_group(q, k, v, do, saved_out=None):
    """Oracle forward/backward one (batch, kv head) at a time: same math, [1, G, S, S] fp32 scores at once. Returns the
    output, the exact gradients and, with `saved_out`, the gradients computed with the stored output in the row term."""
    B, Hq, S, D = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    out = torch.empty(B, Hq, S, D)
    exact = [torch.empty(B, Hq, S, D), torch.empty(B, Hkv, S, D), torch.empty(B, Hkv, S, D)]
    stored = [torch.empty_like(t) for t in exact]
    for b in range(B):
        for h in range(Hkv):
            heads = slice(h * G, (h + 1) * G)
            qs, ks, vs, dos = q[b:b + 1, heads], k[b:b + 1, h:h + 1], v[b:b + 1, h:h + 1], do[b:b + 1, heads]
            out[b, heads] = O.attention(qs, ks, vs)[0][0]
            for grads, so in ((exact, None), (stored, saved_out)):
                if grads is stored and saved_out is None:
                    continue
                a, c, e = O.attention_backward(qs, ks, vs, dos, saved_out=None if so is None else so[b:b + 1, heads])
                grads[0][b, heads], grads[1][b, h], grads[2][b, h] = a[0], c[0, 0], e[0, 0]
    return out, exact, stored


class _GroupPolicy:
    def __init__(self, policy):
        self.policy = policy

    def __enter__(self):
        from qwen3_triton import _abi
        self.old = _abi.lib().q3_attn_bwd_group_policy(self.policy)

    def __exit__(self, *exc):
        from qwen3_triton import _abi
        _abi.lib().q3_attn_bwd_group_policy(self.old)


def _check_against_oracle(B, Hq, Hkv, S, dtype, expect_split):
    from qwen3_triton import _abi
    from qwen3_triton.kernels.attention import causal_attention
    D = 128
    assert _abi.lib().q3_attn_bwd_group_split(B, Hq, Hkv, S) == expect_split
    q, k, v = randn((B, Hq, S, D), 31, dtype), randn((B, Hkv, S, D), 32, dtype), randn((B, Hkv, S, D), 33, dtype)
    do = randn((B, Hq, S, D), 34, dtype)
    qg, kg, vg = (t.cuda().requires_grad_(True) for t in (q, k, v))
    out = causal_attention(qg, kg, vg)
    out.backward(do.cuda())
    assert _abi.read_status() == 0
    ref, exact, stored = _oracle_by_group(q, k, v, do, saved_out=out.detach().float().cpu())
    close(out, ref.to(dtype), what='out', scale='row')
    for name, got, e, s in zip(('dq', 'dk', 'dv'), (qg.grad, kg.grad, vg.grad), exact, stored):
        # against the exact math: per-tensor distance (the rounding of the stored output shifts the row term of dS by
        # about 2^-9 |dO||O|, which is a visible fraction of the few rows whose gradient nearly cancels)
        assert rel_l2(got, e) <= L2_ATTENTION_GRAD[dtype], (name, rel_l2(got, e))
        # against the same math with the stored output in the row term, as flash-attention backward defines it:
        # element by element, floor relative to each row
        close(got, s.to(dtype), what=name, scale='row', atol_mult=5.0, l2=L2_ATTENTION_GRAD[dtype])
    return qg.grad, kg.grad, vg.grad


@pytest.mark.parametrize('B,Hq,Hkv,S', [(4, 32, 8, 1280), (3, 32, 8, 2048)])
def test_backward_group_accumulating_schedule_at_training_shapes(B, Hq, Hkv, S):
    """Grids of 320 and 384 key-tile CTAs: the schedule picked by size is the group-accumulating one."""
    _check_against_oracle(B, Hq, Hkv, S, torch.bfloat16, expect_split=1)


@pytest.mark.parametrize('S', [2048, 4096, 8192])
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16])
def test_backward_schedules_on_long_sequences(S, dtype):
    """One query-head group (4 query heads on 1 kv head) of each sequence length the attention benchmark uses
    (2048, 4096, 8192 = 16, 32, 64 key tiles), both schedules forced in turn; each against the oracle, and against
    each other (they differ only in fp32 summation order)."""
    if dtype == torch.float16 and S != 4096:
        pytest.skip('fp16 covered at one length')
    with _GroupPolicy(1):
        a = _check_against_oracle(1, 4, 1, S, dtype, expect_split=1)
    with _GroupPolicy(2):
        b = _check_against_oracle(1, 4, 1, S, dtype, expect_split=4)
    for x, y, name in zip(a, b, ('dq', 'dk', 'dv')):
        close(x, y.float().cpu().to(dtype), what=name + ' schedules agree', l2=L2[dtype])


@pytest.mark.parametrize('B,Hq,Hkv,S', [(1, 2, 2, 257), (2, 4, 4, 1024)])
def test_backward_without_grouping_at_head_dim_128(B, Hq, Hkv, S):
    """Hq == Hkv: a group is one head, so there is nothing to split."""
    _check_against_oracle(B, Hq, Hkv, S, torch.bfloat16, expect_split=1)


def test_group_policy_switch_round_trip():
    from qwen3_triton import _abi
    lib = _abi.lib()
    assert lib.q3_attn_bwd_group_policy(-1) == 0            # query only
    assert lib.q3_attn_bwd_group_split(1, 32, 8, 2048) == 4  # 128 CTAs on 148 SMs: per-head split
    with _GroupPolicy(1):
        assert lib.q3_attn_bwd_group_split(1, 32, 8, 2048) == 1
        ws1 = lib.q3_attn_bwd_workspace_bytes(1, 32, 8, 2048, 128)
    assert lib.q3_attn_bwd_workspace_bytes(1, 32, 8, 2048, 128) > ws1   # the split schedule needs fp32 partials
    assert lib.q3_attn_bwd_group_policy(-1) == 0
