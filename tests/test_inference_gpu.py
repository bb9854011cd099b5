"""Decode-time operators against the CPU restatement in oracle/inference.py: cache append (bit-exact), attention over
the cache for prefill chunks and single-token decode across chunk boundaries, GEMV with fp32 and fp64 accumulation,
and the greedy selection step (ties, finished rows, end-of-sequence ids)."""
import pytest
import torch

from helpers import close, randn
from oracle import inference as OI

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float32])
@pytest.mark.parametrize('B,S,H,D,C,start', [(2, 5, 2, 64, 16, 3), (1, 1, 8, 128, 600, 599), (3, 64, 1, 128, 64, 0)])
def test_cache_append_is_bit_exact(dtype, B, S, H, D, C, start):
    from qwen3_triton.inference import kernels as K
    k, v = randn((B, S, H, D), 1, dtype), randn((B, S, H, D), 2, dtype)
    ck, cv = randn((B, H, C, D), 3, dtype), randn((B, H, C, D), 4, dtype)
    dk, dv = ck.cuda(), cv.cuda()
    K.append(k.cuda(), v.cuda(), dk, dv, start)
    OI.append(k, v, ck, cv, start)
    assert torch.equal(dk.cpu(), ck) and torch.equal(dv.cpu(), cv)
    with pytest.raises(ValueError):
        K.append(k.cuda(), v.cuda(), dk, dv, C - S + 1)


def test_positions():
    from qwen3_triton.inference import kernels as K
    assert K.positions(3, 5, 17, 'cuda').tolist() == [[17, 18, 19, 20, 21]] * 3


CASES = [  # B, S, Hq, Hkv, D, start
    (1, 1, 4, 1, 128, 0), (2, 1, 32, 8, 128, 255), (2, 1, 32, 8, 128, 256), (1, 1, 8, 2, 128, 1500), (1, 7, 4, 2, 64, 0),
    (2, 65, 8, 2, 128, 0), (1, 33, 4, 4, 128, 250), (1, 3, 8, 1, 64, 700), (1, 2, 2, 1, 256, 300), (1, 300, 4, 1, 128, 0)]


@pytest.mark.parametrize('B,S,Hq,Hkv,D,start', CASES)
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16, torch.float32])
def test_attention_over_the_cache(B, S, Hq, Hkv, D, start, dtype):
    from qwen3_triton.inference import kernels as K
    if dtype == torch.float16 and S > 7:
        pytest.skip('fp16 covered on the decode shapes')
    C = start + S + 9                                  # capacity beyond the live tokens: must never be read as keys
    q = randn((B, S, Hq, D), 11, dtype)
    ck, cv = randn((B, Hkv, C, D), 12, dtype), randn((B, Hkv, C, D), 13, dtype)
    ck[:, :, start + S:] = float('nan')
    cv[:, :, start + S:] = float('nan')
    out = K.attention(q.cuda(), ck.cuda(), cv.cuda(), start, split_decode=S == 1)
    ref = OI.attention(q, ck, cv, start)
    close(out, ref.to(dtype), what='cache attention', scale='row')
    assert torch.equal(out, K.attention(q.cuda(), ck.cuda(), cv.cuda(), start))        # deterministic


@pytest.mark.parametrize('B,S,Hq,Hkv,start', [(2, 1, 32, 8, 1000), (1, 5, 8, 8, 130), (1, 1, 16, 2, 127), (3, 2, 4, 2, 0)])
def test_tensor_core_and_cuda_core_cache_attention_agree(B, S, Hq, Hkv, start):
    """bf16 caches at head_dim 128 take the MMA kernel; the CUDA-core kernel must give the same result up to the bf16
    rounding of the probabilities (the MMA kernel feeds them to the second product in bf16)."""
    from qwen3_triton import _abi
    from qwen3_triton.inference import kernels as K
    dtype, D = torch.bfloat16, 128
    C = start + S
    q = randn((B, S, Hq, D), 41, dtype).cuda()
    ck, cv = randn((B, Hkv, C, D), 42, dtype).cuda(), randn((B, Hkv, C, D), 43, dtype).cuda()
    lib = _abi.lib()
    assert lib.q3_cache_attention_path(-1) == 0
    fast = K.attention(q, ck, cv, start)
    old = lib.q3_cache_attention_path(1)
    try:
        slow = K.attention(q, ck, cv, start)
    finally:
        lib.q3_cache_attention_path(old)
    close(fast, slow.float().cpu().to(dtype), what='mma vs cuda cores', scale='row')
    close(fast, OI.attention(q.cpu(), ck.cpu(), cv.cpu(), start).to(dtype), what='mma vs oracle', scale='row')


def test_grouped_query_heads_read_their_own_kv_head():
    from qwen3_triton.inference import kernels as K
    B, S, Hq, Hkv, D, T = 1, 1, 8, 2, 64, 40
    q = randn((B, S, Hq, D), 5, torch.float32).cuda()
    ck = randn((B, Hkv, T, D), 6, torch.float32).cuda()
    cv = torch.stack([torch.full((T, D), float(i + 1)) for i in range(Hkv)])[None].cuda().contiguous()
    out = K.attention(q, ck, cv, T - 1)
    for h in range(Hq):
        assert torch.allclose(out[0, 0, h], torch.full((D,), float(h // (Hq // Hkv) + 1), device='cuda'), atol=1e-5)


@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float32])
@pytest.mark.parametrize('M,N,K', [(1, 4096, 4096), (8, 1000, 520), (3, 17, 12288), (1, 151936, 1024), (5, 64, 8)])
def test_gemv(dtype, M, N, K):
    from qwen3_triton.inference import kernels as KK
    x, w = randn((M, K), 21, dtype), randn((N, K), 22, dtype, 0.05)
    y = KK.linear(x.cuda(), w.cuda())
    close(y, OI.linear(x, w).to(dtype), what='gemv')
    y64 = KK.linear(x.cuda(), w.cuda(), accurate=True)
    close(y64, OI.linear(x, w, accurate=True).to(dtype), what='gemv fp64')
    if dtype == torch.float32:
        torch.testing.assert_close(y64.cpu(), OI.linear(x, w, accurate=True), rtol=2e-6, atol=1e-6)
    big = randn((2, 5, K), 23, dtype)                   # more than 8 rows: the tensor-core GEMM or its fallback
    close(KK.linear(big.cuda(), w.cuda()), OI.linear(big.reshape(10, K), w).view(2, 5, N).to(dtype), what='linear M=10')


def test_select_step_by_step():
    from qwen3_triton.inference import kernels as K
    g = torch.Generator().manual_seed(9)
    B, V, L = 6, 151936, 5
    eos, pad = (7, 151645), 0
    ids_d = torch.full((B, L), -1, dtype=torch.int64, device='cuda')
    nxt_d = torch.full((B, 1), -1, dtype=torch.int64, device='cuda')
    done_d = torch.zeros(B, dtype=torch.bool, device='cuda')
    ids_h, nxt_h, done_h = ids_d.cpu().clone(), nxt_d.cpu().clone(), done_d.cpu().clone()
    for position in range(1, L):
        logits = torch.randn(B, V, generator=g).to(torch.bfloat16)
        logits[0, 100] = logits[0, 90000] = 50.0        # tie: the lower index wins
        if position == 2:
            logits[1, 7] = 60.0                         # row 1 ends here ...
            logits[2, 151645] = 60.0                    # ... and row 2, on the other end id
        K.select(logits.cuda(), ids_d, nxt_d, done_d, position, eos, pad)
        OI.select(logits, ids_h, nxt_h, done_h, position, eos, pad)
        assert torch.equal(ids_d.cpu(), ids_h) and torch.equal(nxt_d.cpu(), nxt_h) and torch.equal(done_d.cpu(), done_h)
    assert ids_h[0, 1:].tolist() == [100] * (L - 1) and done_h.tolist() == [False, True, True, False, False, False]
    assert ids_h[1].tolist() == [-1, ids_h[1, 1].item(), 7, pad, pad]
    fp32 = torch.randn(3, 1000, generator=g)
    K.select(fp32.cuda(), ids_d[:3].contiguous(), nxt_d[:3].contiguous(), torch.zeros(3, dtype=torch.bool, device='cuda'), 0, (), pad)
    with pytest.raises(ValueError):
        K.select(fp32.cuda(), ids_d[:3].contiguous(), nxt_d[:3].contiguous(), done_d[:3].contiguous(), L, eos, pad)
