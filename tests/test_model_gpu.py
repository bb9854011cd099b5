"""End-to-end parity of the CUDA decoder graph with the oracle model and with the reference's own tiny-model
run (2 layers, hidden 256, vocab 2048, batch 2 x 128): loss, logits, every gradient, one AdamW step. Also the vocab-parallel head at
world size 1 against the materialised-logits loss."""
import pytest
import torch

import recipe
from helpers import close, rel_l2
from oracle.model import OracleQwen3

pytestmark = pytest.mark.gpu


def build(variant, state, dtype):
    from qwen3_triton import model_for_variant
    c = recipe.tiny_config()
    model = model_for_variant(c, variant)
    model.load_hf_state_dict({k: v.clone() for k, v in state.items()})
    return model.to('cuda', dtype)


@pytest.mark.parametrize('variant', ['triton_base', 'triton_optimized'])
def test_tiny_fp32_matches_reference_run(variant, golden_tiny):
    from qwen3_triton.runtime.adamw import TritonAdamW
    c = recipe.tiny_config()
    model = build(variant, recipe.seeded_state(c), torch.float32)
    ids = recipe.seeded_ids(c).cuda()
    out = model(ids, labels=ids)
    out.loss.backward()
    torch.testing.assert_close(out.loss.cpu(), golden_tiny['loss'], rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(out.logits[0, :4, :16].cpu(), golden_tiny['logits_slice'], rtol=2e-3, atol=2e-4)
    for name, p in model.named_parameters():
        torch.testing.assert_close(p.grad.norm().cpu(), golden_tiny['gradnorm/' + name], rtol=2e-3, atol=1e-7)
        torch.testing.assert_close(p.grad.reshape(-1)[:32].cpu(), golden_tiny['gradslice/' + name], rtol=5e-3, atol=2e-6)
    opt = TritonAdamW(model.parameters(), **recipe.ADAMW)
    opt.step()
    for name, p in model.named_parameters():
        torch.testing.assert_close(p.detach().reshape(-1)[:32].cpu(), golden_tiny['stepslice/' + name], rtol=1e-5, atol=1e-7)
    loss2 = model(ids, labels=ids).loss
    torch.testing.assert_close(loss2.cpu(), golden_tiny['loss_after_step'], rtol=1e-4, atol=1e-5)


def test_tiny_bf16_all_gradients_close_to_oracle():
    c = recipe.tiny_config()
    state = {k: v.to(torch.bfloat16).float() for k, v in recipe.seeded_state(c, norm_jitter=0.1).items()}
    model = build('triton_optimized', state, torch.bfloat16)
    ids = recipe.seeded_ids(c, batch=2, seq=129, seed=7).cuda()
    out = model(ids, labels=ids)
    out.loss.backward()
    oracle = OracleQwen3(c, state=state)
    loss, logits = oracle(ids.cpu(), ids.cpu())
    loss.backward()
    assert abs(float(out.loss) - float(loss)) / float(loss) < 1e-3            # loss within 1e-3 relative
    assert rel_l2(out.logits, logits) < 2e-2
    for name, p in model.named_parameters():
        # per-tensor relative L2 (the reference's own whole-model gate is 0.06; ours is tighter)
        assert rel_l2(p.grad, oracle.p(name).grad) < 3e-2, name


def test_vocab_parallel_head_fused_world1_matches_dense_loss():
    """Default VocabParallelCE path: no logits shard in memory."""
    from qwen3_triton.kernels.linear import linear
    from qwen3_triton.kernels.loss import causal_cross_entropy
    from qwen3_triton.training.vocab_parallel import VocabParallelCE
    g = torch.Generator().manual_seed(12)
    B, S, H, V = 2, 65, 256, 4104
    hidden = torch.randn(B, S, H, generator=g).to(torch.bfloat16)
    weight = torch.randn(V, H, generator=g) * 0.05
    labels = torch.randint(0, V, (B, S), generator=g)
    labels[1, 4] = -100
    head = VocabParallelCE(weight, chunk=1024)
    h1 = hidden.cuda().requires_grad_(True)
    loss, dense = head(h1, labels.cuda())
    assert dense is None
    loss.backward()
    h2 = hidden.cuda().requires_grad_(True)
    w2 = weight.to(torch.bfloat16).cuda().requires_grad_(True)
    ref = causal_cross_entropy(linear(h2, w2), labels.cuda())
    ref.backward()
    torch.testing.assert_close(loss, ref, rtol=1e-5, atol=1e-5)
    close(h1.grad, h2.grad, what='dx')
    close(head.weight.grad, w2.grad.float(), dtype=torch.bfloat16, what='dw')
    assert head.weight.grad.dtype == torch.float32


def test_vocab_parallel_head_world1_matches_dense_loss():
    from qwen3_triton.kernels.linear import linear
    from qwen3_triton.kernels.loss import causal_cross_entropy
    from qwen3_triton.training.vocab_parallel import VocabParallelCE
    g = torch.Generator().manual_seed(11)
    B, S, H, V = 2, 33, 256, 1000
    hidden = torch.randn(B, S, H, generator=g).to(torch.bfloat16)
    weight = (torch.randn(V, H, generator=g) * 0.05)
    labels = torch.randint(0, V, (B, S), generator=g)
    labels[1, 4] = -100
    head = VocabParallelCE(weight, fused=False)
    h1 = hidden.cuda().requires_grad_(True)
    loss, dense = head(h1, labels.cuda(), diagnostics=True)
    loss.backward()
    h2 = hidden.cuda().requires_grad_(True)
    w2 = weight.to(torch.bfloat16).cuda().requires_grad_(True)
    logits = linear(h2, w2)
    ref = causal_cross_entropy(logits, labels.cuda())
    ref.backward()
    torch.testing.assert_close(loss, ref, rtol=1e-5, atol=1e-6)
    assert torch.equal(dense, logits)
    close(h1.grad, h2.grad, what='dx')
    close(head.weight.grad, w2.grad.float(), dtype=torch.bfloat16, what='dw')
    assert head.weight.grad.dtype == torch.float32 and head.forward_calls == 1 and head.backward_calls == 1


def small_d128_config():
    from types import SimpleNamespace
    return SimpleNamespace(model_type='qwen3', hidden_act='silu', attention_dropout=0.0, attention_bias=False,
                           use_sliding_window=False, rope_scaling=None, vocab_size=1024, hidden_size=256,
                           intermediate_size=512, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                           head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6, initializer_range=0.02,
                           tie_word_embeddings=False)


@pytest.mark.parametrize('seq', [256, 200])
def test_fused_decoder_layers_match_operator_graph_and_oracle(seq):
    """The fused-layer graph (token-major attention, folded residual adds, hand-written backward) against the
    operator-level graph in bf16 and against the fp32 oracle; recompute on/off must agree bit for bit."""
    from qwen3_triton import model_for_variant
    c = small_d128_config()
    state = {k: v.to(torch.bfloat16).float() for k, v in recipe.seeded_state(c, seed=5, norm_jitter=0.1).items()}
    ids = recipe.seeded_ids(c, batch=2, seq=seq, seed=6).cuda()

    def run(variant, recompute=False):
        model = model_for_variant(c, variant)
        model.load_hf_state_dict({k: v.clone() for k, v in state.items()})
        model = model.to('cuda', torch.bfloat16)
        if variant == 'b200_fused':
            model.model.set_recompute(recompute)
        out = model(ids, labels=ids)
        out.loss.backward()
        return out, {n: p.grad.clone() for n, p in model.named_parameters()}

    out_f, g_f = run('b200_fused')
    out_r, g_r = run('b200_fused', recompute='full')
    out_s, g_s = run('b200_fused', recompute='selective')
    assert torch.equal(out_f.loss, out_s.loss)
    for n in g_f:
        assert torch.equal(g_f[n], g_s[n]), n
    out_o, g_o = run('triton_optimized')
    assert torch.equal(out_f.loss, out_r.loss)
    for n in g_f:
        assert torch.equal(g_f[n], g_r[n]), n
    oracle = OracleQwen3(c, state=state)
    loss, logits = oracle(ids.cpu(), ids.cpu())
    loss.backward()
    assert abs(float(out_f.loss) - float(loss)) / float(loss) < 1e-3
    assert abs(float(out_f.loss) - float(out_o.loss)) / float(loss) < 1e-3
    assert rel_l2(out_f.logits, logits) < 2e-2
    for n in g_f:
        # per-tensor relative L2; the 64/128-element QK-norm weight gradients are the noisiest tensors in bf16
        # (the reference's own whole-model gate is 6e-2 per tensor)
        assert rel_l2(g_f[n], oracle.p(n).grad) < 4e-2, n
        assert rel_l2(g_f[n], g_o[n]) < 4e-2, n


def test_weight_gradients_on_a_second_stream_change_nothing():
    """fused.WeightGradientStream (off by default): the four weight-gradient GEMMs of a layer's backward issued on a
    side stream, joined before the layer's backward returns. Same kernels on the same inputs: every gradient must be
    bit-identical, three steps in a row (the side stream's tensors are reused through the allocator)."""
    from qwen3_triton import fused, model_for_variant
    c = small_d128_config()
    state = {k: v.to(torch.bfloat16).float() for k, v in recipe.seeded_state(c, seed=7, norm_jitter=0.1).items()}
    ids = recipe.seeded_ids(c, batch=2, seq=256, seed=8).cuda()

    def run(side):
        model = model_for_variant(c, 'b200_fused')
        model.load_hf_state_dict({k: v.clone() for k, v in state.items()})
        model = model.to('cuda', torch.bfloat16)
        previous = fused.WeightGradientStream.enabled
        fused.WeightGradientStream.enabled = side
        try:
            for _ in range(3):
                model.zero_grad(set_to_none=True)
                out = model(ids, labels=ids)
                out.loss.backward()
            torch.cuda.synchronize()
        finally:
            fused.WeightGradientStream.enabled = previous
        return out.loss.detach().clone(), {n: p.grad.clone() for n, p in model.named_parameters()}

    loss_a, grads_a = run(False)
    loss_b, grads_b = run(True)
    assert torch.equal(loss_a, loss_b)
    for n in grads_a:
        assert torch.equal(grads_a[n], grads_b[n]), n


@pytest.mark.parametrize('B,S,H,V,chunk', [(2, 33, 256, 1000, 256), (1, 300, 512, 4104, 1024), (3, 17, 128, 520, 16384)])
def test_fused_linear_cross_entropy_matches_materialised_path(B, S, H, V, chunk):
    """hidden -> loss without logits in memory == causal_cross_entropy(linear(hidden, W)) and the fp32 oracle."""
    from oracle import ops as O
    from qwen3_triton.kernels.fused_loss import fused_linear_cross_entropy
    from qwen3_triton.kernels.linear import linear
    from qwen3_triton.kernels.loss import causal_cross_entropy
    g = torch.Generator().manual_seed(21)
    hidden = torch.randn(B, S, H, generator=g).to(torch.bfloat16)
    weight = (torch.randn(V, H, generator=g) * 0.1).to(torch.bfloat16)
    labels = torch.randint(0, V, (B, S), generator=g)
    if S > 6:
        labels[0, 5] = -100
    h1, w1 = hidden.cuda().requires_grad_(True), weight.cuda().requires_grad_(True)
    loss = fused_linear_cross_entropy(h1, w1, labels.cuda(), chunk=chunk)
    (loss * 2.0).backward()
    h2, w2 = hidden.cuda().requires_grad_(True), weight.cuda().requires_grad_(True)
    ref = causal_cross_entropy(linear(h2, w2), labels.cuda())
    (ref * 2.0).backward()
    torch.testing.assert_close(loss, ref, rtol=1e-5, atol=1e-5)
    close(h1.grad, h2.grad, what='dx vs materialised')
    close(w1.grad, w2.grad, what='dw vs materialised')
    logits = O.linear(hidden, weight).to(torch.bfloat16)
    assert abs(float(loss) - float(O.causal_cross_entropy(logits.view(B, S, V), labels))) / float(ref) < 1e-3
