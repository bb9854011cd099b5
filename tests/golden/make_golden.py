"""Generate tests/golden/*.npz by RUNNING THE REFERENCE's own CPU code (ops/reference and model/).

Run in a container that has the reference checkout:
    python tests/golden/make_golden.py /path/to/reference
The outputs are committed; tests never need the reference at run time.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
import recipe  # noqa: E402


def main(ref_root):
    sys.path.insert(0, ref_root)
    from ops.reference.attention import (scaled_dot_product_attention_backward_reference,
                                         scaled_dot_product_attention_reference)
    from ops.reference.fused_qk_norm_rope import fused_qk_norm_rope_backward_reference, fused_qk_norm_rope_reference
    from ops.reference.rms_norm import rms_norm_reference
    from ops.reference.rope import apply_rope_backward_reference, apply_rope_reference, rotate_half_reference
    from ops.reference.swiglu import swiglu_reference
    from model import TinyQwenConfig, TinyQwenForCausalLM

    torch.set_num_threads(1)
    d = recipe.op_inputs()
    out = {}
    out['rms_norm'] = rms_norm_reference(d['norm_x'], d['norm_w'], 1e-6)
    x = d['norm_x'].clone().requires_grad_(True)
    w = d['norm_w'].clone().requires_grad_(True)
    rms_norm_reference(x, w, 1e-6).backward(d['norm_dy'])
    out['rms_norm_dx'], out['rms_norm_dw'] = x.grad, w.grad
    out['rotate_half_arange8'] = rotate_half_reference(torch.arange(8.))
    q_r, k_r = apply_rope_reference(d['q'], d['k'], d['cos'], d['sin'])
    out['rope_q'], out['rope_k'] = q_r, k_r
    gq, gk = apply_rope_backward_reference(d['do'], d['k'], d['cos'], d['sin'])
    out['rope_bwd_q'], out['rope_bwd_k'] = gq, gk
    fq, fk = fused_qk_norm_rope_reference(d['qn'], d['kn'], d['qw'], d['kw'], d['cos'], d['sin'], 1e-6)
    out['fused_q'], out['fused_k'] = fq, fk
    dq, dk, dqw, dkw = fused_qk_norm_rope_backward_reference(d['qn'], d['kn'], d['qw'], d['kw'], d['cos'], d['sin'],
                                                             d['dqn'], d['dkn'], 1e-6)
    out['fused_dq'], out['fused_dk'], out['fused_dqw'], out['fused_dkw'] = dq, dk, dqw, dkw
    out['swiglu'] = swiglu_reference(d['gate'], d['up'])
    g = d['gate'].clone().requires_grad_(True)
    u = d['up'].clone().requires_grad_(True)
    swiglu_reference(g, u).backward(d['dy_act'])
    out['swiglu_dg'], out['swiglu_du'] = g.grad, u.grad
    out['attn'] = scaled_dot_product_attention_reference(d['q'], d['k'], d['v'], is_causal=True, enable_gqa=True)
    aq, ak, av = scaled_dot_product_attention_backward_reference(d['q'], d['k'], d['v'], d['do'], is_causal=True,
                                                                 enable_gqa=True)
    out['attn_dq'], out['attn_dk'], out['attn_dv'] = aq, ak, av
    np.savez_compressed(HERE / 'ops.npz', **{k: v.detach().numpy() for k, v in out.items()})

    # The tiny decoder (2 layers, hidden 256, 4/2 heads of 64, vocab 2048): one forward + CE + backward + AdamW step on
    # CPU in fp32.
    c = recipe.tiny_config()
    cfg = TinyQwenConfig(vocab_size=c.vocab_size, hidden_size=c.hidden_size, intermediate_size=c.intermediate_size,
                         num_hidden_layers=c.num_hidden_layers, num_attention_heads=c.num_attention_heads,
                         num_key_value_heads=c.num_key_value_heads, head_dim=c.head_dim, rope_theta=c.rope_theta,
                         rms_norm_eps=c.rms_norm_eps, tie_word_embeddings=False)
    model = TinyQwenForCausalLM(cfg)
    model.load_state_dict(recipe.seeded_state(c), strict=True)
    ids = recipe.seeded_ids(c)
    opt = torch.optim.AdamW(model.parameters(), **recipe.ADAMW)
    res = model(ids, labels=ids)
    res['loss'].backward()
    tiny = {'loss': res['loss'].detach().numpy(), 'logits_slice': res['logits'][0, :4, :16].detach().numpy()}
    for name, p in model.named_parameters():
        tiny['gradnorm/' + name] = p.grad.norm().numpy()
        tiny['gradslice/' + name] = p.grad.reshape(-1)[:32].clone().numpy()
    opt.step()
    for name, p in model.named_parameters():
        tiny['stepslice/' + name] = p.detach().reshape(-1)[:32].clone().numpy()
    loss2 = model(ids, labels=ids)['loss']
    tiny['loss_after_step'] = loss2.detach().numpy()
    np.savez_compressed(HERE / 'tiny_model.npz', **tiny)
    print('wrote', HERE / 'ops.npz', HERE / 'tiny_model.npz')


DATA_CASES = [  # corpus tokens, seq, seed, offset
    (51, 5, 42, 0), (1000, 7, 20261102, 0), (104729 * 3 + 5, 3, 1, 17), (209458 * 2, 2, 123456789, 5), (64, 8, 0, 3)]
VALIDATION_CASES = [(1, 4, 4), (17, 4, 4), (32, 4, 4), (7, 2, 3), (9, 1, 2)]   # blocks, world, batch


def data_fixtures(ref_root):
    """training/data.py and training/evaluation.py of the reference, run on small synthetic corpora (token value =
    position, so a block identifies itself): served block indices, strides, the validation partition and the shifted
    NLL of seeded logits."""
    import tempfile
    sys.path.insert(0, ref_root)
    from training.data import Blocks
    from training.evaluation import shifted_nll, validation_batches
    out = {}
    with tempfile.TemporaryDirectory() as tmp:
        for case, (tokens, seq, seed, offset) in enumerate(DATA_CASES):
            path = Path(tmp) / f'c{case}.bin'
            np.arange(tokens, dtype='<u4').tofile(path)
            train = Blocks(path, seq, offset=offset, training=True, seed=seed)
            plain = Blocks(path, seq)
            count = min(len(train), 64)
            out[f'data{case}/meta'] = np.array([tokens, seq, seed, offset, len(train), train.stride], dtype=np.int64)
            out[f'data{case}/train_first_tokens'] = np.array([int(train[i][0]) for i in range(count)], dtype=np.int64)
            out[f'data{case}/wrap_first_tokens'] = np.array([int(train[len(train) + i][0]) for i in range(4)], dtype=np.int64)
            out[f'data{case}/eval_last_block'] = plain[len(plain) - 1].numpy()
    gen = torch.Generator().manual_seed(7)
    for case, (size, world, batch) in enumerate(VALIDATION_CASES):
        ids = torch.randint(0, 11, (size, 6), generator=gen)
        table = torch.randn(size, 6, 11, generator=gen)
        masks, served, total, count = [], [], 0.0, 0
        for rank in range(world):
            for call, (data, valid) in enumerate(validation_batches(list(ids), rank, world, batch)):
                start = call * world * batch + rank * batch
                logits = torch.stack([table[i] if i < size else table[0] for i in range(start, start + batch)])
                n, c = shifted_nll(logits, data, valid)
                total += float(n)
                count += int(c)
                masks.append(valid.numpy())
                served.append(data.numpy())
        out[f'val{case}/meta'] = np.array([size, world, batch], dtype=np.int64)
        out[f'val{case}/ids'] = ids.numpy()
        out[f'val{case}/table'] = table.numpy()
        out[f'val{case}/valid'] = np.stack(masks)
        out[f'val{case}/served'] = np.stack(served)
        out[f'val{case}/total_count'] = np.array([total, count], dtype=np.float64)
    np.savez_compressed(HERE / 'data.npz', **out)
    print('wrote', HERE / 'data.npz')


if __name__ == '__main__':
    args = [a for a in sys.argv[1:] if a != '--data-only']
    if len(args) != 1:
        raise SystemExit('usage: make_golden.py [--data-only] <path to a checkout of the reference repository>')
    if '--data-only' not in sys.argv:
        main(args[0])
    data_fixtures(args[0])
