"""Seeded inputs shared by the fixture generator and the tests (no dependency on the reference)."""
from __future__ import annotations

from types import SimpleNamespace

import torch

TINY = dict(vocab_size=2048, hidden_size=256, intermediate_size=688, num_hidden_layers=2, num_attention_heads=4,
            num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-6, rope_theta=1e6, initializer_range=0.02,
            tie_word_embeddings=False)
TINY_SEED = 20261114
ADAMW = dict(lr=1e-4, betas=(0.9, 0.95), weight_decay=0.1, eps=1e-8)


def tiny_config():
    return SimpleNamespace(model_type='qwen3', hidden_act='silu', attention_dropout=0.0, attention_bias=False,
                           use_sliding_window=False, rope_scaling=None, **TINY)


def param_shapes(c):
    shapes = {'model.embed_tokens.weight': (c.vocab_size, c.hidden_size)}
    for i in range(c.num_hidden_layers):
        p = f'model.layers.{i}.'
        shapes[p + 'input_layernorm.weight'] = (c.hidden_size,)
        shapes[p + 'self_attn.q_proj.weight'] = (c.num_attention_heads * c.head_dim, c.hidden_size)
        shapes[p + 'self_attn.k_proj.weight'] = (c.num_key_value_heads * c.head_dim, c.hidden_size)
        shapes[p + 'self_attn.v_proj.weight'] = (c.num_key_value_heads * c.head_dim, c.hidden_size)
        shapes[p + 'self_attn.o_proj.weight'] = (c.hidden_size, c.num_attention_heads * c.head_dim)
        shapes[p + 'self_attn.q_norm.weight'] = (c.head_dim,)
        shapes[p + 'self_attn.k_norm.weight'] = (c.head_dim,)
        shapes[p + 'post_attention_layernorm.weight'] = (c.hidden_size,)
        shapes[p + 'mlp.gate_proj.weight'] = (c.intermediate_size, c.hidden_size)
        shapes[p + 'mlp.up_proj.weight'] = (c.intermediate_size, c.hidden_size)
        shapes[p + 'mlp.down_proj.weight'] = (c.hidden_size, c.intermediate_size)
    shapes['model.norm.weight'] = (c.hidden_size,)
    shapes['lm_head.weight'] = (c.vocab_size, c.hidden_size)
    return shapes


def seeded_state(c, seed=TINY_SEED, norm_jitter=0.0):
    """Matrices ~ N(0, initializer_range), norm weights = 1 (+ optional jitter so their gradients matter)."""
    gen = torch.Generator().manual_seed(seed)
    state = {}
    for name, shape in param_shapes(c).items():
        if len(shape) == 1:
            state[name] = torch.ones(shape) + norm_jitter * torch.randn(shape, generator=gen)
        else:
            state[name] = torch.randn(shape, generator=gen) * c.initializer_range
    return state


def seeded_ids(c, batch=2, seq=128, seed=TINY_SEED + 1):
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, c.vocab_size, (batch, seq), generator=gen)


def op_inputs(seed=20261115):
    """Small fp32 inputs for every operator fixture."""
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    d = {}
    d['norm_x'], d['norm_w'], d['norm_dy'] = r(3, 5, 96), 1 + 0.1 * r(96), r(3, 5, 96)
    B, S, HQ, HK, D = 2, 7, 4, 2, 32
    d['q'], d['k'], d['v'], d['do'] = r(B, HQ, S, D), r(B, HK, S, D), r(B, HK, S, D), r(B, HQ, S, D)
    d['qn'], d['kn'] = r(B, S, HQ, D), r(B, S, HK, D)            # [B,S,heads,D] layout for norm+rope
    d['qw'], d['kw'] = 1 + 0.1 * r(D), 1 + 0.1 * r(D)
    d['cos'], d['sin'] = r(B, S, D), r(B, S, D)                  # independent halves on purpose
    d['dqn'], d['dkn'] = r(B, S, HQ, D), r(B, S, HK, D)
    d['gate'], d['up'], d['dy_act'] = r(4, 6, 40), r(4, 6, 40), r(4, 6, 40)
    return d
