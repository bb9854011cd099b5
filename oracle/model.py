"""fp32 CPU Qwen3 decoder built from the oracle ops, with autograd. TEST INFRASTRUCTURE ONLY.

Follows the graph of the reference model/qwen_tiny.py:105-231 (embedding, per layer RMSNorm -> q/k/v ->
per-head QK RMSNorm -> RoPE -> causal GQA attention -> o_proj -> residual -> RMSNorm -> SwiGLU MLP ->
residual, final RMSNorm, untied lm_head, internally shifted cross-entropy) with the official Qwen3
parameter names, so one state dict drives both this model and the CUDA model.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import nn


def _rms(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def _rot(x):
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


class OracleQwen3(nn.Module):
    def __init__(self, cfg, state=None, seed=0):
        super().__init__()
        self.cfg = cfg
        gen = torch.Generator().manual_seed(seed)
        c = cfg
        shapes = {'model.embed_tokens.weight': (c.vocab_size, c.hidden_size), 'model.norm.weight': (c.hidden_size,),
                  'lm_head.weight': (c.vocab_size, c.hidden_size)}
        for i in range(c.num_hidden_layers):
            p = f'model.layers.{i}.'
            shapes.update({
                p + 'self_attn.q_proj.weight': (c.num_attention_heads * c.head_dim, c.hidden_size),
                p + 'self_attn.k_proj.weight': (c.num_key_value_heads * c.head_dim, c.hidden_size),
                p + 'self_attn.v_proj.weight': (c.num_key_value_heads * c.head_dim, c.hidden_size),
                p + 'self_attn.o_proj.weight': (c.hidden_size, c.num_attention_heads * c.head_dim),
                p + 'self_attn.q_norm.weight': (c.head_dim,), p + 'self_attn.k_norm.weight': (c.head_dim,),
                p + 'mlp.gate_proj.weight': (c.intermediate_size, c.hidden_size),
                p + 'mlp.up_proj.weight': (c.intermediate_size, c.hidden_size),
                p + 'mlp.down_proj.weight': (c.hidden_size, c.intermediate_size),
                p + 'input_layernorm.weight': (c.hidden_size,), p + 'post_attention_layernorm.weight': (c.hidden_size,),
            })
        self.names = list(shapes)
        self.params = nn.ParameterDict()
        for name, shape in shapes.items():
            if state is not None:
                value = state[name].detach().float().clone()
            elif len(shape) == 1:
                value = torch.ones(shape)
            else:
                value = torch.randn(shape, generator=gen) * c.initializer_range
            self.params[name.replace('.', '/')] = nn.Parameter(value)

    def p(self, name):
        return self.params[name.replace('.', '/')]

    def state(self):
        return {n: self.p(n).detach().clone() for n in self.names}

    def grads(self):
        return {n: self.p(n).grad.detach().clone() for n in self.names if self.p(n).grad is not None}

    def hidden(self, ids):
        c = self.cfg
        b, s = ids.shape
        x = self.p('model.embed_tokens.weight')[ids]
        pos = torch.arange(s, dtype=torch.float32)
        freq = 1.0 / (c.rope_theta ** (torch.arange(0, c.head_dim, 2, dtype=torch.float32) / c.head_dim))
        ang = torch.cat((pos[:, None] * freq, pos[:, None] * freq), -1)
        cos, sin = ang.cos()[None, None], ang.sin()[None, None]
        mask = torch.ones(s, s, dtype=torch.bool).tril()
        g = c.num_attention_heads // c.num_key_value_heads
        for i in range(c.num_hidden_layers):
            pre = f'model.layers.{i}.'
            h = _rms(x, self.p(pre + 'input_layernorm.weight'), c.rms_norm_eps)
            q = F.linear(h, self.p(pre + 'self_attn.q_proj.weight')).view(b, s, c.num_attention_heads, c.head_dim)
            k = F.linear(h, self.p(pre + 'self_attn.k_proj.weight')).view(b, s, c.num_key_value_heads, c.head_dim)
            v = F.linear(h, self.p(pre + 'self_attn.v_proj.weight')).view(b, s, c.num_key_value_heads, c.head_dim)
            q = _rms(q, self.p(pre + 'self_attn.q_norm.weight'), c.rms_norm_eps).transpose(1, 2)
            k = _rms(k, self.p(pre + 'self_attn.k_norm.weight'), c.rms_norm_eps).transpose(1, 2)
            v = v.transpose(1, 2)
            q = q * cos + _rot(q) * sin
            k = k * cos + _rot(k) * sin
            k = k.repeat_interleave(g, dim=1)
            v = v.repeat_interleave(g, dim=1)
            sc = torch.matmul(q, k.transpose(-2, -1)) / math.sqrt(c.head_dim)
            sc = sc.masked_fill(~mask, float('-inf'))
            a = torch.matmul(torch.softmax(sc, -1), v).transpose(1, 2).reshape(b, s, -1)
            x = x + F.linear(a, self.p(pre + 'self_attn.o_proj.weight'))
            h = _rms(x, self.p(pre + 'post_attention_layernorm.weight'), c.rms_norm_eps)
            m = F.silu(F.linear(h, self.p(pre + 'mlp.gate_proj.weight'))) * F.linear(h, self.p(pre + 'mlp.up_proj.weight'))
            x = x + F.linear(m, self.p(pre + 'mlp.down_proj.weight'))
        return _rms(x, self.p('model.norm.weight'), c.rms_norm_eps)

    def forward(self, ids, labels=None):
        logits = F.linear(self.hidden(ids), self.p('lm_head.weight'))
        loss = None
        if labels is not None:
            v = logits.shape[-1]
            loss = F.cross_entropy(logits[:, :-1].reshape(-1, v), labels[:, 1:].reshape(-1), ignore_index=-100)
        return loss, logits
