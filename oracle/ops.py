"""fp32 CPU restatement of the reference operator math. TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

Each function names the reference lines it follows. Inputs of any float dtype are promoted to fp32; the
result is returned in fp32 unless stated, so callers round once when they compare with a bf16 kernel.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def _f(t):
    return t.detach().to(torch.float32)


# ---------------------------------------------------------------- RMSNorm
def rms_norm(x, weight, eps=1e-6):
    """ops/reference/rms_norm.py:6-13 - variance over the last dim in fp32, rsqrt, weight after."""
    x, w = _f(x), _f(weight)
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def rms_norm_backward(x, weight, dy, eps=1e-6):
    """ops/reference/fused_qk_norm_rope.py:63-76 (rms_backward): (dx, dweight)."""
    x, w, dy = _f(x), _f(weight), _f(dy)
    inv = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    wg = dy * w
    corr = (wg * x).mean(-1, keepdim=True)
    dx = (wg - x * inv.pow(2) * corr) * inv
    dw = (dy * x * inv).reshape(-1, x.shape[-1]).sum(0)
    return dx, dw


def add_rms_norm(x, residual, weight, eps=1e-6, round_dtype=None):
    """Residual add (qwen3_triton/kernels/residual.py:7-11) followed by RMSNorm; the sum is rounded to
    `round_dtype` first when given, because that rounded tensor is what the next op reads."""
    r = _f(x) + _f(residual)
    if round_dtype is not None:
        r = r.to(round_dtype).float()
    return rms_norm(r, weight, eps), r


# ---------------------------------------------------------------- RoPE
def rotate_half(x):
    """ops/reference/rope.py:6-9: (-second half, first half)."""
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def rotate_half_transposed(x):
    """ops/reference/rope.py:31-34: (second half, -first half)."""
    h = x.shape[-1] // 2
    return torch.cat((x[..., h:], -x[..., :h]), dim=-1)


def rope_tables(position_ids, inv_freq):
    """qwen3_triton/kernels/rotary.py:12-17: angle = float(pos) * inv_freq[i % (D/2)]; fp32 cos, sin [B,S,D]."""
    angle = position_ids.to(torch.float32)[..., None] * inv_freq.to(torch.float32)
    angle = torch.cat((angle, angle), dim=-1)
    return angle.cos(), angle.sin()


def inv_freq(head_dim, theta=1e6):
    """qwen3_triton/_model.py:54."""
    return 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))


def apply_rope(x, cos, sin, heads_dim):
    """ops/reference/rope.py:13-28. cos/sin [B,S,D]; heads_dim is the index of the heads axis of x
    (1 for [B,H,S,D], 2 for [B,S,H,D])."""
    x, c, s = _f(x), _f(cos).unsqueeze(heads_dim), _f(sin).unsqueeze(heads_dim)
    return x * c + rotate_half(x) * s


def apply_rope_backward(dy, cos, sin, heads_dim):
    """ops/reference/rope.py:37-55: dy*cos + R^T(dy*sin)."""
    dy, c, s = _f(dy), _f(cos).unsqueeze(heads_dim), _f(sin).unsqueeze(heads_dim)
    return dy * c + rotate_half_transposed(dy * s)


def norm_rope(x, weight, cos, sin, eps=1e-6):
    """ops/reference/fused_qk_norm_rope.py:9-33 for one tensor x [B,S,heads,D]."""
    return apply_rope(rms_norm(x, weight, eps), cos, sin, 2)


def norm_rope_backward(x, weight, cos, sin, dy, eps=1e-6):
    """ops/reference/fused_qk_norm_rope.py:36-80 for one tensor: (dx, dweight)."""
    return rms_norm_backward(x, weight, apply_rope_backward(dy, cos, sin, 2), eps)


# ---------------------------------------------------------------- SwiGLU
def swiglu(gate, up):
    """ops/reference/swiglu.py:9-21."""
    return F.silu(_f(gate)) * _f(up)


def swiglu_backward(gate, up, dy):
    """Derivative of silu(g)*u: dg = dy*u*s*(1+g*(1-s)), du = dy*g*s (qwen3_triton/kernels/activation.py:14-20)."""
    g, u, dy = _f(gate), _f(up), _f(dy)
    s = torch.sigmoid(g)
    return dy * u * s * (1 + g * (1 - s)), dy * g * s


# ---------------------------------------------------------------- attention
def _expand_kv(t, groups):
    return t.repeat_interleave(groups, dim=1) if groups > 1 else t


def attention(q, k, v, scale=None):
    """ops/reference/attention.py:10-54 (causal, GQA). Returns (out, lse) in fp32; lse is the natural-log
    sum-exp of the scaled masked scores, [B,Hq,S] (reference tests/test_attention_triton.py:36-47)."""
    q, k, v = _f(q), _f(k), _f(v)
    d = q.shape[-1]
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    g = q.shape[1] // k.shape[1]
    k, v = _expand_kv(k, g), _expand_kv(v, g)
    s = torch.matmul(q, k.transpose(-2, -1)) * scale
    n = q.shape[2]
    mask = torch.ones(n, n, dtype=torch.bool).tril()
    s = s.masked_fill(~mask, float('-inf'))
    lse = torch.logsumexp(s, dim=-1)
    return torch.matmul(torch.softmax(s, dim=-1), v), lse


def attention_backward(q, k, v, dout, scale=None, saved_out=None):
    """ops/reference/attention.py:57-124: dV = P^T dO, dP = dO V^T, dS = P*(dP - sum(dP*P)),
    dQ = scale*dS K, dK = scale*dS^T Q, expanded K/V grads summed back per kv head.

    With `saved_out` (the forward output as it was stored, e.g. rounded to bf16) the row term sum(dP*P) is replaced
    by rowsum(dO * saved_out): algebraically the same number, and the form every flash-attention backward uses
    because P is not kept (the reference's kernels do: qwen3_triton/kernels/attention_precision.py:69-76,100 `delta`). The
    rounding of the stored output then enters dS exactly as it does in the kernels."""
    q, k, v, dout = _f(q), _f(k), _f(v), _f(dout)
    b, hq, n, d = q.shape
    hk = k.shape[1]
    g = hq // hk
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    ke, ve = _expand_kv(k, g), _expand_kv(v, g)
    s = torch.matmul(q, ke.transpose(-2, -1)) * scale
    mask = torch.ones(n, n, dtype=torch.bool).tril()
    p = torch.softmax(s.masked_fill(~mask, float('-inf')), dim=-1)
    dv = torch.matmul(p.transpose(-2, -1), dout)
    dp = torch.matmul(dout, ve.transpose(-2, -1))
    row = (dp * p).sum(-1, keepdim=True) if saved_out is None else (dout * _f(saved_out)).sum(-1, keepdim=True)
    ds = p * (dp - row)
    dq = torch.matmul(ds, ke) * scale
    dk = torch.matmul(ds.transpose(-2, -1), q) * scale
    dk = dk.view(b, hk, g, n, d).sum(2)
    dv = dv.view(b, hk, g, n, d).sum(2)
    return dq, dk, dv


# ---------------------------------------------------------------- linear / embedding / loss
def linear(x, weight):
    """y = x W^T in fp32 (the reference checks its GEMMs against torch.mm: scripts/tune_qwen3_ampere_gemm.py:130)."""
    return F.linear(_f(x), _f(weight))


def embedding(ids, weight):
    return _f(weight)[ids.long()]


def embedding_backward(ids, dy, vocab):
    dy = _f(dy)
    dw = torch.zeros(vocab, dy.shape[-1], dtype=torch.float32)
    dw.index_add_(0, ids.reshape(-1).long(), dy.reshape(-1, dy.shape[-1]))
    return dw


def causal_cross_entropy(logits, labels, ignore_index=-100):
    """Shift inside the op, token mean over non-ignored targets, fp32 logits
    (model/qwen_tiny.py:224-227; training/evaluation.py:20-26)."""
    logits = logits.to(torch.float32)  # keeps the autograd graph when the caller asked for one
    v = logits.shape[-1]
    return F.cross_entropy(logits[:, :-1].reshape(-1, v), labels[:, 1:].reshape(-1), ignore_index=ignore_index)


def causal_cross_entropy_backward(logits, labels, ignore_index=-100, upstream=1.0):
    """d loss / d logits: (softmax - onehot) * upstream / count on scored rows, zero elsewhere."""
    x = _f(logits).clone().requires_grad_(True)
    causal_cross_entropy(x, labels, ignore_index).backward(torch.tensor(float(upstream)))
    return x.grad


# ---------------------------------------------------------------- AdamW
def adamw_step(p, g, m, v, step, lr, beta1, beta2, eps, weight_decay):
    """One decoupled-decay Adam step in fp64, returning fp32 (p, m, v). Order: decay, moments, bias
    corrections bc1 = 1-b1^t, bc2 = 1-b2^t, step size lr/bc1, denominator sqrt(v)/sqrt(bc2)+eps
    (qwen3_triton/runtime/adamw.py:52-60; the independent check in scripts/check_triton_adamw_v14.py:37-47).
    `step` is the step count AFTER the increment (1 for the first step)."""
    p, g, m, v = (t.detach().to(torch.float64) for t in (p, g, m, v))
    p = p - lr * weight_decay * p
    m = beta1 * m + (1 - beta1) * g
    v = beta2 * v + (1 - beta2) * g * g
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    p = p - (lr / bc1) * m / (v.sqrt() / math.sqrt(bc2) + eps)
    return p.float(), m.float(), v.float()
