"""CPU restatement of the decode-time operators. TEST INFRASTRUCTURE ONLY (imported by tests/ alone).

Restates the arithmetic of the reference's qwen3_triton/inference/kernels.py in plain torch CPU ops: cache append
(:25-36: token-major [B,S,H,D] into [B,H,C,D] at `start`), attention of new queries over the cache (:39-66: key t is
visible to query s iff t <= start + s and t < start + S, softmax scale D^-1/2, kv head = q head // (Hq/Hkv)), the
small-M linear (:117-129), and the greedy selection step (:150-166: lowest index among equal maxima, pad for finished
rows, finished |= token in eos). The reference ships no tests or stored outputs for this module, so this oracle is
pinned only against textbook definitions (torch.softmax / torch.argmax): parity unpinned.
"""
import torch


def append(k, v, cache_k, cache_v, start):
    s = k.shape[1]
    cache_k[:, :, start:start + s] = k.transpose(1, 2)
    cache_v[:, :, start:start + s] = v.transpose(1, 2)


def attention(q, cache_k, cache_v, start):
    b, s, hq, d = q.shape
    hk = cache_k.shape[1]
    total = start + s
    k = cache_k[:, :, :total].float().repeat_interleave(hq // hk, dim=1)       # [B,Hq,T,D]
    v = cache_v[:, :, :total].float().repeat_interleave(hq // hk, dim=1)
    scores = torch.einsum('bshd,bhtd->bhst', q.float(), k) * d ** -0.5
    t = torch.arange(total)[None, :]
    visible = t <= (start + torch.arange(s))[:, None]
    scores = scores.masked_fill(~visible, float('-inf'))
    return torch.einsum('bhst,bhtd->bshd', torch.softmax(scores, dim=-1), v)


def linear(x, weight, accurate=False):
    dt = torch.float64 if accurate else torch.float32
    return (x.to(dt) @ weight.to(dt).t()).float()


def select(logits, ids, next_token, done, position, eos, pad):
    best = logits.float().max(dim=1, keepdim=True).values
    index = torch.arange(logits.shape[1])[None].expand_as(logits)
    token = torch.where(logits.float() == best, index, torch.full_like(index, 2 ** 62)).min(dim=1).values
    token = torch.where(done, torch.full_like(token, pad), token)
    ids[:, position] = token
    next_token.view(-1).copy_(token)
    done |= torch.isin(token, torch.tensor(list(eos), dtype=torch.int64))
