"""Decode-time operators: positions, KV-cache append, attention over the cache, small-M linear and greedy selection.

Same functions and argument meaning as the reference's qwen3_triton/inference/kernels.py (positions :19-22, append
:33-36, attention :103-115, linear :131-148, select :168-173, rms_norm :176-186, norm_rope :189-194); every one is a
launch into csrc/libq3b200.so. The reference keeps several variants per operator that reproduce another library's
rounding order on its GPU (`sliced`, `prefill_tiling`, `reference_accumulation`, 32- versus 64-key tiles); those
switches are accepted and select nothing here - there is one kernel per operator, fp32 accumulation (fp64 for
`accurate`), and the cache attention always takes the split form, which on a GPU with 148 SMs is the only one that
fills the machine at batch sizes a decoder sees.
"""
import torch

from .. import _abi
from ..kernels.linear import matmul

_FLOATS = _abi.FLOAT_DTYPES


def positions(batch, sequence, start, device):
    """int64 [batch, sequence]: start, start+1, ... in every row."""
    out = torch.empty((batch, sequence), device=device, dtype=torch.int64)
    with torch.cuda.device(out.device):
        _abi.call('q3_inf_positions', out.data_ptr(), batch, sequence, start, _abi.stream())
    return out


def append(k, v, cache_k, cache_v, start):
    """Write the new k, v [B,S,H,D] into the caches [B,H,C,D] at tokens start .. start+S-1."""
    if k.ndim != 4 or k.shape != v.shape or cache_k.shape != cache_v.shape or cache_k.ndim != 4:
        raise ValueError('Expected k, v [B,S,H,D] and caches [B,H,C,D]')
    b, s, h, d = k.shape
    if cache_k.shape[0] != b or cache_k.shape[1] != h or cache_k.shape[3] != d or start < 0 or start + s > cache_k.shape[2]:
        raise ValueError('New tokens do not fit the cache')
    tensors = (k, v, cache_k, cache_v)
    if not all(t.is_cuda and t.is_contiguous() and t.dtype == k.dtype and t.device == k.device for t in tensors):
        raise ValueError('Matching contiguous CUDA tensors required; no fallback')
    _abi.call('q3_kv_append', k.data_ptr(), v.data_ptr(), cache_k.data_ptr(), cache_v.data_ptr(), b, s, h, d,
              cache_k.shape[2], start, _abi.dt(k.dtype), _abi.stream())


def attention(q, cache_k, cache_v, start, *, split_decode=False):
    """q [B,S,Hq,D] against cache tokens 0 .. start+S-1 (causal within the new tokens): [B,S,Hq,D].
    `split_decode` is accepted for call-site compatibility: the chunked form is always used."""
    if q.ndim != 4 or cache_k.ndim != 4 or cache_k.shape != cache_v.shape:
        raise ValueError('Expected q [B,S,Hq,D] and caches [B,Hkv,C,D]')
    b, s, hq, d = q.shape
    hk, capacity = cache_k.shape[1], cache_k.shape[2]
    if cache_k.shape[0] != b or cache_k.shape[3] != d or hq % hk or start < 0 or start + s > capacity:
        raise ValueError('Query does not match the cache')
    tensors = (q, cache_k, cache_v)
    if not all(t.is_cuda and t.is_contiguous() and t.dtype == q.dtype and t.device == q.device for t in tensors):
        raise ValueError('Matching contiguous CUDA tensors required; no fallback')
    out = torch.empty_like(q)
    ws = _abi.workspace(_abi.lib().q3_cache_attention_workspace_bytes(b, s, hq, d, start, _abi.dt(q.dtype)), q.device)
    _abi.call('q3_cache_attention', q.data_ptr(), cache_k.data_ptr(), cache_v.data_ptr(), out.data_ptr(), ws.data_ptr(),
              ws.numel(), b, s, hq, hk, d, capacity, start, d ** -0.5, _abi.dt(q.dtype), _abi.stream())
    return out


def linear(x, weight, *, gemv=True, accurate=False, sliced=False, prefill_tiling=False, reference_accumulation=False):
    """x [..., K] @ weight[N, K]^T. Up to 8 rows go through the weight-streaming GEMV (fp64 accumulation with
    `accurate`), more through the tensor-core GEMM."""
    shape = x.shape
    k, n = shape[-1], weight.shape[0]
    m = x.numel() // k
    if weight.ndim != 2 or weight.shape[1] != k or x.dtype != weight.dtype or x.dtype not in _FLOATS:
        raise ValueError('Expected x [..., K] and weight [N, K] of one floating dtype')
    if not (x.is_cuda and weight.device == x.device):
        raise ValueError('Same-device CUDA tensors required; no fallback')
    fits = m <= 8 and x.is_contiguous() and weight.is_contiguous() and (k * x.element_size()) % 16 == 0
    if (gemv or accurate) and fits:
        y = torch.empty((*shape[:-1], n), device=x.device, dtype=x.dtype)
        _abi.call('q3_gemv', x.data_ptr(), weight.data_ptr(), y.data_ptr(), m, n, k, _abi.dt(x.dtype), int(bool(accurate)),
                  _abi.stream())
        return y
    return matmul(x.reshape(m, k), weight.t(), optimized=True).view(*shape[:-1], n)


def select(logits, ids, next_token, done, position, eos, pad):
    """One greedy decoding step, in place: ids[:, position] and next_token get the argmax of each logits row (lowest
    index on ties; `pad` for rows already done), and rows that produced an end-of-sequence id become done."""
    if logits.ndim != 2 or ids.ndim != 2 or ids.shape[0] != logits.shape[0] or not 0 <= position < ids.shape[1]:
        raise ValueError('Expected logits [B,V], ids [B,L] and a position inside ids')
    if ids.dtype != torch.int64 or next_token.dtype != torch.int64 or done.dtype != torch.bool:
        raise ValueError('int64 ids / next_token and a boolean done mask required')
    if next_token.numel() != logits.shape[0] or done.numel() != logits.shape[0]:
        raise ValueError('One next token and one done flag per row required')
    tensors = (logits, ids, next_token, done)
    if not all(t.is_cuda and t.is_contiguous() and t.device == logits.device for t in tensors):
        raise ValueError('Contiguous same-device CUDA tensors required; no fallback')
    stops = torch.tensor(list(eos), device=logits.device, dtype=torch.int64) if len(eos) else None
    ws = _abi.workspace(_abi.lib().q3_select_tokens_workspace_bytes(logits.shape[0], logits.shape[1]), logits.device)
    _abi.call('q3_select_tokens', logits.data_ptr(), logits.shape[0], logits.shape[1], ids.data_ptr(), ids.shape[1],
              position, next_token.data_ptr(), done.data_ptr(), _abi.ptr(stops), len(eos), pad, ws.data_ptr(), ws.numel(),
              _abi.dt(logits.dtype), _abi.stream())


def rms_norm(x, weight, eps, *, reference_accumulation=False):
    """RMSNorm over the last dimension for any number of rows (the training wrapper's minimum does not apply)."""
    rows = x.numel() // weight.numel()
    y = torch.empty_like(x)
    inv = torch.empty(rows, device=x.device, dtype=torch.float32)
    _abi.call('q3_rmsnorm_fwd', x.data_ptr(), weight.data_ptr(), y.data_ptr(), inv.data_ptr(), rows, weight.numel(),
              float(eps), _abi.dt(x.dtype), _abi.stream())
    return y


def norm_rope(x, weight, cos, sin, eps):
    """Per-head RMSNorm + RoPE of x [B,S,heads,D] with cos/sin [B,S,D], forward only."""
    b, s, heads, d = x.shape
    y = torch.empty_like(x)
    inv = torch.empty(b * s * heads, device=x.device, dtype=torch.float32)
    _abi.call('q3_norm_rope_fwd', x.data_ptr(), weight.data_ptr(), cos.data_ptr(), sin.data_ptr(), y.data_ptr(),
              inv.data_ptr(), b * s, heads, d, float(eps), _abi.dt(x.dtype), _abi.stream())
    return y
