"""Decoder layer as ONE autograd node with a hand-written backward, driving the C ABI directly.

The operator-level graph (one autograd.Function per RMSNorm / linear / RoPE / attention / SwiGLU, as in the
reference qwen3_triton/components.py:9-54 and _model.py:84-108) costs about forty Python autograd nodes, four transpose copies and
two residual-add kernels per layer and direction. At 2048 tokens per GPU a B200 finishes those kernels faster
than Python can launch them. This module keeps the same math and the same parameters but

  * keeps q/k/v and the attention output token-major ([B, S, heads, 128]): the attention kernels read and
    write that layout through TMA, so no transpose copy exists;
  * carries the residual stream between layers as a pair (resid, delta) and folds `resid + delta` into the
    next RMSNorm (q3_add_rmsnorm_fwd/bwd), so no stand-alone residual-add kernel runs;
  * does per-layer activation checkpointing inside its own backward, without the generic checkpoint wrapper
    (reference: training/fsdp/activation_checkpoint.py:15-19). `recompute` = 0 keeps every intermediate,
    2 ("full") keeps only the layer input and re-runs the whole forward, 1 ("selective") keeps the outputs of
    the GEMMs and of attention (x, q, k, v, o, lse, x1, gate, up: about 175 MB per layer at 2048 tokens) and
    re-runs only the bandwidth-bound pieces (two RMSNorms, QK-norm+RoPE, SwiGLU) - all of the memory saving
    that matters on a 180 GB GPU for 4 % instead of 33 % extra work.

Requires bf16/fp16 tensors and head_dim 128 (the tensor-core attention path); other shapes use the
operator-level modules.
"""
import os

import torch

from . import _abi
from ._model import Backbone, DecoderBlock


def _empty(shape, like, dtype=None):
    return torch.empty(shape, device=like.device, dtype=dtype or like.dtype)


class WeightGradientStream:
    """Weight-gradient GEMMs of the fused layer's backward on a second stream.

    In a linear layer's backward the input gradient (dY W) and the weight gradient (dY^T X) are independent, and each
    is a persistent GEMM whose last wave leaves SMs idle (256 tiles on 148 SMs: 1.73 waves). Issued on two streams,
    the CTAs of the second kernel become resident as those of the first run out of tiles, so the tail of one is filled
    by the head of the other; this needs the GEMM tiles to be drawn from a counter (q3_gemm_tile_schedule(1)), or the
    late CTAs would still own a full share. Nothing reads a weight gradient before the layer's backward returns, which
    is where the streams are joined. Off by default: `WeightGradientStream.enabled = True` (or Q3_WGRAD_SIDE_STREAM=1)."""
    enabled = os.environ.get('Q3_WGRAD_SIDE_STREAM', '0') == '1'
    _streams = {}

    @classmethod
    def run(cls, fn, inputs):
        """outputs = fn() on the side stream, ordered after the current stream's work so far."""
        if not cls.enabled:
            return fn()
        main = torch.cuda.current_stream()
        side = cls._streams.get(main.device)
        if side is None:
            side = cls._streams[main.device] = torch.cuda.Stream(device=main.device)
        side.wait_stream(main)
        with torch.cuda.stream(side):
            outputs = fn()
        for t in inputs:
            t.record_stream(side)              # freed on the main stream while the side stream may still read it
        for t in (outputs if isinstance(outputs, (list, tuple)) else [outputs]):
            t.record_stream(main)              # allocated under the side stream, consumed on the main stream
        return outputs

    @classmethod
    def join(cls):
        if cls.enabled:
            main = torch.cuda.current_stream()
            side = cls._streams.get(main.device)
            if side is not None:
                main.wait_stream(side)


class GradientHomes:
    """Where the fused layer's backward may put its weight gradients. `provider` (runtime/peer_reduce.py:
    PeerGradientReducer after register_units) hands out views inside the buffer the gradient reduction reads, so that
    the gradients need no packing pass; None: ordinary tensors."""
    provider = None

    @classmethod
    def handles(cls, layer):
        """Per weight of `layer.weights()`: the provider's handle of that parameter's home, or None."""
        provider = cls.provider
        if provider is None:
            return None
        a, m = layer.self_attn, layer.mlp
        owners = (layer.input_layernorm, a.q_proj, a.k_proj, a.v_proj, a.o_proj, a.q_norm, a.k_norm,
                  layer.post_attention_layernorm, m.gate_proj, m.up_proj, m.down_proj)
        handles = tuple(provider.home(owner, 'weight') for owner in owners)
        return handles if any(h is not None for h in handles) else None

    @classmethod
    def view(cls, handles, position, shape, like):
        """The home of weight number `position` if it has one of this shape and dtype, else a fresh tensor."""
        provider = cls.provider
        if provider is not None and handles is not None and handles[position] is not None:
            t = provider.gradient_view(handles[position], like.dtype)
            if t is not None and tuple(t.shape) == tuple(shape) and t.device == like.device:
                return t
        return _empty(shape, like)


def _gemm(a_ptr, a_sm, a_sk, b_ptr, b_sk, b_sn, m, n, k, like, out_dtype=None, out=None):
    if out is None:
        out = _empty((m, n), like, out_dtype)
    _abi.call('q3_gemm', a_ptr, a_sm, a_sk, b_ptr, b_sk, b_sn, out.data_ptr(), m, n, k, _abi.dt(like.dtype),
              _abi.dt(out.dtype), _abi.status_word(like.device).data_ptr(), _abi.stream())
    return out


def mm_nt(x, w):
    """x [M,K] @ w[N,K]^T -> [M,N]"""
    return _gemm(x.data_ptr(), x.shape[1], 1, w.data_ptr(), 1, w.shape[1], x.shape[0], w.shape[0], x.shape[1], x)


def mm_nn(dy, w):
    """dy [M,N] @ w[N,K] -> [M,K]"""
    return _gemm(dy.data_ptr(), dy.shape[1], 1, w.data_ptr(), w.shape[1], 1, dy.shape[0], w.shape[1], dy.shape[1], dy)


def mm_tn(dy, x, out=None):
    """dy[M,N]^T @ x[M,K] -> [N,K]"""
    return _gemm(dy.data_ptr(), 1, dy.shape[1], x.data_ptr(), x.shape[1], 1, dy.shape[1], x.shape[1], dy.shape[0], dy,
                 out=out)


def _grouped_ok(x, weights):
    return all(w.shape[0] % 64 == 0 for w in weights) and x.shape[1] % 8 == 0


def linear_group_fwd(x, weights):
    """[x @ w.T for w in weights] in one launch."""
    if not _grouped_ok(x, weights):
        return [mm_nt(x, w) for w in weights]
    ys = [_empty((x.shape[0], w.shape[0]), x) for w in weights]
    wp, yp, n = _abi.pointer_array(weights), _abi.pointer_array(ys), _abi.size_array([w.shape[0] for w in weights])
    _abi.call('q3_linear_fwd_grouped', x.data_ptr(), wp, yp, n, len(weights), x.shape[0], x.shape[1], _abi.dt(x.dtype),
              _abi.status_word(x.device).data_ptr(), _abi.stream())
    return ys


def linear_group_dgrad(dys, weights):
    """sum(dy @ w for dy, w in zip(dys, weights)) in one launch (one accumulator, no add kernels)."""
    if not _grouped_ok(dys[0], weights):
        out = mm_nn(dys[0], weights[0])
        for dy, w in zip(dys[1:], weights[1:]):
            mm_nn_acc(out, dy, w)
        return out
    dx = _empty((dys[0].shape[0], weights[0].shape[1]), dys[0])
    dp, wp, n = _abi.pointer_array(dys), _abi.pointer_array(weights), _abi.size_array([w.shape[0] for w in weights])
    _abi.call('q3_linear_dgrad_grouped', dp, wp, dx.data_ptr(), n, len(weights), dx.shape[0], dx.shape[1],
              _abi.dt(dx.dtype), _abi.status_word(dx.device).data_ptr(), _abi.stream())
    return dx


def linear_group_wgrad(dys, x, outs=None):
    """[dy.T @ x for dy in dys] in one launch; `outs`: tensors to write into."""
    if not all(dy.shape[1] % 8 == 0 for dy in dys) or x.shape[1] % 8:
        return [mm_tn(dy, x, out=None if outs is None else outs[i]) for i, dy in enumerate(dys)]
    dws = outs if outs is not None else [_empty((dy.shape[1], x.shape[1]), x) for dy in dys]
    dp, gp, n = _abi.pointer_array(dys), _abi.pointer_array(dws), _abi.size_array([dy.shape[1] for dy in dys])
    _abi.call('q3_linear_wgrad_grouped', dp, x.data_ptr(), gp, n, len(dys), x.shape[0], x.shape[1], _abi.dt(x.dtype),
              _abi.status_word(x.device).data_ptr(), _abi.stream())
    return dws


def mm_nn_acc(out, dy, w):
    """out [M,K] += dy [M,N] @ w[N,K] (read-add-round in the GEMM epilogue; no separate add pass)"""
    _abi.call('q3_gemm_acc', dy.data_ptr(), dy.shape[1], 1, w.data_ptr(), w.shape[1], 1, out.data_ptr(), dy.shape[0],
              w.shape[1], dy.shape[1], _abi.dt(dy.dtype), _abi.dt(out.dtype), _abi.status_word(dy.device).data_ptr(),
              _abi.stream())
    return out


def _norm_fwd(x, delta, w, eps):
    """(h, x_sum, inv): h = RMSNorm(x + delta) * w; x_sum = x + delta (x itself when delta is None)."""
    rows, hdim = x.shape
    h = torch.empty_like(x)
    inv = _empty((rows,), x, torch.float32)
    if delta is None:
        _abi.call('q3_rmsnorm_fwd', x.data_ptr(), w.data_ptr(), h.data_ptr(), inv.data_ptr(), rows, hdim, eps,
                  _abi.dt(x.dtype), _abi.stream())
        return h, x, inv
    xs = torch.empty_like(x)
    _abi.call('q3_add_rmsnorm_fwd', delta.data_ptr(), x.data_ptr(), w.data_ptr(), h.data_ptr(), xs.data_ptr(),
              inv.data_ptr(), rows, hdim, eps, _abi.dt(x.dtype), _abi.stream())
    return h, xs, inv


def _norm_bwd(xs, w, dh, dres, inv):
    """(dx, dw): RMSNorm backward on xs plus the residual-path gradient dres (may be None)."""
    rows, hdim = xs.shape
    dx = torch.empty_like(xs)
    dw = torch.empty_like(w)
    ws = _abi.workspace(_abi.lib().q3_rmsnorm_bwd_workspace_bytes(rows, hdim), xs.device)
    _abi.call('q3_add_rmsnorm_bwd', xs.data_ptr(), w.data_ptr(), dh.data_ptr(), _abi.ptr(dres), inv.data_ptr(),
              dx.data_ptr(), dw.data_ptr(), ws.data_ptr(), ws.numel(), rows, hdim, _abi.dt(xs.dtype), _abi.stream())
    return dx, dw


def _norm_rope_fwd(x, w, cos, sin, tokens, heads, d, eps):
    y = torch.empty_like(x)
    inv = _empty((tokens * heads,), x, torch.float32)
    _abi.call('q3_norm_rope_fwd', x.data_ptr(), w.data_ptr(), cos.data_ptr(), sin.data_ptr(), y.data_ptr(),
              inv.data_ptr(), tokens, heads, d, eps, _abi.dt(x.dtype), _abi.stream())
    return y, inv


def _norm_rope_bwd(x, w, cos, sin, dy, inv, tokens, heads, d):
    dx = torch.empty_like(x)
    dw = torch.empty_like(w)
    ws = _abi.workspace(_abi.lib().q3_norm_rope_bwd_workspace_bytes(tokens, heads, d), x.device)
    _abi.call('q3_norm_rope_bwd', x.data_ptr(), w.data_ptr(), cos.data_ptr(), sin.data_ptr(), dy.data_ptr(),
              inv.data_ptr(), dx.data_ptr(), dw.data_ptr(), ws.data_ptr(), ws.numel(), tokens, heads, d,
              _abi.dt(x.dtype), _abi.stream())
    return dx, dw


def _qk_norm_rope_fwd(q, k, wq, wk, cos, sin, tokens, hq, hk, d, eps):
    """q and k through per-head RMSNorm + RoPE in one launch: (qn, invq, kn, invk)."""
    yq, yk = torch.empty_like(q), torch.empty_like(k)
    invq, invk = _empty((tokens * hq,), q, torch.float32), _empty((tokens * hk,), k, torch.float32)
    _abi.call('q3_qk_norm_rope_fwd', q.data_ptr(), k.data_ptr(), wq.data_ptr(), wk.data_ptr(), cos.data_ptr(),
              sin.data_ptr(), yq.data_ptr(), yk.data_ptr(), invq.data_ptr(), invk.data_ptr(), tokens, hq, hk, d, eps,
              _abi.dt(q.dtype), _abi.stream())
    return yq, invq, yk, invk


def _qk_norm_rope_bwd(q, k, wq, wk, cos, sin, dyq, dyk, invq, invk, tokens, hq, hk, d):
    dq, dk, dwq, dwk = torch.empty_like(q), torch.empty_like(k), torch.empty_like(wq), torch.empty_like(wk)
    ws = _abi.workspace(_abi.lib().q3_qk_norm_rope_bwd_workspace_bytes(tokens, hq, hk, d), q.device)
    _abi.call('q3_qk_norm_rope_bwd', q.data_ptr(), k.data_ptr(), wq.data_ptr(), wk.data_ptr(), cos.data_ptr(),
              sin.data_ptr(), dyq.data_ptr(), dyk.data_ptr(), invq.data_ptr(), invk.data_ptr(), dq.data_ptr(),
              dk.data_ptr(), dwq.data_ptr(), dwk.data_ptr(), ws.data_ptr(), ws.numel(), tokens, hq, hk, d,
              _abi.dt(q.dtype), _abi.stream())
    return dq, dwq, dk, dwk


def layer_forward(resid, delta, cos, sin, w, meta):
    """All intermediates of one decoder layer. resid/delta [T, H]; returns a dict."""
    b, s, hq, hk, d, eps = meta
    t = resid.shape[0]
    w_in, wq, wk, wv, wo, wqn, wkn, w_post, wg, wu, wd = w
    r = {}
    r['h'], r['x'], r['inv1'] = _norm_fwd(resid, delta, w_in, eps)
    r['q'], r['k'], r['v'] = linear_group_fwd(r['h'], [wq, wk, wv])
    r['qn'], r['invq'], r['kn'], r['invk'] = _qk_norm_rope_fwd(r['q'], r['k'], wqn, wkn, cos, sin, t, hq, hk, d, eps)
    r['o'] = torch.empty_like(r['q'])
    r['lse'] = _empty((b, hq, s), resid, torch.float32)
    _abi.call('q3_attn_fwd_bshd', r['qn'].data_ptr(), r['kn'].data_ptr(), r['v'].data_ptr(), r['o'].data_ptr(),
              r['lse'].data_ptr(), b, s, hq, hk, d, d ** -0.5, _abi.dt(resid.dtype),
              _abi.status_word(resid.device).data_ptr(), _abi.stream())
    a = mm_nt(r['o'], wo)
    r['h2'], r['x1'], r['inv2'] = _norm_fwd(r['x'], a, w_post, eps)
    n = wg.shape[0]
    r['g'], r['u'], r['y'] = _empty((t, n), resid), _empty((t, n), resid), _empty((t, n), resid)
    _abi.call('q3_gate_up_swiglu_fwd', r['h2'].data_ptr(), wg.data_ptr(), wu.data_ptr(), r['g'].data_ptr(),
              r['u'].data_ptr(), r['y'].data_ptr(), t, n, wg.shape[1], _abi.dt(resid.dtype),
              _abi.status_word(resid.device).data_ptr(), _abi.stream())
    r['m'] = mm_nt(r['y'], wd)
    return r


_KEEP = ('h', 'x', 'inv1', 'q', 'k', 'v', 'qn', 'invq', 'kn', 'invk', 'o', 'lse', 'h2', 'x1', 'inv2', 'g', 'u', 'y')
_KEEP_SELECTIVE = ('x', 'q', 'k', 'v', 'o', 'lse', 'x1', 'g', 'u')


def recompute_cheap(r, cos, sin, w, meta):
    """Rebuild the bandwidth-bound intermediates (h, qn, kn, h2, y and the saved inverse RMS values) from the
    tensors kept by selective checkpointing."""
    b, s, hq, hk, d, eps = meta
    t = r['x'].shape[0]
    w_in, wq, wk, wv, wo, wqn, wkn, w_post, wg, wu, wd = w
    r['h'], _, r['inv1'] = _norm_fwd(r['x'], None, w_in, eps)
    r['qn'], r['invq'], r['kn'], r['invk'] = _qk_norm_rope_fwd(r['q'], r['k'], wqn, wkn, cos, sin, t, hq, hk, d, eps)
    r['h2'], _, r['inv2'] = _norm_fwd(r['x1'], None, w_post, eps)
    r['y'] = torch.empty_like(r['g'])
    _abi.call('q3_swiglu_fwd', r['g'].data_ptr(), r['u'].data_ptr(), r['y'].data_ptr(), r['g'].numel(),
              _abi.dt(r['g'].dtype), _abi.stream())
    return r


class FusedLayerFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, resid, delta, cos, sin, meta, recompute, homes, *weights):
        b, s, hq, hk, d, eps = meta
        shape = resid.shape
        r2 = resid.reshape(-1, shape[-1])
        d2 = delta.reshape(-1, shape[-1]) if delta is not None else None
        r = layer_forward(r2, d2, cos, sin, weights, meta)
        recompute = int(recompute)
        ctx.meta, ctx.recompute, ctx.shape, ctx.has_delta = meta, recompute, shape, delta is not None
        ctx.homes = homes
        if recompute == 2:
            ctx.save_for_backward(r2, d2 if d2 is not None else r2, cos, sin, *weights)
        elif recompute == 1:
            ctx.save_for_backward(cos, sin, *weights, *[r[k] for k in _KEEP_SELECTIVE])
        else:
            ctx.save_for_backward(cos, sin, *weights, *[r[k] for k in _KEEP])
        return r['x1'].view(shape), r['m'].view(shape)

    @staticmethod
    def backward(ctx, g_x1, g_m):
        b, s, hq, hk, d, eps = ctx.meta
        if ctx.recompute == 2:
            r2, d2, cos, sin, *weights = ctx.saved_tensors
            r = layer_forward(r2, d2 if ctx.has_delta else None, cos, sin, weights, ctx.meta)
        elif ctx.recompute == 1:
            saved = ctx.saved_tensors
            cos, sin = saved[0], saved[1]
            weights = saved[2:13]
            r = recompute_cheap(dict(zip(_KEEP_SELECTIVE, saved[13:])), cos, sin, weights, ctx.meta)
        else:
            saved = ctx.saved_tensors
            cos, sin = saved[0], saved[1]
            weights = saved[2:13]
            r = dict(zip(_KEEP, saved[13:]))
        w_in, wq, wk, wv, wo, wqn, wkn, w_post, wg, wu, wd = weights
        hdim = ctx.shape[-1]
        t = r['x'].shape[0]
        dm = g_m.reshape(t, hdim).contiguous()
        dres = g_x1.reshape(t, hdim).contiguous() if g_x1 is not None else None
        # MLP
        homes = ctx.homes

        def home(position, weight):
            # the parameter's place in the buffer the gradient reduction reads, or a fresh tensor
            return GradientHomes.view(homes, position, weight.shape, dm)

        dwd = WeightGradientStream.run(lambda: mm_tn(dm, r['y'], out=home(10, wd)), (dm, r['y']))
        dg, du = torch.empty_like(r['g']), torch.empty_like(r['u'])
        if wd.shape[0] % 8 == 0 and wd.shape[1] % 8 == 0:
            # dY = dM @ W_down never leaves tensor memory: the GEMM epilogue turns it into dG, dU
            _abi.call('q3_down_dgrad_swiglu_bwd', dm.data_ptr(), wd.data_ptr(), r['g'].data_ptr(), r['u'].data_ptr(),
                      dg.data_ptr(), du.data_ptr(), t, wd.shape[1], wd.shape[0], _abi.dt(dg.dtype),
                      _abi.status_word(dm.device).data_ptr(), _abi.stream())
        else:
            dy = mm_nn(dm, wd)
            _abi.call('q3_swiglu_bwd', r['g'].data_ptr(), r['u'].data_ptr(), dy.data_ptr(), dg.data_ptr(), du.data_ptr(),
                      dg.numel(), _abi.dt(dg.dtype), _abi.stream())
            del dy
        dh2 = linear_group_dgrad([dg, du], [wg, wu])
        dwg, dwu = WeightGradientStream.run(
            lambda: linear_group_wgrad([dg, du], r['h2'], outs=[home(8, wg), home(9, wu)]), (dg, du, r['h2']))
        del dg, du
        dx1, dw_post = _norm_bwd(r['x1'], w_post, dh2, dres, r['inv2'])
        # attention block
        do = mm_nn(dx1, wo)
        dwo = WeightGradientStream.run(lambda: mm_tn(dx1, r['o'], out=home(4, wo)), (dx1, r['o']))
        dqn, dkn, dv = torch.empty_like(r['qn']), torch.empty_like(r['kn']), torch.empty_like(r['v'])
        ws = _abi.workspace(_abi.lib().q3_attn_bwd_workspace_bytes(b, hq, hk, s, d), dx1.device)
        _abi.call('q3_attn_bwd_bshd', r['qn'].data_ptr(), r['kn'].data_ptr(), r['v'].data_ptr(), r['o'].data_ptr(),
                  do.data_ptr(), r['lse'].data_ptr(), dqn.data_ptr(), dkn.data_ptr(), dv.data_ptr(), ws.data_ptr(),
                  ws.numel(), b, s, hq, hk, d, d ** -0.5, _abi.dt(dx1.dtype), _abi.status_word(dx1.device).data_ptr(),
                  _abi.stream())
        dq, dwqn, dk, dwkn = _qk_norm_rope_bwd(r['q'], r['k'], wqn, wkn, cos, sin, dqn, dkn, r['invq'], r['invk'],
                                               t, hq, hk, d)
        dh = linear_group_dgrad([dq, dk, dv], [wq, wk, wv])
        dwq, dwk, dwv = WeightGradientStream.run(
            lambda: linear_group_wgrad([dq, dk, dv], r['h'], outs=[home(1, wq), home(2, wk), home(3, wv)]),
            (dq, dk, dv, r['h']))
        dx, dw_in = _norm_bwd(r['x'], w_in, dh, dx1, r['inv1'])
        dx = dx.view(ctx.shape)
        WeightGradientStream.join()
        return (dx, dx if ctx.has_delta else None, None, None, None, None, None,
                dw_in, dwq, dwk, dwv, dwo, dwqn, dwkn, dw_post, dwg, dwu, dwd)


def fused_layer_supported(x, head_dim):
    return x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and head_dim == 128


class FusedDecoderLayer(DecoderBlock):
    """Same parameters (and names) as the operator-level DecoderBlock; forward maps (resid, delta) to
    (resid', delta') through FusedLayerFn."""

    def __init__(self, c, recipe):
        super().__init__(c, recipe)
        self.recompute = 0      # 0 none, 1 selective, 2 full (see module docstring)

    def weights(self):
        a, m = self.self_attn, self.mlp
        return (self.input_layernorm.weight, a.q_proj.weight, a.k_proj.weight, a.v_proj.weight, a.o_proj.weight,
                a.q_norm.weight, a.k_norm.weight, self.post_attention_layernorm.weight, m.gate_proj.weight,
                m.up_proj.weight, m.down_proj.weight)

    def forward(self, resid, delta, rope):
        cos, sin = rope
        b, s, _ = resid.shape
        meta = (b, s, self.heads, self.kv_heads, self.head_dim, float(self.input_layernorm.eps))
        return FusedLayerFn.apply(resid, delta, cos, sin, meta, self.recompute, GradientHomes.handles(self),
                                  *self.weights())


def _final_norm(resid, delta, scale):
    """RMSNorm of the (resid, delta) pair the last layer hands over."""
    from .kernels.norm import add_rms_norm, rms_norm
    if delta is None:
        return rms_norm(resid, scale.weight, scale.eps)
    return add_rms_norm(delta, resid, scale.weight, scale.eps)[0]


class FusedBackbone(Backbone):
    block_class = FusedDecoderLayer

    def set_recompute(self, level):
        """0 / False: keep everything; 1 / 'selective'; 2 / True / 'full'."""
        level = {'none': 0, 'selective': 1, 'full': 2, False: 0, True: 2}.get(level, level)
        for layer in self.layers:
            layer.recompute = int(level)

    def forward(self, ids, position_ids=None):
        x = self.lookup(ids)
        if not fused_layer_supported(x, self.layers[0].head_dim):
            raise ValueError('Fused decoder layers need bf16/fp16 CUDA tensors and head_dim 128')
        rope = self.rope_for(ids, position_ids, x.dtype)
        resid, delta = x, None
        for layer in self.layers:
            resid, delta = layer(resid, delta, rope)
        return self.norm(_final_norm, resid, delta)
