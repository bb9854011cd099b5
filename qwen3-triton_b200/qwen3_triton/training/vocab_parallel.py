"""Vocabulary-parallel lm_head projection and exact full cross-entropy.

Ranks keep their data-parallel decoder inputs and a contiguous FP32 master shard of the vocabulary.
Hidden states and labels are all-gathered, each rank scores its vocabulary slice, two small all-reduces
(MAX, then SUM of exp-shifted partition sums and target logits) give the exact loss, dX is a FP32
reduce-scatter and dW stays local, already averaged over data ranks - so this parameter must be kept out
of FSDP. Same surface and semantics as the reference qwen3_triton/training/vocab_parallel.py:38-107;
works for any world size (including 1, where the collectives are skipped).
"""
import torch
import torch.distributed as dist

from ..kernels.attention import cast_tensor
from ..kernels.linear import matmul
from ..kernels.vocab_ce import (accumulate_weight_gradient, finish_statistics, local_statistics, logit_gradient,
                                packed_statistics)


def _world():
    return (dist.get_world_size(), dist.get_rank()) if dist.is_available() and dist.is_initialized() else (1, 0)


def _gather(owner, output, source):
    if owner.world == 1:
        output.copy_(source.view_as(output))
    elif owner.communication is None:
        dist.all_gather_into_tensor(output, source)
    else:
        owner.communication.all_gather(output, source)


def _reduce(owner, tensor, op):
    if owner.world == 1:
        return
    if owner.communication is None:
        dist.all_reduce(tensor, op=op)
    else:
        if op == dist.ReduceOp.MAX:
            operation = 'max'
        elif op == dist.ReduceOp.SUM:
            operation = 'sum'
        else:
            raise ValueError('Head only uses MAX/SUM')
        owner.communication.all_reduce(tensor, operation)


def _check_head_inputs(hidden, weight, labels):
    b, s, _ = hidden.shape
    ok = (hidden.dtype == torch.bfloat16 and weight.dtype == torch.float32 and labels.dtype == torch.int64
          and labels.shape == (b, s) and s >= 2 and hidden.is_contiguous() and labels.is_contiguous()
          and hidden.device == weight.device == labels.device)
    if not ok:
        raise ValueError('Matching contiguous BF16 hidden, int64 labels and local FP32 weight required')


def _reduce_scatter_rows(owner, partial, rows, dtype):
    """Each rank's own `rows` rows of the sum over ranks of `partial` [world*rows, H]."""
    if owner.world == 1:
        return partial
    out = torch.empty((rows, partial.shape[1]), device=partial.device, dtype=dtype)
    if owner.communication is None:
        dist.reduce_scatter_tensor(out, partial, op=dist.ReduceOp.SUM)
    else:
        owner.communication.reduce_scatter(out, partial, 'sum')
    return out


class _StreamedScores:
    """Scores of the local vocabulary slice that never exist in memory: the projection GEMM reduces every logit
    tile to softmax statistics in its epilogue, and backward walks the slice in chunks, recomputing one chunk of
    logits into dZ at a time (qwen3_triton/kernels/fused_loss.py)."""
    keeps_logits = False

    def statistics(self, all_hidden, w, all_labels, batch_rows, sequence, start, total, ignore):
        from ..kernels import fused_loss as F
        eff = F.shifted_labels(all_labels.view(-1, sequence), ignore, total)
        local_lse, target = F.local_lse_and_target(all_hidden, w, eff, start, ignore)
        return local_lse, target, (eff,)

    def finish(self, maximum, packed, kept, rows, sequence, world, ignore):
        from ..kernels import fused_loss as F
        lse = torch.empty_like(maximum)
        _, counts, means = F.finish(lse, packed[1], kept[0], rows, ignore, maximum, packed)
        return lse, counts, means

    def gradients(self, owner, all_hidden, w, kept, lse, counts, ups, rows, sequence, start, ignore):
        from ..kernels import fused_loss as F
        partial_dx, dw = F.head_backward(all_hidden, w, kept[0], lse, ups, counts, rows, start, ignore, owner.chunk,
                                         torch.float32)
        if owner.world > 1:
            accumulate_weight_gradient(dw, dw, owner.world, True)     # mean over data ranks, in place
        return partial_dx, dw


class _StoredScores:
    """The reference's arrangement (qwen3_triton/training/vocab_parallel.py:38-89 there): the [world*rows, V/world]
    logits slice is written once by the projection GEMM, read by the statistics and gradient kernels, and can be
    handed back in full for diagnostics."""
    keeps_logits = True

    def statistics(self, all_hidden, w, all_labels, batch_rows, sequence, start, total, ignore):
        logits = matmul(all_hidden, w.t(), optimized=True)
        local_lse, target = local_statistics(logits, all_labels, sequence, start, vocab_total=total, ignore=ignore)
        return local_lse, target, (all_labels, logits)

    def finish(self, maximum, packed, kept, rows, sequence, world, ignore):
        return finish_statistics(maximum, packed, kept[0], rows, sequence, world, ignore)

    def gradients(self, owner, all_hidden, w, kept, lse, counts, ups, rows, sequence, start, ignore):
        labels, logits = kept
        world = owner.world
        dz = logit_gradient(logits, labels, lse, counts, ups, rows, sequence, start, ignore,
                            vocab_total=world * w.shape[0])
        partial_dx = matmul(dz, w, optimized=True, output_dtype=torch.float32)
        if owner.fused_dw:
            from ..kernels.vocab_dw import weight_gradient_mean
            return partial_dx, weight_gradient_mean(dz, all_hidden, rows, world, owner.dw_config)
        dw = torch.empty(w.shape, device=w.device, dtype=torch.float32)
        for source in range(world):          # one product per data rank, averaged in rank order
            part = slice(source * rows, (source + 1) * rows)
            accumulate_weight_gradient(matmul(dz[part].t(), all_hidden[part], optimized=True), dw, world, source == 0)
        return partial_dx, dw

    def dense_logits(self, owner, kept, batch, rows, sequence):
        """[B, S, V] logits of this rank's tokens: every rank sends each peer that peer's rows of its slice."""
        logits = kept[1]
        world, v = owner.world, logits.shape[1]
        received = torch.empty_like(logits)
        if world == 1:
            received.copy_(logits)
        elif owner.communication is None:
            dist.all_to_all_single(received, logits)
        else:
            owner.communication.all_to_all(received, logits)
        return received.view(world, rows, v).transpose(0, 1).contiguous().view(batch, sequence, world * v)


class _VocabCE(torch.autograd.Function):
    """hidden [B,S,H] (this rank's tokens), weight [V/world, H] (this rank's vocabulary rows) -> (loss, logits or
    None). One protocol for both ways of handling the scores: all-gather hidden states and labels; score the local
    slice (per-row log-sum-exp and the target logit where the slice owns the label); all-reduce MAX, then SUM of
    the exp-shifted partition sums and targets; finish to this rank's token-mean loss. Backward: all-gather the
    upstream scalars, form dZ against the global log-sum-exp, reduce-scatter the fp32 partial dX, keep dW local
    (already averaged over data ranks). Same arguments and saved quantities as the reference's _VocabCE, with the
    score handling delegated to `scores`."""

    @staticmethod
    def forward(ctx, hidden, weight, labels, ignore, diagnostics, owner, scores=None):
        scores = scores or _StoredScores()
        _check_head_inputs(hidden, weight, labels)
        if diagnostics and not scores.keeps_logits:
            raise ValueError('Diagnostic logits need the stored-scores path')
        world, rank = owner.world, owner.rank
        b, s, k = hidden.shape
        rows, v = b * s, weight.shape[0]
        all_hidden = torch.empty((world * rows, k), device=hidden.device, dtype=hidden.dtype)
        all_labels = torch.empty(world * rows, device=hidden.device, dtype=labels.dtype)
        _gather(owner, all_hidden, hidden.view(rows, k))
        _gather(owner, all_labels, labels.view(-1))
        w = cast_tensor(weight, torch.bfloat16)
        local_lse, target, kept = scores.statistics(all_hidden, w, all_labels, rows, s, rank * v, world * v, ignore)
        maximum = local_lse.clone()
        _reduce(owner, maximum, dist.ReduceOp.MAX)
        packed = packed_statistics(local_lse, maximum, target)
        _reduce(owner, packed, dist.ReduceOp.SUM)
        lse, counts, means = scores.finish(maximum, packed, kept, rows, s, world, ignore)
        dense = None
        if diagnostics:
            dense = scores.dense_logits(owner, kept, b, rows, s)
            ctx.mark_non_differentiable(dense)
        ctx.save_for_backward(all_hidden, w, lse, counts, *kept)
        ctx.rows, ctx.sequence, ctx.start, ctx.ignore, ctx.owner, ctx.scores = rows, s, rank * v, ignore, owner, scores
        owner.forward_calls += 1
        return means[rank].clone(), dense

    @staticmethod
    def backward(ctx, up, _dense_grad):
        all_hidden, w, lse, counts, *kept = ctx.saved_tensors
        owner = ctx.owner
        ups = torch.empty(owner.world, device=up.device, dtype=up.dtype)
        _gather(owner, ups, up.contiguous().view(1))
        partial_dx, dw = ctx.scores.gradients(owner, all_hidden, w, tuple(kept), lse, counts, ups, ctx.rows,
                                              ctx.sequence, ctx.start, ctx.ignore)
        dx = cast_tensor(_reduce_scatter_rows(owner, partial_dx, ctx.rows, torch.float32), torch.bfloat16)
        owner.backward_calls += 1
        return dx.view(-1, ctx.sequence, all_hidden.shape[1]), dw, None, None, None, None, None


class VocabParallelCE(torch.nn.Module):
    def __init__(self, full_weight_cpu, *, fused_dw=False, communication=None, fused=True, chunk=16384):
        """`fused` (an addition to the reference signature): compute the loss without materialising the logits
        shard; `diagnostics=True` in forward always takes the materialising path because it returns the logits."""
        super().__init__()
        self.fused = bool(fused)
        self.chunk = int(chunk)
        self.world, self.rank = _world()
        if full_weight_cpu.device.type != 'cpu' or full_weight_cpu.ndim != 2 or full_weight_cpu.shape[0] % self.world:
            raise ValueError('Equal CPU vocabulary shards required')
        self.out_features, self.in_features = full_weight_cpu.shape
        v = self.out_features // self.world
        self.weight = torch.nn.Parameter(full_weight_cpu[self.rank * v:(self.rank + 1) * v].float().cuda().clone())
        self.forward_calls = 0
        self.backward_calls = 0
        self.fused_dw = bool(fused_dw)
        self.dw_config = None
        self.communication = communication

    def forward(self, hidden, labels, *, ignore_index=-100, diagnostics=False):
        if hidden.ndim != 3 or hidden.shape[-1] != self.in_features:
            raise ValueError('Expected [B,S,H] hidden states')
        streamed = self.fused and not diagnostics and self.in_features % 8 == 0 and self.weight.shape[0] % 8 == 0
        scores = _StreamedScores() if streamed else _StoredScores()
        return _VocabCE.apply(hidden, self.weight, labels, ignore_index, diagnostics, self, scores)


class _VocabEmbedding(torch.autograd.Function):
    """Lookup in a row-sharded table. Forward: all-gather the token ids (a few KB), every rank looks up the rows it
    owns for the tokens of all ranks (zeros elsewhere), a reduce-scatter SUM hands each rank its own tokens' rows
    (each row has exactly one non-zero contribution, so the sum is exact). Backward: all-gather the hidden
    gradients, accumulate the owned rows locally in FP32 in a fixed order, divide by the number of data ranks
    (the mean FSDP's reduce-scatter AVG would give). Traffic per step: [W*T, H] BF16 each way instead of the
    whole table (BF16 gather + FP32 gradient reduce-scatter)."""

    @staticmethod
    def forward(ctx, ids, weight, owner):
        from ..kernels.embedding import shard_lookup
        world, rank = owner.world, owner.rank
        if ids.dtype != torch.int64 or not ids.is_contiguous() or weight.dtype != torch.float32 or ids.device != weight.device:
            raise ValueError('Contiguous int64 IDs and a local FP32 table shard on one device required')
        n = ids.numel()
        rows, h = weight.shape
        all_ids = torch.empty(world * n, device=ids.device, dtype=ids.dtype)
        _gather(owner, all_ids, ids.view(-1))
        partial = shard_lookup(all_ids, weight, rank * rows, world * rows, torch.bfloat16)
        out = _reduce_scatter_rows(owner, partial, n, torch.bfloat16)
        ctx.save_for_backward(all_ids)
        ctx.owner, ctx.rows = owner, rows
        owner.forward_calls += 1
        return out.view(*ids.shape, h)

    @staticmethod
    def backward(ctx, dy):
        from ..kernels.embedding import shard_weight_gradient
        all_ids, = ctx.saved_tensors
        owner = ctx.owner
        world, rank = owner.world, owner.rank
        h = dy.shape[-1]
        dy = dy.contiguous().view(-1, h)
        all_dy = torch.empty((world * dy.shape[0], h), device=dy.device, dtype=dy.dtype)
        _gather(owner, all_dy, dy)
        dw = shard_weight_gradient(all_ids, all_dy, rank * ctx.rows, ctx.rows, 1.0 / world)
        owner.backward_calls += 1
        return None, dw, None


class VocabParallelEmbedding(torch.nn.Module):
    """Token embedding whose table is split by rows over the data ranks and never gathered; the counterpart of
    VocabParallelCE for the input side. `weight` is this rank's contiguous FP32 master shard and must be kept out
    of FSDP; its gradient arrives already averaged over data ranks. No counterpart in the reference, which lets
    FSDP gather the whole table every step (qwen3_triton/_model.py:110-118 under scripts/vocab_model_v12.py:43-44)."""

    def __init__(self, full_weight_cpu, *, communication=None):
        super().__init__()
        self.world, self.rank = _world()
        if full_weight_cpu.device.type != 'cpu' or full_weight_cpu.ndim != 2 or full_weight_cpu.shape[0] % self.world:
            raise ValueError('Equal CPU vocabulary shards required')
        if full_weight_cpu.shape[1] % 8:
            raise ValueError('Hidden size must be a multiple of 8')
        self.num_embeddings, self.embedding_dim = full_weight_cpu.shape
        v = self.num_embeddings // self.world
        self.weight = torch.nn.Parameter(full_weight_cpu[self.rank * v:(self.rank + 1) * v].float().cuda().clone())
        self.communication = communication
        self.forward_calls = 0
        self.backward_calls = 0

    def forward(self, ids):
        if ids.dtype != torch.int64:
            raise TypeError('int64 token ids required')
        return _VocabEmbedding.apply(ids.contiguous(), self.weight, self)
