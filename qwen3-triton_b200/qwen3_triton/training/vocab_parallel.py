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


class _FusedVocabCE(torch.autograd.Function):
    """Same contract as _VocabCE, but neither the logits shard nor its gradient is ever materialised: the
    projection GEMM reduces to softmax statistics in its epilogue, and backward walks the local vocabulary in
    chunks (qwen3_triton/kernels/fused_loss.py)."""

    @staticmethod
    def forward(ctx, hidden, weight, labels, ignore, owner):
        from ..kernels import fused_loss as F
        world, rank = owner.world, owner.rank
        b, s, k = hidden.shape
        r = b * s
        v = weight.shape[0]
        if (hidden.dtype != torch.bfloat16 or weight.dtype != torch.float32 or labels.dtype != torch.int64
                or labels.shape != (b, s) or s < 2 or not hidden.is_contiguous() or not labels.is_contiguous()
                or hidden.device != weight.device or hidden.device != labels.device):
            raise ValueError('Matching contiguous BF16 hidden, int64 labels and local FP32 weight required')
        all_hidden = torch.empty((world * r, k), device=hidden.device, dtype=hidden.dtype)
        all_labels = torch.empty(world * r, device=hidden.device, dtype=labels.dtype)
        _gather(owner, all_hidden, hidden.view(r, k))
        _gather(owner, all_labels, labels.view(-1))
        w = cast_tensor(weight, torch.bfloat16)
        eff = F.shifted_labels(all_labels.view(world * b, s), ignore, world * v)
        local_lse, target = F.local_lse_and_target(all_hidden, w, eff, rank * v, ignore)
        maximum = local_lse.clone()
        _reduce(owner, maximum, dist.ReduceOp.MAX)
        packed = packed_statistics(local_lse, maximum, target)
        _reduce(owner, packed, dist.ReduceOp.SUM)
        lse = torch.empty_like(local_lse)
        _, counts, means = F.finish(lse, packed[1], eff, r, ignore, maximum, packed)
        loss = means[rank].clone()
        ctx.save_for_backward(all_hidden, w, eff, lse, counts)
        ctx.rows, ctx.sequence, ctx.start, ctx.ignore, ctx.owner = r, s, rank * v, ignore, owner
        owner.forward_calls += 1
        return loss

    @staticmethod
    def backward(ctx, up):
        from ..kernels import fused_loss as F
        h, w, eff, lse, counts = ctx.saved_tensors
        owner = ctx.owner
        world, r, k = owner.world, ctx.rows, h.shape[1]
        ups = torch.empty(world, device=h.device, dtype=up.dtype)
        _gather(owner, ups, up.contiguous().view(1))
        partial_dx, dw = F.head_backward(h, w, eff, lse, ups, counts, r, ctx.start, ctx.ignore, owner.chunk,
                                         torch.float32)
        if world == 1:
            local_dx = partial_dx
        else:
            local_dx = torch.empty((r, k), device=h.device, dtype=torch.float32)
            if owner.communication is None:
                dist.reduce_scatter_tensor(local_dx, partial_dx, op=dist.ReduceOp.SUM)
            else:
                owner.communication.reduce_scatter(local_dx, partial_dx, 'sum')
            accumulate_weight_gradient(dw, dw, world, True)     # mean over data ranks, in place
        dx = cast_tensor(local_dx, torch.bfloat16)
        owner.backward_calls += 1
        return dx.view(-1, ctx.sequence, k), dw, None, None, None


class _VocabCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, labels, ignore, diagnostics, owner):
        world, rank = owner.world, owner.rank
        b, s, k = hidden.shape
        r = b * s
        v = weight.shape[0]
        if (hidden.dtype != torch.bfloat16 or weight.dtype != torch.float32 or labels.dtype != torch.int64
                or labels.shape != (b, s) or s < 2 or not hidden.is_contiguous() or not labels.is_contiguous()
                or hidden.device != weight.device or hidden.device != labels.device):
            raise ValueError('Matching contiguous BF16 hidden, int64 labels and local FP32 weight required')
        all_hidden = torch.empty((world * r, k), device=hidden.device, dtype=hidden.dtype)
        all_labels = torch.empty(world * r, device=hidden.device, dtype=labels.dtype)
        _gather(owner, all_hidden, hidden.view(r, k))
        _gather(owner, all_labels, labels.view(-1))
        w = cast_tensor(weight, torch.bfloat16)
        logits = matmul(all_hidden, w.t(), optimized=True)
        local_lse, target = local_statistics(logits, all_labels, s, rank * v, vocab_total=world * v, ignore=ignore)
        maximum = local_lse.clone()
        _reduce(owner, maximum, dist.ReduceOp.MAX)
        packed = packed_statistics(local_lse, maximum, target)
        _reduce(owner, packed, dist.ReduceOp.SUM)
        lse, counts, means = finish_statistics(maximum, packed, all_labels, r, s, world, ignore)
        loss = means[rank].clone()
        dense = None
        if diagnostics:
            received = torch.empty_like(logits)
            if world == 1:
                received.copy_(logits)
            elif owner.communication is None:
                dist.all_to_all_single(received, logits)
            else:
                owner.communication.all_to_all(received, logits)
            dense = received.view(world, r, v).transpose(0, 1).contiguous().view(b, s, world * v)
            ctx.mark_non_differentiable(dense)
        ctx.save_for_backward(all_hidden, w, all_labels, logits, lse, counts)
        ctx.rows = r
        ctx.sequence = s
        ctx.start = rank * v
        ctx.ignore = ignore
        ctx.owner = owner
        owner.forward_calls += 1
        return loss, dense

    @staticmethod
    def backward(ctx, up, _diagnostic_grad):
        h, w, labels, logits, lse, counts = ctx.saved_tensors
        owner = ctx.owner
        world = owner.world
        r = ctx.rows
        k = h.shape[1]
        ups = torch.empty(world, device=h.device, dtype=up.dtype)
        _gather(owner, ups, up.contiguous().view(1))
        dz = logit_gradient(logits, labels, lse, counts, ups, r, ctx.sequence, ctx.start, ctx.ignore,
                            vocab_total=world * w.shape[0])
        partial_dx = matmul(dz, w, optimized=True, output_dtype=torch.float32)
        if world == 1:
            local_dx = partial_dx
        else:
            local_dx = torch.empty((r, k), device=h.device, dtype=torch.float32)
            if owner.communication is None:
                dist.reduce_scatter_tensor(local_dx, partial_dx, op=dist.ReduceOp.SUM)
            else:
                owner.communication.reduce_scatter(local_dx, partial_dx, 'sum')
        dx = cast_tensor(local_dx, torch.bfloat16)
        if owner.fused_dw:
            from ..kernels.vocab_dw import weight_gradient_mean
            dw = weight_gradient_mean(dz, h, r, world, owner.dw_config)
        else:
            dw = torch.empty(w.shape, device=w.device, dtype=torch.float32)
            for source in range(world):
                partial_dw = matmul(dz[source * r:(source + 1) * r].t(), h[source * r:(source + 1) * r], optimized=True)
                accumulate_weight_gradient(partial_dw, dw, world, source == 0)
        owner.backward_calls += 1
        return dx.view(-1, ctx.sequence, k), dw, None, None, None, None


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
        if self.fused and not diagnostics and self.in_features % 8 == 0 and self.weight.shape[0] % 8 == 0:
            return _FusedVocabCE.apply(hidden, self.weight, labels, ignore_index, self), None
        return _VocabCE.apply(hidden, self.weight, labels, ignore_index, diagnostics, self)


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
        if world == 1:
            out = partial
        else:
            out = torch.empty((n, h), device=ids.device, dtype=torch.bfloat16)
            if owner.communication is None:
                dist.reduce_scatter_tensor(out, partial, op=dist.ReduceOp.SUM)
            else:
                owner.communication.reduce_scatter(out, partial, 'sum')
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
