"""FSDP2 wrapping of the Qwen3 graph with a vocabulary-parallel loss head and per-layer recomputation.

Behaviour of the reference's scripts/vocab_model_v12.py:17-56, training/fsdp/official.py:22-63 and
training/fsdp/activation_checkpoint.py:4-19: every decoder layer, the embedding and the final norm are their
own FSDP unit with bf16 parameters / fp32 reductions; the last `keep_full_layers` layers stay gathered after
forward (no second all-gather in backward); every `checkpoint_every`-th layer is recomputed in backward
(non-reentrant); the lm_head becomes a VocabParallelCE whose fp32 vocabulary shard is kept out of FSDP because
its gradient is already averaged over data ranks. The wrapped model maps (input_ids, labels) to a loss only.
"""
import torch
from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

from ..model import PrecisionQwen3ForCausalLM
from .vocab_parallel import VocabParallelCE


def checkpoint_layer_indices(layer_count, *, all_layers=False, every=0):
    if layer_count < 1 or type(every) is not int or every < 0:
        raise ValueError('Positive layer count and nonnegative integer checkpoint interval required')
    if all_layers and every:
        raise ValueError('Choose all-layer or interval checkpoint, not both')
    if all_layers:
        return tuple(range(layer_count))
    return tuple(range(0, layer_count, every)) if every else ()


def canonical_parameter_name(name):
    return name.replace('_checkpoint_wrapped_module.', '')


def wrap_decoder_checkpoint(layer, *, mode='full'):
    if mode != 'full':
        raise ValueError('Only full recomputation is supported')
    from torch.distributed.algorithms._checkpoint.checkpoint_wrapper import CheckpointImpl, checkpoint_wrapper
    return checkpoint_wrapper(layer, preserve_rng_state=True, checkpoint_impl=CheckpointImpl.NO_REENTRANT)


def shard_vocab_loss_model(model, *, keep_full_layers, checkpoint_every, skip_embedding_backward_gather,
                           fused_vocab_dw=False, communication=None, mesh=None, checkpoint_mode='full',
                           layers_per_unit=1, vocab_parallel_embedding=False, forward_prefetch=1):
    """Reference surface (scripts/vocab_model_v12.py:35-56) plus three knobs: `checkpoint_mode` ('full' as the
    reference, 'selective', or 'none' where memory allows: 36 layers at 2048 tokens keep about 5 GB), `layers_per_unit`
    (an int, or a sequence of unit sizes that sums to the layer count), `forward_prefetch` (all-gathers issued that
    many units ahead in forward) and `vocab_parallel_embedding` (the token
    table stays row-sharded outside FSDP instead of being gathered and its dense gradient reduce-scattered)."""
    if model.config.tie_word_embeddings:
        raise ValueError('Untied head required')
    if not 0 <= keep_full_layers <= len(model.model.layers):
        raise ValueError('Invalid retention count')
    if not isinstance(model, PrecisionQwen3ForCausalLM):
        raise TypeError('Supported Qwen3 graph required')
    # the graph hands (hidden, labels) to any lm_head that is not a plain weight leaf: the model becomes loss-only
    model.lm_head = VocabParallelCE(model.lm_head.weight.detach().cpu(), fused_dw=fused_vocab_dw,
                                    communication=communication)
    body = model.model
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
    kw = dict(mp_policy=mp) if mesh is None else dict(mp_policy=mp, mesh=mesh)
    ignored = {model.lm_head.weight}
    if vocab_parallel_embedding:
        from .vocab_parallel import VocabParallelEmbedding
        body.embed_tokens = VocabParallelEmbedding(body.embed_tokens.weight.detach().cpu(), communication=communication)
        ignored.add(body.embed_tokens.weight)
    else:
        fully_shard(body.embed_tokens.float(), reshard_after_forward=True, **kw)
        if skip_embedding_backward_gather:
            body.embed_tokens.set_unshard_in_backward(False)
    checkpointed = checkpoint_layer_indices(len(body.layers), every=checkpoint_every)
    if isinstance(layers_per_unit, int):
        if layers_per_unit < 1:
            raise ValueError('layers_per_unit must be positive')
        sizes = [min(layers_per_unit, len(body.layers) - first) for first in range(0, len(body.layers), layers_per_unit)]
    else:
        sizes = [int(n) for n in layers_per_unit]
        if not sizes or min(sizes) < 1 or sum(sizes) != len(body.layers):
            raise ValueError('layers_per_unit sizes must be positive and sum to the number of layers')
    for index, layer in enumerate(body.layers):
        layer = layer.float()
        if index in checkpointed:
            if hasattr(layer, 'recompute'):
                # fused layers checkpoint inside their own backward ('full' or 'selective')
                layer.recompute = {'full': 2, 'selective': 1, 'none': 0}[checkpoint_mode]
            else:
                if checkpoint_mode != 'none':
                    layer = wrap_decoder_checkpoint(layer, mode='full')
        body.layers[index] = layer
    # One FSDP unit per `layers_per_unit` consecutive layers (1 = the reference's policy). FSDP2's Python
    # hooks cost about a millisecond per unit and direction; at 2048 tokens per GPU a B200 finishes a
    # layer's forward in about that time, so larger units keep the GPU fed. Collective payloads grow by
    # the same factor (4 layers: 1.5 GB gathered, 3 GB reduced), still far below the memory budget.
    first = 0
    heads = []
    for size in sizes:
        group = [body.layers[i] for i in range(first, first + size)]
        retain = first + len(group) - 1 >= len(body.layers) - keep_full_layers
        fully_shard(group if len(group) > 1 else group[0], reshard_after_forward=not retain, **kw)
        heads.append(group[0])
        first += size
    # `forward_prefetch` units ahead: FSDP2's default issues the next unit's all-gather when the current unit starts,
    # which does not cover the ~1 ms all-gather latency when the first units are single layers
    if forward_prefetch > 1:
        for index, head in enumerate(heads):
            ahead = heads[index + 1:index + 1 + forward_prefetch]
            if ahead:
                head.set_modules_to_forward_prefetch(ahead)
    fully_shard(body.norm.float(), reshard_after_forward=True, **kw)
    body.rotary_emb.cuda()
    fully_shard(model, reshard_after_forward=True, ignored_params=ignored, **kw)
    if forward_prefetch > 1 and heads:
        # the root unit runs first: let it start the first decoder units' all-gathers before the embedding lookup
        model.set_modules_to_forward_prefetch(heads[:forward_prefetch])
    model.config.use_cache = False
    return model
