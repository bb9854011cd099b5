"""Public Qwen3 training model and variant factory (reference qwen3_triton/model.py:7-23). Unlike the
reference, any Qwen3-shaped configuration is accepted (layer count, widths), so the 4-layer slice and the
tiny test model use the same class as the 8B model."""
from dataclasses import fields, replace

from ._model import TritonQwen3ForCausalLM
from .components import Backbone, HFOrderNorm  # noqa: F401
from .configuration import OptimizationOptions, options_for_variant

_PRECISION_KEYS = {'xor_sum', 'lse_fma', 'native_delta', 'native_dq', 'sum_fma'}


class PrecisionQwen3ForCausalLM(TritonQwen3ForCausalLM):
    backbone_class = Backbone

    def __init__(self, config, options=None, *, precision_options=None):
        if precision_options is None:
            precision_options = dict(xor_sum=True, lse_fma=True, native_delta=True, native_dq=True, sum_fma=True)
        if set(precision_options) != _PRECISION_KEYS or any(type(v) is not bool for v in precision_options.values()):
            raise ValueError('Explicit five boolean precision options required')
        names = [f.name for f in fields(OptimizationOptions) if f.name != 'precision_options']
        if options is None:
            options = OptimizationOptions(**{n: False for n in names})
        elif not isinstance(options, OptimizationOptions):
            options = OptimizationOptions(**{n: getattr(options, n, False) for n in names})
        options = replace(options, precision_options=tuple(precision_options.items()))
        super().__init__(config, options)


class FusedQwen3ForCausalLM(PrecisionQwen3ForCausalLM):
    """Same parameters and state dict; every decoder layer is one fused autograd node (qwen3_triton/fused.py)."""

    def __init__(self, config, options=None, *, precision_options=None):
        from .fused import FusedBackbone
        self.backbone_class = FusedBackbone
        super().__init__(config, options, precision_options=precision_options)
        self.fused_loss = False     # True: forward(ids, labels) returns the loss only; logits are never materialised

    def forward(self, input_ids, labels=None, **kwargs):
        if not self.fused_loss or labels is None:
            return super().forward(input_ids, labels, **kwargs)
        from types import SimpleNamespace
        from .kernels.fused_loss import fused_linear_cross_entropy
        if any(kwargs.get(k) for k in ('use_cache', 'past_key_values', 'attention_mask', 'output_attentions',
                                       'output_hidden_states', 'logits_to_keep')):
            raise ValueError('Only dense unpadded causal training without cache/extra outputs is implemented; no fallback')
        hidden = self.model(input_ids, kwargs.get('position_ids'))
        loss = fused_linear_cross_entropy(hidden, self.lm_head.weight, labels)
        return SimpleNamespace(loss=loss, logits=None)


def model_for_variant(config, name, *, precision_options=None):
    """The reference's variant names plus 'b200_fused' (fused decoder layers, token-major attention)."""
    if name == 'b200_fused':
        return FusedQwen3ForCausalLM(config, OptimizationOptions(), precision_options=precision_options)
    return PrecisionQwen3ForCausalLM(config, options_for_variant(name), precision_options=precision_options)
