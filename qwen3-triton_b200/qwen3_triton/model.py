"""Public Qwen3 training model and variant factory (import path of the reference's qwen3_triton/model.py).

Unlike the reference class, any Qwen3-shaped configuration is accepted (layer count, widths), so the 4-layer slice and
the tiny test model use the same class as the 8B model.
"""
from dataclasses import replace

from ._model import OptimizationOptions, TritonQwen3ForCausalLM, options_for_variant, widen_options

PRECISION_SWITCHES = ('xor_sum', 'lse_fma', 'native_delta', 'native_dq', 'sum_fma')


def checked_precision_options(given):
    """The five attention precision switches of the reference API, all explicit booleans (default: all on). The CUDA
    attention kernels have one arithmetic, so the switches are validated, stored with the options and passed on."""
    if given is None:
        return dict.fromkeys(PRECISION_SWITCHES, True)
    if sorted(given) != sorted(PRECISION_SWITCHES) or not all(isinstance(v, bool) for v in given.values()):
        raise ValueError('Explicit five boolean precision options required')
    return dict(given)


class PrecisionQwen3ForCausalLM(TritonQwen3ForCausalLM):
    """The graph the 8B training runs use: options widened to the full switch set (missing switches off, as when the
    reference is handed a bare ComputeOptions) plus the attention precision switches."""

    def __init__(self, config, options=None, *, precision_options=None):
        chosen = checked_precision_options(precision_options)
        wide = widen_options(options if options is not None else object())
        super().__init__(config, replace(wide, precision_options=tuple(chosen.items())))


class FusedQwen3ForCausalLM(PrecisionQwen3ForCausalLM):
    """Same parameters and state dict; every decoder layer is one fused autograd node (qwen3_triton/fused.py).
    With `fused_loss` set, forward(ids, labels) goes from hidden states to the loss without materialising logits."""

    def __init__(self, config, options=None, *, precision_options=None):
        from .fused import FusedBackbone
        self.backbone_class = FusedBackbone
        super().__init__(config, options, precision_options=precision_options)
        self.fused_loss = False

    def forward(self, input_ids, labels=None, **kwargs):
        from ._model import Leaf
        if not self.fused_loss or labels is None or not isinstance(self.lm_head, Leaf):
            return super().forward(input_ids, labels, **kwargs)
        from types import SimpleNamespace
        from ._model import _UNSUPPORTED
        from .kernels.fused_loss import fused_linear_cross_entropy
        if any(kwargs.get(k) for k in _UNSUPPORTED):
            raise ValueError('Only dense unpadded causal training without cache/extra outputs is implemented; no fallback')
        hidden = self.model(input_ids, kwargs.get('position_ids'))
        loss = fused_linear_cross_entropy(hidden, self.lm_head.weight, labels)
        return SimpleNamespace(loss=loss, logits=None)


def model_for_variant(config, name, *, precision_options=None):
    """The reference's variant names plus 'b200_fused' (fused decoder layers, token-major attention)."""
    if name == 'b200_fused':
        return FusedQwen3ForCausalLM(config, OptimizationOptions(), precision_options=precision_options)
    return PrecisionQwen3ForCausalLM(config, options_for_variant(name), precision_options=precision_options)
