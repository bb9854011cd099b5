"""Qwen3 training operators and graph on hand-written sm_100a CUDA kernels behind a C ABI.

Drop-in for the operator API of the reference qwen3_triton package: the same module paths, function names
and torch.autograd.Function signatures, with every kernel launch going through csrc/libq3b200.so.
"""
from .model import PrecisionQwen3ForCausalLM, model_for_variant
from ._model import Qwen3Config

TritonQwen3ForCausalLM = PrecisionQwen3ForCausalLM
__all__ = ["TritonQwen3ForCausalLM", "PrecisionQwen3ForCausalLM", "model_for_variant", "Qwen3Config"]
