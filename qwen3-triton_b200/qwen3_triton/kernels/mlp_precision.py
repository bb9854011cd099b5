"""Name used by the 8B training graph (reference qwen3_triton/kernels/mlp_precision.py:65-66)."""
from .mlp import _GateUp, gate_up_swiglu  # noqa: F401
