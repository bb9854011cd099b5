"""`gate_up_swiglu_triton(x, gate_weight, up_weight)` (reference ops/triton/gate_up_swiglu.py:274-288)."""
from qwen3_triton.kernels.mlp import _GateUp


def gate_up_swiglu_triton(x, gate_weight, up_weight):
    if not x.is_cuda:
        raise ValueError("gate_up_swiglu_triton requires CUDA tensors")
    return _GateUp.apply(x.contiguous(), gate_weight.contiguous(), up_weight.contiguous(), True)
