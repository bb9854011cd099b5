"""Stand-alone CUDA operators under the public names of the reference ops/triton package."""
from .attention import attention_triton, attention_triton_autograd, attention_triton_with_lse
from .attention_backward import attention_backward_triton
from .fused_qk_norm_rope import fused_qk_norm_rope_triton
from .gate_up_swiglu import gate_up_swiglu_triton
from .rms_norm import rms_norm_triton
from .rope import apply_rope_triton
from .silu_and_mul import silu_and_mul_triton

__all__ = ["attention_triton", "attention_triton_autograd", "attention_triton_with_lse", "attention_backward_triton",
           "fused_qk_norm_rope_triton", "gate_up_swiglu_triton", "rms_norm_triton", "apply_rope_triton",
           "silu_and_mul_triton"]
