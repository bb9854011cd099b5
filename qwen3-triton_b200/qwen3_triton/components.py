"""Recipe: which operator-API call carries out each step of a decoder block, chosen from the optimisation switches.

The reference expresses the optimised graph as subclasses of its module tree (qwen3_triton/components.py:9-54 there:
HF-order norm, fused QK-norm+RoPE, fused gate/up+SwiGLU, the `candidate` attention entry). Here the graph
(qwen3_triton/_model.py) is one set of classes and this object is its only variable part, so an ablation variant is
a Recipe with one switch off, not another class. Every method takes the parameter leaf (or branch) it needs and
calls the public operators of qwen3_triton.kernels - the same entry points a user of the operator API calls.
"""
import torch

from ._model import widen_options
from .kernels import math_precision
from .kernels.activation import swiglu
from .kernels.attention import causal_attention
from .kernels.attention_precision import candidate
from .kernels.embedding import embedding
from .kernels.linear import linear
from .kernels.loss import causal_cross_entropy
from .kernels.mlp_precision import gate_up_swiglu
from .kernels.norm import rms_norm
from .kernels.residual import residual_add
from .kernels.rotary import apply_rotary


class Recipe:
    def __init__(self, options):
        self.options = options
        self.wide = widen_options(options)
        # the plain graph (ComputeOptions: no fusion switches at all) goes through the first-generation operator
        # names, the optimised graph and its ablations through the ones the 8B training graph imports
        self.optimised_graph = hasattr(options, 'norm_rope_fusion')
        self.precision = dict(self.wide.precision_options)

    # -- elementwise / lookup
    def embed(self, ids, table):
        return embedding(ids, table.weight)

    def add(self, a, b):
        return residual_add(a, b)

    def normalise(self, x, scale):
        fn = math_precision.rms_norm if self.optimised_graph else rms_norm
        return fn(x, scale.weight, scale.eps)

    def project(self, x, matrix):
        return linear(x, matrix.weight, optimized=self.options.linear_optimized)

    # -- attention
    def normalise_and_rotate(self, x, scale, rope):
        """x [B,S,heads,D]: per-head RMSNorm then split-half RoPE, in one kernel when the fusion is on."""
        cos, sin = rope
        if self.optimised_graph and self.wide.norm_rope_fusion:
            return math_precision.norm_rope(x, scale.weight, cos, sin, scale.eps)
        return apply_rotary(self.normalise(x, scale), cos, sin)

    def attend(self, q, k, v):
        """[B,heads,S,D] contiguous -> [B,Hq,S,D]; softmax scale 1/sqrt(D)."""
        d = q.shape[-1]
        if self.optimised_graph and d == 128 and q.dtype == torch.bfloat16:
            return candidate(q, k, v, fusion=False, lane_sum=True, round_kv=True, reciprocal=1,
                             stages=2 if self.options.attention_optimized else 1, **self.precision)
        return causal_attention(q, k, v, scale=d ** -0.5, optimized=self.options.attention_optimized)

    # -- MLP
    def gated_mlp(self, x, mlp):
        if self.optimised_graph and self.wide.mlp_fusion:
            y = gate_up_swiglu(x, mlp.gate_proj.weight, mlp.up_proj.weight, optimized=self.options.linear_optimized)
        elif self.optimised_graph:
            y = math_precision.swiglu(self.project(x, mlp.gate_proj), self.project(x, mlp.up_proj))
        else:
            y = swiglu(self.project(x, mlp.gate_proj), self.project(x, mlp.up_proj))
        return self.project(y, mlp.down_proj)

    # -- loss on materialised logits (shift inside the operator)
    def loss(self, logits, labels):
        return causal_cross_entropy(logits, labels, optimized=self.options.loss_optimized)
