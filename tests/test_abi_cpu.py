"""The C-ABI library loads without a GPU and exports every symbol include/q3b200.h declares; host-side
validation rejects bad calls before any launch."""
import re
from pathlib import Path

import pytest
import torch

from qwen3_triton import _abi

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "q3b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(q3_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _abi.lib()
    names = declared_symbols()
    assert len(names) >= 30
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/q3b200.h but not exported"
        assert name in _abi.SIGNATURES, f"{name} has no ctypes signature"
    assert set(_abi.SIGNATURES) == set(names)
    assert lib.q3_abi_version() == 1
    assert lib.q3_error_string(-2).decode() == "unsupported shape"


def test_entry_points_reject_null_and_bad_shapes_without_launching():
    lib = _abi.lib()
    assert lib.q3_residual_add(None, None, None, 16, _abi.Q3_BF16, None) == -1
    assert lib.q3_rmsnorm_fwd(1, 1, 1, 1, 4, 9000, 1e-6, _abi.Q3_BF16, None) == -2      # H > 8192
    assert lib.q3_rmsnorm_fwd(1, 1, 1, 1, 4, 64, 0.0, _abi.Q3_BF16, None) == -2          # eps must be > 0
    assert lib.q3_gemm(1, 1, 1, 1, 1, 1, 1, 0, 4, 4, _abi.Q3_BF16, _abi.Q3_BF16, None, None) == -2
    assert lib.q3_attn_fwd(1, 1, 1, 1, 1, 1, 3, 2, 8, 64, 0.125, _abi.Q3_BF16, None, None) == -2  # Hq % Hkv
    assert lib.q3_attn_fwd(1, 1, 1, 1, 1, 1, 4, 2, 8, 63, 0.125, _abi.Q3_BF16, None, None) == -2  # odd D
    assert lib.q3_norm_rope_fwd(1, 1, 1, 1, 1, 1, 4, 2, 7, 1e-6, _abi.Q3_BF16, None) == -2
    assert lib.q3_cast(1, 7, 1, 0, 4, None) == -3
    assert lib.q3_adamw_multi(1, 1, 0, 1, 4096, 1e-3, .9, .99, .1, 1e-8, None) == -2
    assert lib.q3_rmsnorm_bwd_workspace_bytes(10, 4096) > 0


def test_operators_refuse_cpu_tensors_no_fallback():
    from qwen3_triton.kernels.activation import swiglu
    from qwen3_triton.kernels.attention import causal_attention
    from qwen3_triton.kernels.embedding import embedding
    from qwen3_triton.kernels.linear import linear, matmul
    from qwen3_triton.kernels.loss import causal_cross_entropy
    from qwen3_triton.kernels.norm import rms_norm
    from qwen3_triton.kernels.norm_rope import norm_rope
    from qwen3_triton.kernels.residual import residual_add
    x = torch.randn(2, 3, 8)
    w = torch.randn(8)
    with pytest.raises(ValueError):
        rms_norm(x, w)
    with pytest.raises(ValueError):
        residual_add(x, x)
    with pytest.raises(ValueError):
        swiglu(x, x)
    with pytest.raises(ValueError):
        matmul(torch.randn(2, 3), torch.randn(3, 2))
    with pytest.raises(ValueError):
        embedding(torch.zeros(2, 3, dtype=torch.long), torch.randn(5, 8))
    with pytest.raises(ValueError):
        causal_cross_entropy(torch.randn(1, 3, 5), torch.zeros(1, 3, dtype=torch.long))
    with pytest.raises(ValueError):
        causal_attention(torch.randn(1, 2, 4, 8), torch.randn(1, 2, 4, 8), torch.randn(1, 2, 4, 8))
    with pytest.raises(ValueError):
        norm_rope(torch.randn(1, 2, 2, 8), w, torch.randn(1, 2, 8), torch.randn(1, 2, 8))
    with pytest.raises(ValueError):
        linear(torch.randn(2, 8).t(), torch.randn(4, 2))


def test_adamw_configuration_errors():
    from qwen3_triton.runtime.adamw import TritonAdamW
    p = torch.nn.Parameter(torch.zeros(4))
    with pytest.raises(ValueError):
        TritonAdamW([p], lr=-1)
    with pytest.raises(ValueError):
        TritonAdamW([p], block=1000)
    opt = TritonAdamW([p])
    p.grad = torch.zeros(4)
    with pytest.raises(ValueError):   # CPU parameter: no fallback
        opt.step()
