"""ctypes binding of the q3b200 C-ABI library (csrc/libq3b200.so).

Every operator in this package reaches the GPU through this module: it declares the argument
types of each `extern "C"` entry point listed in include/q3b200.h, converts torch tensors to raw
device pointers, and raises when the library is missing or a call is rejected. There is no CPU or
eager-PyTorch fallback.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_double, c_int, c_int64, c_void_p
from pathlib import Path

import torch

Q3_F32, Q3_BF16, Q3_F16 = 0, 1, 2
STATUS_ID_RANGE, STATUS_LABEL_RANGE, STATUS_WAIT_TIMEOUT, STATUS_EMPTY_TARGETS = 1, 2, 4, 8

_DTYPES = {torch.float32: Q3_F32, torch.bfloat16: Q3_BF16, torch.float16: Q3_F16}
FLOAT_DTYPES = tuple(_DTYPES)

LIB_PATH = Path(__file__).resolve().parent.parent / "csrc" / "libq3b200.so"

P, I, L, D = c_void_p, c_int, c_int64, c_double

# name -> (restype, argtypes); must list every symbol declared in include/q3b200.h
SIGNATURES = {
    "q3_abi_version": (I, []),
    "q3_error_string": (c_char_p, [I]),
    "q3_device_sm_count": (I, []),
    "q3_async_status": (I, [I, P]),
    "q3_residual_add": (I, [P, P, P, L, I, P]),
    "q3_cast": (I, [P, I, P, I, L, P]),
    "q3_swiglu_fwd": (I, [P, P, P, L, I, P]),
    "q3_swiglu_bwd": (I, [P, P, P, P, P, L, I, P]),
    "q3_positions": (I, [P, L, L, P]),
    "q3_rmsnorm_fwd": (I, [P, P, P, P, L, L, D, I, P]),
    "q3_rmsnorm_bwd_workspace_bytes": (L, [L, L]),
    "q3_rmsnorm_bwd": (I, [P, P, P, P, P, P, P, L, L, L, I, P]),
    "q3_rmsnorm_bwd_noalloc": (I, [P, P, P, P, P, P, L, L, I, P]),
    "q3_add_rmsnorm_fwd": (I, [P, P, P, P, P, P, L, L, D, I, P]),
    "q3_add_rmsnorm_bwd": (I, [P, P, P, P, P, P, P, P, L, L, L, I, P]),
    "q3_norm_rope_fwd": (I, [P, P, P, P, P, P, L, L, L, D, I, P]),
    "q3_norm_rope_bwd_workspace_bytes": (L, [L, L, L]),
    "q3_norm_rope_bwd": (I, [P, P, P, P, P, P, P, P, P, L, L, L, L, I, P]),
    "q3_qk_norm_rope_fwd": (I, [P, P, P, P, P, P, P, P, P, P, L, L, L, L, D, I, P]),
    "q3_qk_norm_rope_bwd_workspace_bytes": (L, [L, L, L, L]),
    "q3_qk_norm_rope_bwd": (I, [P] * 15 + [L, L, L, L, L, I, P]),
    "q3_rope_apply": (I, [P, P, P, P, L, L, L, L, I, I, I, P]),
    "q3_rope_tables": (I, [P, I, P, P, P, L, L, I, P]),
    "q3_embedding_fwd": (I, [P, I, P, P, L, L, L, I, P, P]),
    "q3_embedding_bwd_workspace_bytes": (L, [L]),
    "q3_embedding_bwd": (I, [P, I, P, P, P, L, L, L, L, I, P]),
    "q3_embedding_shard_fwd": (I, [P, I, P, I, P, I, L, L, L, L, L, P, P]),
    "q3_embedding_shard_bwd": (I, [P, I, P, I, P, P, L, L, L, L, L, D, P]),
    "q3_ce_fwd": (I, [P, P, P, P, P, P, P, L, L, L, L, I, P, P]),
    "q3_ce_local_rows": (I, [P, P, P, P, L, L, L, L, L, L, I, P, P]),
    "q3_ce_grad": (I, [P, P, P, P, P, P, L, L, L, L, L, L, L, I, P]),
    "q3_vce_pack": (I, [P, P, P, P, L, P]),
    "q3_vce_finish": (I, [P, P, P, P, P, P, P, L, L, L, L, L, P, P]),
    "q3_vce_accumulate": (I, [P, I, P, L, L, I, P]),
    "q3_adamw_multi": (I, [P, P, L, L, I, D, D, D, D, D, P]),
    "q3_adamw_multi_mp": (I, [P, P, L, L, I, I, I, D, D, D, D, D, P]),
    "q3_multi_copy": (I, [P, L, L, I, I, P]),
    "q3_gemm": (I, [P, L, L, P, L, L, P, L, L, L, I, I, P, P]),
    "q3_gemm_acc_f32": (I, [P, L, L, P, L, L, P, L, L, L, I, P, P]),
    "q3_gemm_acc": (I, [P, L, L, P, L, L, P, L, L, L, I, I, P, P]),
    "q3_linear_fwd_grouped": (I, [P, P, P, P, I, L, L, I, P, P]),
    "q3_linear_dgrad_grouped": (I, [P, P, P, P, I, L, L, I, P, P]),
    "q3_linear_wgrad_grouped": (I, [P, P, P, P, I, L, L, I, P, P]),
    "q3_down_dgrad_swiglu_bwd": (I, [P, P, P, P, P, P, L, L, L, I, P, P]),
    "q3_linear_ce_tiles": (L, [L]),
    "q3_shift_labels": (I, [P, P, L, L, L, L, P, P]),
    "q3_linear_ce_stats": (I, [P, P, P, P, P, P, L, L, L, L, L, I, P, P]),
    "q3_linear_ce_combine": (I, [P, P, P, L, L, P]),
    "q3_linear_ce_finish": (I, [P, P, P, P, P, P, P, P, L, L, L, P, P]),
    "q3_linear_ce_grad": (I, [P, P, P, P, P, P, P, L, L, L, L, L, L, I, P, P]),
    "q3_gemm_path": (I, [P, L, L, P, L, L, P, L, L, L, I, I]),
    "q3_gate_up_swiglu_fwd": (I, [P, P, P, P, P, P, L, L, L, I, P, P]),
    "q3_gate_up_path": (I, [P, P, P, P, P, P, L, L, L, I]),
    "q3_attn_fwd": (I, [P, P, P, P, P, L, L, L, L, L, D, I, P, P]),
    "q3_attn_bwd_workspace_bytes": (L, [L, L, L, L, L]),
    "q3_attn_bwd": (I, [P, P, P, P, P, P, P, P, P, P, L, L, L, L, L, L, D, I, P, P]),
    "q3_attn_fwd_bshd": (I, [P, P, P, P, P, L, L, L, L, L, D, I, P, P]),
    "q3_attn_bwd_bshd": (I, [P, P, P, P, P, P, P, P, P, P, L, L, L, L, L, L, D, I, P, P]),
    "q3_attn_path": (I, [P, P, P, P, L, I]),
    "q3_attn_bwd_group_split": (I, [L, L, L, L]),
    "q3_attn_bwd_group_policy": (I, [I]),
    "q3_gemm_tile_schedule": (I, [I]),
    "q3_gemm_cta_pairs": (I, [I]),
    "q3_selftest_wait_timeout": (I, [L, P, P, P]),
    "q3_peer_alloc": (I, [L, P, P]),
    "q3_peer_open": (I, [P, P]),
    "q3_peer_close": (I, [P]),
    "q3_peer_free": (I, [P]),
    "q3_peer_copy": (I, [P, P, L, P]),
    "q3_peer_copy_many": (I, [P, P, P, L, P]),
    "q3_reduce_scatter_pull": (I, [P, I, P, L, L, D, I, P]),
    "q3_inf_positions": (I, [P, L, L, L, P]),
    "q3_kv_append": (I, [P, P, P, P, L, L, L, L, L, L, I, P]),
    "q3_cache_attention_workspace_bytes": (L, [L, L, L, L, L, I]),
    "q3_cache_attention": (I, [P, P, P, P, P, L, L, L, L, L, L, L, L, D, I, P]),
    "q3_cache_attention_path": (I, [I]),
    "q3_gemv": (I, [P, P, P, L, L, L, I, I, P]),
    "q3_select_tokens_workspace_bytes": (L, [L, L]),
    "q3_select_tokens": (I, [P, L, L, P, L, L, P, P, P, I, L, P, L, I, P]),
    "q3_block_order": (I, [P, L, L, L, L, L, L, I, P]),
    "q3_token_blocks": (I, [P, L, P, P, L, L, P, P]),
    "q3_validation_accumulate": (I, [P, P, L, P]),
    "q3_validation_rows": (I, [P, P, L, L, L, P, P]),
}

_lib = None


class Q3Error(RuntimeError):
    """A q3b200 entry point rejected the call or a kernel reported a device-side violation."""


def lib() -> ctypes.CDLL:
    """Load libq3b200.so once. Raises if it has not been built: nothing runs without it."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise Q3Error(f"{LIB_PATH} is missing: build it with `python {LIB_PATH.parent / 'build.py'}`; "
                          "there is no fallback path")
        handle = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError here means header and library disagree
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def dt(dtype: torch.dtype) -> int:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {dtype}; float32, bfloat16 or float16 required") from None


def ptr(t):
    return None if t is None else t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def check(code: int, what: str) -> None:
    if code != 0:
        msg = lib().q3_error_string(code).decode()
        raise Q3Error(f"{what}: {msg} (code {code})")


def pointer_array(tensors):
    """Host array of device pointers for the grouped entry points (keep it alive until the call returns)."""
    return (c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def size_array(sizes):
    return (c_int64 * len(sizes))(*[int(v) for v in sizes])


def call(name: str, *args) -> None:
    check(getattr(lib(), name)(*args), name)


def workspace(nbytes: int, device) -> torch.Tensor:
    return torch.empty(max(int(nbytes), 16), dtype=torch.uint8, device=device)


_status = {}


def status_word(device) -> torch.Tensor:
    """Per-device int32 word that kernels OR violation bits into (never a trap)."""
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    word = _status.get(key)
    if word is None:
        word = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
        _status[key] = word
    return word


def read_status(device=None, *, clear=True) -> int:
    """Synchronising read of the device status word."""
    index = device if device is not None else torch.cuda.current_device()
    word = status_word(index)
    value = int(word.item())
    if clear and value:
        word.zero_()
    # the library's own word, flagged by entry points that take no status argument
    own = ctypes.c_int(0)
    with torch.cuda.device(word.device):
        check(lib().q3_async_status(1 if clear else 0, ctypes.byref(own)), "q3_async_status")
    return value | own.value


def raise_on_status(device=None) -> None:
    value = read_status(device)
    if value:
        names = [n for bit, n in ((1, "embedding id out of range"), (2, "label out of range"),
                                  (4, "kernel wait timed out"), (8, "no valid cross-entropy target")) if value & bit]
        raise Q3Error("device status: " + ", ".join(names))
