"""Decode-time operators on the CUDA library (import path of the reference's qwen3_triton/inference package; only its
kernels module is in scope here)."""
