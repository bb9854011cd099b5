"""Operator API of the training hot path; every operator launches sm_100a CUDA kernels through the C ABI."""
