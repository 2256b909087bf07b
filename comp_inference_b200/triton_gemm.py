"""Import-path alias: the reference exposes these ops from comp_inference/triton_gemm.py."""
from .ops import triton_matmul  # noqa: F401
