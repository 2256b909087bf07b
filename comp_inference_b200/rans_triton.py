"""Import-path alias: the reference exposes these ops from comp_inference/rans_triton.py."""
from .ops import rans_decomp_triton, rans_decomp_triton_tiled  # noqa: F401
