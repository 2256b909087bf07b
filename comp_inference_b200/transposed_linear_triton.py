"""Import-path alias: the reference exposes these ops from comp_inference/transposed_linear_triton.py."""
from .ops import fused_rans_linear_transposed_triton, fused_rans_linear_transposed_triton_uncoalesced  # noqa: F401
