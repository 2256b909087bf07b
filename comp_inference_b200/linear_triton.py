"""Import-path alias: the reference exposes these ops from comp_inference/linear_triton.py."""
from .ops import fused_rans_linear_triton, fused_rans_linear_triton_uncoalesced  # noqa: F401
