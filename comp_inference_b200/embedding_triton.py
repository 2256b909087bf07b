"""Import-path alias: the reference exposes these ops from comp_inference/embedding_triton.py."""
from .ops import fused_rans_embedding_triton, fused_rans_embedding_triton_uncoalesced  # noqa: F401
