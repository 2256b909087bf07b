"""B200-native implementation of comp_inference's compressed-weight path.

Same import surface as the reference package (comp_inference/__init__.py:13-59);
the compute is hand-written CUDA for sm_100a behind the C ABI of
include/comp_inference_b200.h, loaded from csrc/libci_b200.so.
"""
from . import ccore  # noqa: F401
from .comp_inference import (  # noqa: F401
    compress_weight_cuda,
    extract_exp_and_mantissa,
    get_rans_lut,
    interleave_mantissas,
    rans_compress_gate_up_fused,
    rans_compress_module_weight,
    rans_compress_qkv_fused,
    rans_decompress_module_weight,
    reconstruct_from_exp_and_mantissa,
    uninterleave_mantissas,
)
from .ops import (  # noqa: F401
    fused_rans_embedding_triton,
    fused_rans_embedding_triton_uncoalesced,
    fused_rans_linear_transposed_triton,
    fused_rans_linear_transposed_triton_uncoalesced,
    fused_rans_linear_triton,
    fused_rans_linear_triton_uncoalesced,
    rans_decomp_triton,
    rans_decomp_triton_tiled,
    rans_decompress_bf16,
    triton_matmul,
)
from .rans_saving import (  # noqa: F401
    compress_model,
    compressed_state_dict,
    load_compressed_model,
    pack_and_save_tensors,
    save_rans_model_package,
)
from .rans_gguf import hf_to_gguf_name, read_rans_gguf, save_rans_model_gguf  # noqa: F401
from .pytorch_runtime import (  # noqa: F401
    RansEmbedding,
    RansLinear,
    RansLMHead,
    RansRowParallelLinear,
    RansWorkspace,
    RansFusedLinear,
    RansFusedSlice,
    RansVocabParallelLMHead,
    close_tensor_parallel,
    load_compressed_model_with_auto_model,
    patch_model,
    patch_model_tensor_parallel,
    prepare_model,
)
from ._lib import check_status, reserve_workspace, validate_compressed  # noqa: F401

__all__ = [n for n in dir() if not n.startswith("_")]
