"""The reference's compress / decompress API (comp_inference/comp_inference.py),
same function names, keyword arguments and module attributes, computed on the
GPU through libci_b200.so.  Inputs may live on the CPU (the reference's scripts
pass CPU tensors); they are moved to the current CUDA device, results come back
on the device the reference would have left them on.
"""
from typing import Tuple

import numpy as np
import torch
import torch.nn as nn

from . import _lib, ccore
from .ops import rans_decompress_bf16


def _cuda(t):
    if t.is_cuda:
        return t
    if not torch.cuda.is_available():
        raise RuntimeError("comp_inference_b200 needs a CUDA device; there is no CPU path")
    return t.cuda()


def extract_exp_and_mantissa(tensor: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """bf16 -> (exponent byte, sign<<7 | mantissa byte), both uint8 with the input's shape
    (comp_inference/comp_inference.py:10-32)."""
    if tensor.dtype != torch.bfloat16:
        raise ValueError("Only bfloat16 dtype is supported for exponent/mantissa extraction.")
    src = _cuda(tensor).contiguous()
    n = src.numel()
    e = torch.empty(src.shape, dtype=torch.uint8, device=src.device)
    m = torch.empty(src.shape, dtype=torch.uint8, device=src.device)
    if n:
        _lib.check(_lib.load().ci_split_bf16(_lib.ptr(src), 1, n, 0, 0, _lib.ptr(e), _lib.ptr(m), None, None,
                                             _lib.stream()))
    return e.to(tensor.device), m.to(tensor.device)


def reconstruct_from_exp_and_mantissa(exponent, mantissa_and_sign, dtype=torch.bfloat16):
    """(sign << 15) | (exponent << 7) | mantissa -> bf16 (comp_inference/comp_inference.py:156-180).
    Plain element-wise bit arithmetic on whatever device the inputs live on."""
    if dtype != torch.bfloat16:
        raise ValueError("only bfloat16 is supported")
    e = exponent.to(torch.int32)
    m = mantissa_and_sign.to(torch.int32)
    bits = ((m & 0x80) << 8) | (e << 7) | (m & 0x7F)
    return bits.to(torch.uint16).view(torch.bfloat16)


def interleave_mantissas(mantissas: torch.Tensor, TILE_K=1024, TILE_N=32):
    """[K,N] -> zero-padded [tiles_k][tiles_n][TILE_K][TILE_N], flattened
    (comp_inference/comp_inference.py:35-64).  A pure re-layout; torch does it."""
    assert mantissas.is_contiguous(), "Mantissas tensor must be contiguous for interleaving."
    K, N = mantissas.shape
    tk, tn = -(-K // TILE_K), -(-N // TILE_N)
    pad_k, pad_n = tk * TILE_K - K, tn * TILE_N - N
    if pad_k or pad_n:
        mantissas = torch.nn.functional.pad(mantissas, (0, pad_n, 0, pad_k))
    return mantissas.view(tk, TILE_K, tn, TILE_N).permute(0, 2, 1, 3).contiguous().view(-1)


def uninterleave_mantissas(interleaved_mantissas, K, N, TILE_K=1024, TILE_N=32):
    """Inverse of interleave_mantissas; a short buffer is zero-extended
    (comp_inference/comp_inference.py:67-93)."""
    tk, tn = -(-K // TILE_K), -(-N // TILE_N)
    expected = tk * tn * TILE_K * TILE_N
    if interleaved_mantissas.numel() < expected:
        interleaved_mantissas = torch.nn.functional.pad(interleaved_mantissas, (0, expected - interleaved_mantissas.numel()))
    tiled = interleaved_mantissas.view(tk, tn, TILE_K, TILE_N)
    return tiled.permute(0, 2, 1, 3).contiguous().view(tk * TILE_K, tn * TILE_N)[:K, :N]


def _normalize(hist_dev):
    hist = hist_dev.cpu().numpy().astype(np.uint64)
    freqs = np.empty(256, np.uint16)
    cdf = np.empty(256, np.uint16)
    _lib.check(_lib.load().ci_normalize_freqs(hist.ctypes.data, freqs.ctypes.data, cdf.ctypes.data))
    return torch.from_numpy(freqs), torch.from_numpy(cdf)


def get_rans_lut(data: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """12-bit frequency and cumulative tables of a uint8 tensor, as uint16[256] CPU tensors
    (comp_inference/comp_inference.py:183-239): histogram on the GPU, normalisation on the host."""
    if data.dtype != torch.uint8:
        raise ValueError("get_rans_lut expects a uint8 tensor")
    d = _cuda(data).contiguous().view(-1)
    hist = torch.empty(256, dtype=torch.int64, device=d.device)
    _lib.check(_lib.load().ci_histogram_u8(_lib.ptr(d), d.numel(), _lib.ptr(hist), _lib.stream()))
    return _normalize(hist)


def compress_weight_cuda(weight_kn: torch.Tensor, tile_height=1024, tile_width=32, uncoalesced_interleaving=False):
    """Compresses a bf16 matrix already laid out [K,N]; every result tensor stays on the GPU.

    The one-call form of what rans_compress_module_weight_bf16 does step by step
    (split -> histogram -> table -> encode -> mantissa tiling); used by the runtime and the benchmark.
    Returns a dict with the names the saved package uses (rans_exp_stream, ...).
    """
    w = _cuda(weight_kn).contiguous()
    if w.dtype != torch.bfloat16 or w.dim() != 2:
        raise ValueError("expected a 2-D bfloat16 tensor")
    K, N = w.shape
    th, tw = ccore.effective_tile(K, N, int(tile_height), int(tile_width))
    tk, tn = -(-K // th), -(-N // tw)
    dev = w.device
    exp = torch.empty((K, N), dtype=torch.uint8, device=dev)
    man = torch.empty(tk * tn * th * tw, dtype=torch.uint8, device=dev)
    hist = torch.empty(256, dtype=torch.int64, device=dev)
    _lib.check(_lib.load().ci_split_bf16(_lib.ptr(w), K, N, th, tw, _lib.ptr(exp), _lib.ptr(man), _lib.ptr(hist), None,
                                         _lib.stream()))
    freqs, cdf = _normalize(hist)
    mgr = ccore.RansManager(K * N)
    if uncoalesced_interleaving:
        r = mgr.compress_tiled_uncoalesced(exp, freqs, cdf, th, tw, _keep_on_device=True)
    else:
        r = mgr.compress_tiled(exp, freqs, cdf, th, tw, _keep_on_device=True)
    out = dict(rans_exp_stream=r.stream, rans_exp_states=r.states, rans_exp_tables=r.tables,
               rans_exp_slot_map=r.slot_map, rans_man_raw=man, exponent_freqs=freqs, exponent_cdf=cdf,
               output_sizes=r.output_sizes, shape=(K, N), tile_height=r.tile_height, tile_width=r.tile_width,
               num_tiles_k=r.num_tiles_k, num_tiles_n=r.num_tiles_n, num_streams=r.num_streams)
    if uncoalesced_interleaving:
        out["rans_exp_stream_offsets"] = r.stream_offsets
    else:
        out["rans_exp_tile_offsets"] = r.tile_offsets
        out["rans_exp_tile_max_lens"] = r.tile_max_lens
    return out


def rans_compress_module_weight_bf16(module: nn.Module, skip_mantissa=True, tile_height=1024, tile_width=32,
                                     transpose_weight=True, uncoalesced_interleaving=False,
                                     keep_on_device=False) -> None:
    """Replaces module.weight by the compressed attributes the reference sets
    (comp_inference/comp_inference.py:344-502); attribute tensors are CPU tensors, as there, unless
    ``keep_on_device`` (not in the reference) asks to leave them on the GPU that produced them."""
    if not hasattr(module, "weight"):
        return
    if module.weight.dtype != torch.bfloat16:
        print(f"Skipping {module.weight.dtype}, expected bfloat16.")
        return
    if not skip_mantissa:
        raise NotImplementedError("mantissa entropy coding is dead code in the reference (undefined block_size, "
                                  "comp_inference.py:429-436); the sign+mantissa plane is always stored raw")
    weight = module.weight.detach()
    if transpose_weight:                                        # [out,in] -> [K=in, N=out]
        weight = weight.t()
    wk = _cuda(weight).contiguous()
    module.input_shape = list(wk.shape)
    module.expanded_size = wk.numel()
    K, N = wk.shape
    th, tw = ccore.effective_tile(K, N, int(tile_height), int(tile_width))
    tk, tn = -(-K // th), -(-N // tw)
    dev = wk.device
    exp = torch.empty((K, N), dtype=torch.uint8, device=dev)
    man = torch.empty(tk * tn * th * tw, dtype=torch.uint8, device=dev)
    hist = torch.empty(256, dtype=torch.int64, device=dev)
    mhist = torch.empty(256, dtype=torch.int64, device=dev)
    _lib.check(_lib.load().ci_split_bf16(_lib.ptr(wk), K, N, th, tw, _lib.ptr(exp), _lib.ptr(man), _lib.ptr(hist),
                                         _lib.ptr(mhist), _lib.stream()))
    module.exponent_freqs, module.exponent_cdf = _normalize(hist)
    module.mantissa_freqs, module.mantissa_cdf = _normalize(mhist)
    mgr = ccore.RansManager(module.expanded_size)
    if uncoalesced_interleaving:
        r = mgr.compress_tiled_uncoalesced(exp, module.exponent_freqs, module.exponent_cdf, th, tw,
                                           _keep_on_device=keep_on_device)
    else:
        r = mgr.compress_tiled(exp, module.exponent_freqs, module.exponent_cdf, th, tw,
                               _keep_on_device=keep_on_device)
    if r.success:
        module.exponent_compressed_weight = r.stream
        module.exponent_states = r.states
        module.exponent_output_sizes = r.output_sizes
        module.exponent_num_streams = r.num_streams
        module.exponent_tables = r.tables
        module.exponent_slot_map = r.slot_map
        module.exponent_num_tiles_n = r.num_tiles_n
        module.exponent_num_tiles_k = r.num_tiles_k
        module.exponent_tile_height = r.tile_height
        module.exponent_tile_width = r.tile_width
        module.exponent_uncoalesced_interleaving = bool(uncoalesced_interleaving)
        if uncoalesced_interleaving:
            module.exponent_stream_offsets = r.stream_offsets
        else:
            module.exponent_tile_offsets = r.tile_offsets
            module.exponent_tile_max_lens = r.tile_max_lens
    else:
        module.exponent_raw = exp if keep_on_device else exp.cpu()
    module.mantissa_raw = man if keep_on_device else man.cpu()
    module.compressed = "rans_bfloat16"
    del module.weight


def _fused(modules, tile_height, tile_width, uncoalesced_interleaving, keep_on_device=False):
    ws = [m.weight for m in modules]
    assert all(w.dtype == torch.bfloat16 for w in ws)
    assert all(w.shape[1] == ws[0].shape[1] for w in ws)
    fused = torch.cat(ws, dim=0).contiguous()
    lin = nn.Linear(fused.shape[1], fused.shape[0], bias=False, device=fused.device, dtype=fused.dtype)
    lin.weight = nn.Parameter(fused, requires_grad=False)
    rans_compress_module_weight_bf16(lin, tile_height=tile_height, tile_width=tile_width,
                                     uncoalesced_interleaving=uncoalesced_interleaving, keep_on_device=keep_on_device)
    return lin


def rans_compress_qkv_fused(self_attn_module: nn.Module, tile_height=1024, tile_width=32,
                            uncoalesced_interleaving=False, keep_on_device=False):
    """q/k/v concatenated along the output dimension and compressed as one tensor, attached under the
    name q_proj (comp_inference/comp_inference.py:242-292)."""
    a = self_attn_module
    a.q_proj = _fused([a.q_proj, a.k_proj, a.v_proj], tile_height, tile_width, uncoalesced_interleaving, keep_on_device)
    a.qkv_fused = True
    del a.k_proj
    del a.v_proj


def rans_compress_gate_up_fused(ffn_module: nn.Module, tile_height=1024, tile_width=32,
                                uncoalesced_interleaving=False, keep_on_device=False):
    """gate/up concatenated and compressed as one tensor, attached as gate_proj
    (comp_inference/comp_inference.py:295-341)."""
    f = ffn_module
    f.gate_proj = _fused([f.gate_proj, f.up_proj], tile_height, tile_width, uncoalesced_interleaving, keep_on_device)
    f.gate_up_fused = True
    del f.up_proj


def rans_compress_module_weight(module: nn.Module, tile_height=1024, tile_width=32, transpose_weight=True,
                                uncoalesced_interleaving=False, keep_on_device=False) -> None:
    """Dispatcher of comp_inference/comp_inference.py:548-570 (the int8 branch is broken upstream and not offered)."""
    if not hasattr(module, "weight"):
        return
    if module.weight.dtype == torch.bfloat16:
        rans_compress_module_weight_bf16(module, tile_height=tile_height, tile_width=tile_width,
                                         transpose_weight=transpose_weight,
                                         uncoalesced_interleaving=uncoalesced_interleaving,
                                         keep_on_device=keep_on_device)
    else:
        print(f"Module weight dtype is {module.weight.dtype}, not supported for RANS compression. Skipping.")


def rans_decompress_module_weight_bf16(module: nn.Module) -> None:
    """Restores module.weight ([K,N] as stored) from the compressed attributes in one kernel
    (comp_inference/comp_inference.py:573-713), using the module's own tile size instead of the
    hard-coded 1024x32 of :642-643."""
    if getattr(module, "compressed", None) != "rans_bfloat16":
        return
    shape = getattr(module, "input_shape", None) or getattr(module, "exponent_shape", None)
    if shape is None:
        raise RuntimeError(f"Missing shape for {module}")
    K, N = int(shape[0]), int(shape[1])
    dev = torch.device("cuda", torch.cuda.current_device())
    if hasattr(module, "exponent_compressed_weight"):
        th = int(getattr(module, "exponent_tile_height", 1024))
        tw = int(getattr(module, "exponent_tile_width", 32))
        if getattr(module, "exponent_uncoalesced_interleaving", False):
            from .ops import rans_decomp_uncoalesced
            e = rans_decomp_uncoalesced(module.exponent_compressed_weight.to(dev), module.exponent_states.to(dev),
                                        module.exponent_tables.to(dev), module.exponent_slot_map.to(dev), (K, N),
                                        module.exponent_stream_offsets.to(dev), module.exponent_output_sizes.to(dev),
                                        th, tw)
            m = uninterleave_mantissas(module.mantissa_raw.to(dev), K, N, th, tw)
            weight = reconstruct_from_exp_and_mantissa(e, m)
        else:
            weight = rans_decompress_bf16(
                module.exponent_compressed_weight.to(dev), module.exponent_states.to(dev),
                module.exponent_tables.to(dev), module.exponent_slot_map.to(dev), (K, N),
                module.exponent_tile_offsets.to(dev), module.exponent_tile_max_lens.to(dev), th, tw,
                module.mantissa_raw.to(dev))
    elif hasattr(module, "exponent_raw"):
        th = int(getattr(module, "exponent_tile_height", 1024))
        tw = int(getattr(module, "exponent_tile_width", 32))
        m = uninterleave_mantissas(module.mantissa_raw.to(dev), K, N, th, tw)
        weight = reconstruct_from_exp_and_mantissa(module.exponent_raw.to(dev).view(K, N), m)
    else:
        raise RuntimeError(f"Missing exponent data for {module}")
    module.weight = weight.cpu()


def rans_decompress_module_weight(module: nn.Module) -> None:
    """Dispatcher of comp_inference/comp_inference.py:755-778; leaves an nn.Parameter behind."""
    if not hasattr(module, "compressed"):
        return
    if module.compressed == "rans_bfloat16":
        rans_decompress_module_weight_bf16(module)
    else:
        print(f"Unknown compression type: {module.compressed}")
        return
    if not isinstance(module.weight, nn.Parameter):
        module.weight = nn.Parameter(module.weight, requires_grad=False)
