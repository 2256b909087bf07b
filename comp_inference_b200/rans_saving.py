"""Compressed model packages on disk: the reference's safetensors + config.json layout
(comp_inference/rans_saving.py), same key names, dtypes and ``rans_info`` record, so a package
written by either side loads on the other.

    <module>.rans_exp_stream        uint8     <module>.rans_exp_tile_offsets   uint32
    <module>.rans_exp_states        uint32    <module>.rans_exp_tile_max_lens  uint32
    <module>.rans_exp_tables        uint32    <module>.rans_man_raw            uint8
    <module>.rans_exp_slot_map      uint8     <module>.rans_info               int32
    (dense layout: rans_exp_stream_offsets instead of the two tile arrays, plus rans_exp_sizes)

``rans_info`` = [1, numel, exp_compressed, exp_streams, man_compressed, man_streams, rank,
num_tiles_n, num_tiles_k, tile_height, tile_width, *shape]  (rans_saving.py:461-475).
"""
import json
import os

import torch
import torch.nn as nn

from . import comp_inference as ci
from .pytorch_runtime import patch_model, prepare_model

METADATA = {"format": "pt", "compression_method": "rans_bfloat16"}


def _bf16_linear(m):
    return isinstance(m, nn.Linear) and m.weight.dtype == torch.bfloat16 and m.bias is None


def compress_model(model, tile_height=1024, tile_width=32, layer_tiles=None, tied_lm_head=None, fuse=False,
                   keep_on_device=False):
    """Compresses every bf16 nn.Linear / nn.Embedding of a Hugging Face causal LM in place, the way the
    reference's end-to-end script does (tests/test_full_model_rans.py:75-130): linears are stored
    transposed ([in, out]); the embedding table and the LM head keep their [vocab, hidden] layout.
    ``layer_tiles`` maps a module name to (tile_height, tile_width) for per-layer tile sizes.
    ``fuse``: q/k/v and gate/up projections are concatenated and compressed as one tensor each
    (rans_compress_qkv_fused / rans_compress_gate_up_fused, as the reference's script does with its
    fuse option, tests/test_full_model_rans.py:97-118); save such a model with ``fuse=True``.
    ``keep_on_device``: leave the compressed tensors on the GPU instead of moving them to the host as the
    reference does (for a model that is patched and run right away, compressed_state_dict(to_cpu=False))."""
    layer_tiles = layer_tiles or {}
    if tied_lm_head is None:
        tied_lm_head = bool(getattr(model.config, "tie_word_embeddings", False))
    if fuse:
        for name, module in list(model.named_modules()):
            if all(_bf16_linear(getattr(module, a, None)) for a in ("q_proj", "k_proj", "v_proj")):
                th, tw = layer_tiles.get(name + ".q_proj", (tile_height, tile_width))
                ci.rans_compress_qkv_fused(module, tile_height=th, tile_width=tw, keep_on_device=keep_on_device)
            if all(_bf16_linear(getattr(module, a, None)) for a in ("gate_proj", "up_proj")):
                th, tw = layer_tiles.get(name + ".gate_proj", (tile_height, tile_width))
                ci.rans_compress_gate_up_fused(module, tile_height=th, tile_width=tw, keep_on_device=keep_on_device)
    for name, module in list(model.named_modules()):
        if getattr(module, "compressed", None) is not None:
            continue
        if not isinstance(module, (nn.Linear, nn.Embedding)) or module.weight.dtype != torch.bfloat16:
            continue
        is_head = name.endswith("lm_head")
        if is_head and tied_lm_head:
            continue
        th, tw = layer_tiles.get(name, (tile_height, tile_width))
        keep_layout = is_head or isinstance(module, nn.Embedding)
        ci.rans_compress_module_weight(module, tile_height=th, tile_width=tw, transpose_weight=not keep_layout,
                                       keep_on_device=keep_on_device)
    return model


def _save_rans_attributes(tensors, base, module, to_cpu=True):
    """One module's tensors under the reference's key names (rans_saving.py:352-481)."""
    mv = (lambda t: t.cpu()) if to_cpu else (lambda t: t)
    u32 = lambda t: mv(t).view(torch.uint32) if t.dtype == torch.int32 else mv(t).to(torch.uint32)
    dense = bool(getattr(module, "exponent_uncoalesced_interleaving", False))
    if hasattr(module, "exponent_compressed_weight"):
        tensors[base + "rans_exp_stream"] = mv(module.exponent_compressed_weight).to(torch.uint8)
        tensors[base + "rans_exp_states"] = u32(module.exponent_states)
        tensors[base + "rans_exp_tables"] = u32(module.exponent_tables)
        tensors[base + "rans_exp_slot_map"] = mv(module.exponent_slot_map).to(torch.uint8)
        if dense:
            tensors[base + "rans_exp_stream_offsets"] = u32(module.exponent_stream_offsets)
            tensors[base + "rans_exp_sizes"] = u32(module.exponent_output_sizes)
        else:
            tensors[base + "rans_exp_tile_offsets"] = u32(module.exponent_tile_offsets)
            tensors[base + "rans_exp_tile_max_lens"] = u32(module.exponent_tile_max_lens)
        exp_compressed, exp_streams = 1, int(module.exponent_num_streams)
    else:
        tensors[base + "rans_exp_raw"] = mv(module.exponent_raw)
        exp_compressed, exp_streams = 0, 0
    tensors[base + "rans_man_raw"] = mv(module.mantissa_raw).to(torch.uint8)
    shape = list(getattr(module, "input_shape", []))
    info = [1, int(module.expanded_size), exp_compressed, exp_streams, 0, 0, len(shape),
            int(getattr(module, "exponent_num_tiles_n", 0)), int(getattr(module, "exponent_num_tiles_k", 0)),
            int(getattr(module, "exponent_tile_height", 0)), int(getattr(module, "exponent_tile_width", 0))] + shape
    tensors[base + "rans_info"] = torch.tensor(info, dtype=torch.int32)
    if getattr(module, "bias", None) is not None:
        tensors[base + "bias"] = mv(module.bias.detach())


def compressed_state_dict(model, tied_lm_head: bool = False, to_cpu: bool = True):
    """The tensors pack_and_save_tensors would write, as a dict: what patch_model and
    patch_model_tensor_parallel take, without the round trip through a file.  CPU tensors like a loaded
    package, or -- ``to_cpu=False`` -- wherever the compressed attributes live (compress_model(keep_on_device=True))."""
    mv = (lambda t: t.cpu()) if to_cpu else (lambda t: t)
    tensors, handled = {}, set()
    if tied_lm_head:
        handled.update({"lm_head.weight", "model.lm_head.weight"})
    for name, module in model.named_modules():
        if getattr(module, "compressed", None) == "rans_bfloat16":
            _save_rans_attributes(tensors, name + ".", module, to_cpu)
            handled.add(name + ".weight")
            handled.add(name + ".bias")
    for pname, param in model.named_parameters():
        if pname not in handled:
            tensors[pname] = mv(param.detach()).contiguous()
    return tensors


def pack_and_save_tensors(model, output_path: str, fuse: bool = False, tied_lm_head: bool = False):
    """model.safetensors of a package (rans_saving.py:177-245): compressed modules under their rans_* keys,
    every other parameter under its own name, a tied LM head dropped."""
    from safetensors.torch import save_file
    tensors = compressed_state_dict(model, tied_lm_head=tied_lm_head)
    meta = dict(METADATA, fused_projections=str(fuse))
    save_file(tensors, output_path, metadata=meta)
    return len(tensors)


def save_rans_model_package(model, tokenizer, output_dir: str, fuse: bool = False, tied_lm_head: bool = False):
    """config.json (with quantization_config.layer_configs), tokenizer files and model.safetensors
    (rans_saving.py:19-109).  As in the reference, an unfused package goes to ``output_dir + "_unfused"``."""
    if not fuse:
        output_dir = output_dir + "_unfused"
    os.makedirs(output_dir, exist_ok=True)
    layer_configs = {}
    for name, module in model.named_modules():
        if tied_lm_head and "lm_head" in name:
            continue
        if getattr(module, "compressed", None) == "rans_bfloat16":
            key = name
            if fuse:
                key = key.replace("gate_proj", "gate_up_proj") if "gate_proj" in key else key.replace("q_proj", "qkv_proj")
            layer_configs[key] = {"tile_height": int(getattr(module, "exponent_tile_height", 1024)),
                                  "tile_width": int(getattr(module, "exponent_tile_width", 32)),
                                  "uncoalesced_interleaving": bool(getattr(module, "exponent_uncoalesced_interleaving", False))}
    quant = {"quant_method": "rans", "compression": "rans_bfloat16", "layer_configs": layer_configs,
             "default_tile_height": 1024, "default_tile_width": 32, "fused_projections": fuse}
    cfg = model.config.to_dict()
    cfg["quantization_config"] = quant
    with open(os.path.join(output_dir, "config.json"), "w") as f:
        json.dump(cfg, f, indent=2, default=str)
    if tokenizer is not None:
        tokenizer.save_pretrained(output_dir)
    pack_and_save_tensors(model, os.path.join(output_dir, "model.safetensors"), fuse=fuse, tied_lm_head=tied_lm_head)
    return output_dir


def load_compressed_model(package_dir: str, device="cuda", split_k: int = 1):
    """Rebuilds the model of a package without the dense checkpoint: architecture from config.json (random
    init, immediately overwritten), compressed modules swapped in by name, all tensors assigned from
    model.safetensors.  (The reference's loader of this name is stale -- it reads keys its writer never
    writes, rans_saving.py:577 -- so this follows the live loader, pytorch_runtime.py:552-642, minus the
    download of the dense model.)"""
    from safetensors.torch import load_file
    from transformers import AutoConfig, AutoModelForCausalLM
    with open(os.path.join(package_dir, "config.json")) as f:
        raw = json.load(f)
    quant = raw.pop("quantization_config", {}) or {}
    config = AutoConfig.for_model(raw.pop("model_type"), **raw)
    model = AutoModelForCausalLM.from_config(config, torch_dtype=torch.bfloat16)
    state = load_file(os.path.join(package_dir, "model.safetensors"), device="cpu")
    patch_model(model, state, quant.get("layer_configs", {}), quant.get("default_tile_height", 1024),
                quant.get("default_tile_width", 32), split_k)
    if getattr(config, "tie_word_embeddings", False) and "lm_head.rans_exp_stream" not in state:
        raise RuntimeError("a package with a tied LM head needs the dense embedding to tie to; untie before compressing")
    return prepare_model(model.to(device))
