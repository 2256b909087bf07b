"""GGUF export of a compressed model (comp_inference/rans_gguf.py:10-238).

Tensor names follow the reference: Hugging Face module paths shortened by ``hf_to_gguf_name`` and, per
compressed module, ``<name>.rans_exp_stream / rans_exp_states / rans_exp_sizes / rans_exp_freqs /
rans_exp_cdf / rans_man_raw / rans_info`` (or ``rans_exp_raw`` for an exponent plane stored as is), with
GGUF's signed integer types standing in for the unsigned ones (uint8 -> I8, uint16/bf16 -> I16,
uint32 -> I32: a reinterpretation, never a conversion).

The reference's writer leaves out the arrays a tiled stream cannot be decoded without.  This writer adds
them, so that a file is self-contained:

    <name>.rans_exp_tables          I32 [256]   freq | cdf << 16
    <name>.rans_exp_slot_map        I8  [4096]
    <name>.rans_exp_tile_offsets    I32 [tiles]         (tiled layout)
    <name>.rans_exp_tile_max_lens   I32 [tiles]         (tiled layout)
    <name>.rans_exp_stream_offsets  I32 [streams]       (dense layout)

and ``rans_info`` carries the package record of the safetensors writer (rans_saving.py:461-475):
[1, numel, exp_compressed, exp_streams, man_compressed, man_streams, rank, tiles_n, tiles_k, tile_height,
tile_width, *shape] instead of the reference's shorter [.., rank, *shape] (rans_gguf.py:196-205); the key
``quantization.rans_info_layout`` = "tiled_v1" tells the two apart.
"""
import json
import os
import re

import numpy as np
import torch

_RENAMES = (
    ("model.embed_tokens", "token_embd"), ("model.norm", "output_norm"), ("lm_head", "output"),
    ("self_attn.q_proj", "attn_q"), ("self_attn.k_proj", "attn_k"), ("self_attn.v_proj", "attn_v"),
    ("self_attn.o_proj", "attn_output"), ("mlp.gate_proj", "ffn_gate"), ("mlp.up_proj", "ffn_up"),
    ("mlp.down_proj", "ffn_down"), ("input_layernorm", "attn_norm"), ("post_attention_layernorm", "ffn_norm"),
)

_SIGNED = {torch.bfloat16: torch.int16, torch.uint8: torch.int8, torch.uint16: torch.int16,
           torch.uint32: torch.int32}


def hf_to_gguf_name(name: str) -> str:
    """``model.layers.3.self_attn.q_proj.weight`` -> ``blk.3.attn_q`` (rans_gguf.py:10-27)."""
    out = re.sub(r"^model\.layers\.(\d+)", r"blk.\1", name)
    for old, new in _RENAMES:
        out = out.replace(old, new)
    return out[:-len(".weight")] if out.endswith(".weight") else out


def sanitize_merges(raw_merges):
    """BPE merges as "left right" strings whatever the tokenizer backend returned (rans_gguf.py:29-42)."""
    out = []
    for m in raw_merges or []:
        if isinstance(m, str):
            out.append(m)
        elif hasattr(m, "__getitem__") and len(m) >= 2:
            out.append(f"{m[0]} {m[1]}")
        else:
            out.append(str(m))
    return out


def _find_merges(tokenizer, model_path_or_name):
    backend = getattr(tokenizer, "backend_tokenizer", None)
    if backend is not None:
        try:
            merges = sanitize_merges(backend.model.get_merges())
            if merges:
                return merges
        except Exception:
            pass
        try:                                     # the serialised backend always carries them for a BPE model
            merges = sanitize_merges(json.loads(backend.to_str()).get("model", {}).get("merges", []))
            if merges:
                return merges
        except Exception:
            pass
    if model_path_or_name:
        path = os.path.join(str(model_path_or_name), "tokenizer.json")
        if os.path.exists(path):
            with open(path, "r", encoding="utf-8") as f:
                return sanitize_merges(json.load(f).get("model", {}).get("merges", []))
    return []


def write_tokenizer(gguf_writer, tokenizer, model_path_or_name=None):
    """Vocabulary, merges, token types and special ids of a BPE tokenizer (rans_gguf.py:45-108).  Like the
    reference it refuses a tokenizer whose merges cannot be found; unlike it, it never goes to the network."""
    merges = _find_merges(tokenizer, model_path_or_name)
    if not merges:
        raise ValueError("Could not extract BPE merges.")
    gguf_writer.add_tokenizer_model("gpt2")
    gguf_writer.add_tokenizer_pre("qwen2")
    gguf_writer.add_token_merges(merges)
    vocab = tokenizer.get_vocab()
    size = max(len(vocab), max(vocab.values()) + 1 if vocab else 0)
    tokens = [b"<unk>"] * size
    for token, idx in vocab.items():
        raw = token.encode("utf-8", errors="ignore") if isinstance(token, str) else token
        if raw:
            tokens[idx] = raw
    gguf_writer.add_token_list(tokens)
    types = [1] * size
    for sid in getattr(tokenizer, "all_special_ids", []):
        if sid < size:
            types[sid] = 3
    gguf_writer.add_token_types(types)
    gguf_writer.add_token_scores([0.0] * size)
    for attr, add in (("bos_token_id", gguf_writer.add_bos_token_id), ("eos_token_id", gguf_writer.add_eos_token_id),
                      ("pad_token_id", gguf_writer.add_pad_token_id)):
        if getattr(tokenizer, attr, None) is not None:
            add(getattr(tokenizer, attr))


def _as_numpy(tensor):
    t = tensor.detach().cpu().contiguous()
    if t.dtype in _SIGNED:
        t = t.view(_SIGNED[t.dtype])
    return t.numpy()


def _u32(t):
    return t.view(torch.uint32) if t.dtype == torch.int32 else t.to(torch.uint32)


def rans_module_tensors(module):
    """(suffix, numpy array) pairs of one compressed module, in file order."""
    out = []
    dense = bool(getattr(module, "exponent_uncoalesced_interleaving", False))
    if hasattr(module, "exponent_compressed_weight"):
        out.append(("rans_exp_stream", module.exponent_compressed_weight.to(torch.uint8)))
        out.append(("rans_exp_states", _u32(module.exponent_states)))
        if getattr(module, "exponent_output_sizes", None) is not None:
            out.append(("rans_exp_sizes", _u32(module.exponent_output_sizes)))
        for key in ("freqs", "cdf"):
            val = getattr(module, "exponent_" + key, None)
            if val is not None:
                out.append(("rans_exp_" + key, val))
        out.append(("rans_exp_tables", _u32(module.exponent_tables)))
        out.append(("rans_exp_slot_map", module.exponent_slot_map.to(torch.uint8)))
        if dense:
            out.append(("rans_exp_stream_offsets", _u32(module.exponent_stream_offsets)))
        else:
            out.append(("rans_exp_tile_offsets", _u32(module.exponent_tile_offsets)))
            out.append(("rans_exp_tile_max_lens", _u32(module.exponent_tile_max_lens)))
        exp_compressed, exp_streams = 1, int(module.exponent_num_streams)
    else:
        out.append(("rans_exp_raw", module.exponent_raw))
        exp_compressed, exp_streams = 0, 0
    out.append(("rans_man_raw", module.mantissa_raw.to(torch.uint8).flatten()))
    shape = list(getattr(module, "input_shape", [])) or [int(module.expanded_size)]
    info = [1, int(module.expanded_size), exp_compressed, exp_streams, 0, 0, len(shape),
            int(getattr(module, "exponent_num_tiles_n", 0)), int(getattr(module, "exponent_num_tiles_k", 0)),
            int(getattr(module, "exponent_tile_height", 0)), int(getattr(module, "exponent_tile_width", 0))] + shape
    out.append(("rans_info", torch.tensor(info, dtype=torch.int32)))
    if getattr(module, "bias", None) is not None:
        out.append(("bias", module.bias.float()))
    return [(k, _as_numpy(v)) for k, v in out]


def save_rans_model_gguf(model, tokenizer, output_path: str, model_name: str = None, arch: str = "qwen3"):
    """Writes model + tokenizer to one GGUF file (rans_gguf.py:110-238).  ``arch`` defaults to the string the
    reference hard-codes; pass "llama" for a Llama checkpoint.  ``tokenizer`` may be None (tensors only)."""
    import gguf
    cfg = model.config
    w = gguf.GGUFWriter(output_path, arch)
    w.add_architecture()
    w.add_block_count(cfg.num_hidden_layers)
    w.add_context_length(getattr(cfg, "max_position_embeddings", 32768))
    w.add_embedding_length(cfg.hidden_size)
    w.add_feed_forward_length(cfg.intermediate_size)
    w.add_head_count(cfg.num_attention_heads)
    w.add_head_count_kv(getattr(cfg, "num_key_value_heads", None) or cfg.num_attention_heads)
    w.add_rope_dimension_count(getattr(cfg, "head_dim", None) or cfg.hidden_size // cfg.num_attention_heads)
    rope = getattr(cfg, "rope_theta", None)
    if rope is None:
        rope = (getattr(cfg, "rope_parameters", None) or {}).get("rope_theta", 1000000.0)
    w.add_rope_freq_base(float(rope))
    w.add_layer_norm_rms_eps(getattr(cfg, "rms_norm_eps", getattr(cfg, "layer_norm_epsilon", 1e-6)))
    w.add_string("quantization.method", "rans_bfloat16")
    w.add_string("quantization.rans_info_layout", "tiled_v1")
    if tokenizer is not None:
        write_tokenizer(w, tokenizer, model_name)
    count = 0
    for name, module in model.named_modules():
        if getattr(module, "compressed", None) == "rans_bfloat16":
            base = hf_to_gguf_name(name)
            for suffix, data in rans_module_tensors(module):
                w.add_tensor(f"{base}.{suffix}", data)
                count += 1
            continue
        for pname, param in module.named_parameters(recurse=False):
            if pname == "weight" and hasattr(module, "compressed"):
                continue
            full = f"{name}.{pname}" if name else pname
            w.add_tensor(hf_to_gguf_name(full), _as_numpy(param))
            count += 1
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    return count


_UNSIGNED = {"rans_exp_stream": np.uint8, "rans_exp_states": np.uint32, "rans_exp_sizes": np.uint32,
             "rans_exp_tables": np.uint32, "rans_exp_slot_map": np.uint8, "rans_exp_tile_offsets": np.uint32,
             "rans_exp_tile_max_lens": np.uint32, "rans_exp_stream_offsets": np.uint32, "rans_man_raw": np.uint8,
             "rans_exp_raw": np.uint8, "rans_exp_freqs": np.uint16, "rans_exp_cdf": np.uint16}


def read_rans_gguf(path: str):
    """Reads a file written above back into {tensor name: numpy array}, the rans_* arrays reinterpreted as the
    unsigned types they hold, plus the file's string metadata under "__meta__"."""
    import gguf
    reader = gguf.GGUFReader(path)
    out = {}
    for t in reader.tensors:
        data = np.array(t.data)
        suffix = t.name.rsplit(".", 1)[-1]
        if suffix in _UNSIGNED and data.dtype.kind == "i" and data.dtype.itemsize == np.dtype(_UNSIGNED[suffix]).itemsize:
            data = data.view(_UNSIGNED[suffix])
        out[t.name] = data
    meta = {}
    for key, field in reader.fields.items():
        if field.types and field.types[0] == gguf.GGUFValueType.STRING:
            meta[key] = bytes(field.parts[-1]).decode("utf-8", errors="replace")
    out["__meta__"] = meta
    return out
