"""GGUF export: names follow the reference's mapping, the unsigned arrays survive the signed GGUF types, and
a written file decodes back to the original weights with nothing but the file (CPU oracle as the decoder)."""
import types

import numpy as np
import pytest
import torch
import torch.nn as nn

from conftest import bits, make_weight

gguf = pytest.importorskip("gguf")

from comp_inference_b200 import rans_gguf  # noqa: E402


def test_names_follow_reference_mapping():
    cases = {
        "model.layers.3.self_attn.q_proj.weight": "blk.3.attn_q",
        "model.layers.11.mlp.down_proj": "blk.11.ffn_down",
        "model.layers.0.input_layernorm.weight": "blk.0.attn_norm",
        "model.layers.0.post_attention_layernorm.weight": "blk.0.ffn_norm",
        "model.embed_tokens.weight": "token_embd",
        "model.norm.weight": "output_norm",
        "lm_head": "output",
        "model.layers.7.self_attn.o_proj.bias": "blk.7.attn_output.bias",
    }
    for hf, want in cases.items():
        assert rans_gguf.hf_to_gguf_name(hf) == want


def test_sanitize_merges_forms():
    assert rans_gguf.sanitize_merges(["a b", ("c", "d"), ["e", "f"]]) == ["a b", "c d", "e f"]
    assert rans_gguf.sanitize_merges(None) == []


def _attach(module, w, O, th, tw, dense=False):
    """Module attributes as the compressor sets them, produced here by the CPU oracle."""
    K, N = w.shape
    r = O.compress_bf16(bits(w), th, tw)
    t = torch.from_numpy
    module.input_shape = [K, N]
    module.expanded_size = K * N
    module.exponent_freqs = t(r["freqs"].astype(np.int16)).view(torch.uint16)
    module.exponent_cdf = t(r["cdf"].astype(np.int16)).view(torch.uint16)
    module.exponent_compressed_weight = t(r.stream.copy())
    module.exponent_states = t(r.states.view(np.int32).copy())
    module.exponent_output_sizes = t(r.output_sizes.view(np.int32).copy())
    module.exponent_num_streams = r.num_streams
    module.exponent_tables = t(r.tables.view(np.int32).copy())
    module.exponent_slot_map = t(r.slot_map.copy())
    module.exponent_num_tiles_n, module.exponent_num_tiles_k = r.num_tiles_n, r.num_tiles_k
    module.exponent_tile_height, module.exponent_tile_width = r.tile_height, r.tile_width
    module.exponent_uncoalesced_interleaving = False
    module.exponent_tile_offsets = t(r.tile_offsets.view(np.int32).copy())
    module.exponent_tile_max_lens = t(r.tile_max_lens.view(np.int32).copy())
    module.mantissa_raw = t(r["mantissa"].copy())
    module.compressed = "rans_bfloat16"
    module.weight = None
    return r


class _Block(nn.Module):
    def __init__(self):
        super().__init__()
        self.self_attn = nn.Module()
        self.self_attn.q_proj = nn.Linear(96, 160, bias=True, dtype=torch.bfloat16)
        self.mlp = nn.Module()
        self.mlp.down_proj = nn.Linear(160, 96, bias=False, dtype=torch.bfloat16)
        self.input_layernorm = nn.LayerNorm(96, dtype=torch.bfloat16)


class _Model(nn.Module):
    def __init__(self):
        super().__init__()
        self.model = nn.Module()
        self.model.layers = nn.ModuleList([_Block()])
        self.model.norm = nn.LayerNorm(96, dtype=torch.bfloat16)
        self.config = types.SimpleNamespace(num_hidden_layers=1, max_position_embeddings=128, hidden_size=96,
                                            intermediate_size=160, num_attention_heads=4, num_key_value_heads=2,
                                            rope_theta=10000.0, rms_norm_eps=1e-5)


def test_file_is_self_contained(oracle, tmp_path):
    model = _Model()
    blk = model.model.layers[0]
    wq = make_weight(96, 160, 11)            # stored [in, out]
    wd = make_weight(160, 96, 12)
    rq = _attach(blk.self_attn.q_proj, wq, oracle, 64, 32)
    _attach(blk.mlp.down_proj, wd, oracle, 128, 16)
    path = str(tmp_path / "m.gguf")
    n = rans_gguf.save_rans_model_gguf(model, None, path, arch="llama")
    got = rans_gguf.read_rans_gguf(path)
    assert n == len(got) - 1
    assert got["__meta__"]["quantization.method"] == "rans_bfloat16"
    assert got["__meta__"]["quantization.rans_info_layout"] == "tiled_v1"

    # plain parameters keep their bits under the shortened names
    assert got["blk.0.attn_norm"].dtype == np.int16 and got["blk.0.attn_norm"].shape == (96,)
    assert np.array_equal(got["output_norm"].view(np.uint16), bits(model.model.norm.weight.detach()))
    assert "blk.0.attn_q.bias" in got and got["blk.0.attn_q.bias"].dtype == np.float32

    # unsigned arrays survive the signed container types
    assert np.array_equal(got["blk.0.attn_q.rans_exp_stream"], rq.stream)
    assert got["blk.0.attn_q.rans_exp_states"].dtype == np.uint32
    assert np.array_equal(got["blk.0.attn_q.rans_exp_states"], rq.states)
    assert np.array_equal(got["blk.0.attn_q.rans_exp_freqs"], rq["freqs"])

    # decode each module from the file alone
    for base, w in (("blk.0.attn_q", wq), ("blk.0.ffn_down", wd)):
        info = got[base + ".rans_info"].tolist()
        assert info[0] == 1 and info[2] == 1 and info[4] == 0
        rank = info[6]
        tn, tk, th, tw = info[7:11]
        K, N = info[11:11 + rank]
        assert info[1] == K * N and info[3] == tn * tk * 2 * tw
        r = dict(stream=got[base + ".rans_exp_stream"], states=got[base + ".rans_exp_states"],
                 tables=got[base + ".rans_exp_tables"], slot_map=got[base + ".rans_exp_slot_map"],
                 tile_offsets=got[base + ".rans_exp_tile_offsets"],
                 tile_max_lens=got[base + ".rans_exp_tile_max_lens"])
        out = oracle.decode_bf16(r, got[base + ".rans_man_raw"], K, N, th, tw)
        assert np.array_equal(out, bits(w))


def test_raw_exponent_plane_module(oracle, tmp_path):
    model = _Model()
    mod = model.model.layers[0].mlp.down_proj
    w = make_weight(160, 96, 5)
    e, m = oracle.split_bf16(bits(w))
    mod.input_shape, mod.expanded_size = [160, 96], 160 * 96
    mod.exponent_raw = torch.from_numpy(e.copy())
    mod.mantissa_raw = torch.from_numpy(m.copy())
    mod.compressed = "rans_bfloat16"
    path = str(tmp_path / "raw.gguf")
    rans_gguf.save_rans_model_gguf(model, None, path)
    got = rans_gguf.read_rans_gguf(path)
    info = got["blk.0.ffn_down.rans_info"].tolist()
    assert info[2] == 0 and info[3] == 0
    assert np.array_equal(got["blk.0.ffn_down.rans_exp_raw"].reshape(160, 96), e)
    assert np.array_equal(oracle.merge_bf16(got["blk.0.ffn_down.rans_exp_raw"].reshape(160, 96),
                                            got["blk.0.ffn_down.rans_man_raw"].reshape(160, 96)), bits(w))


@pytest.mark.gpu
def test_gpu_compressed_module_through_a_file_and_back(tmp_path):
    """The whole way on the GPU path: modules compressed by the CUDA encoder -> GGUF file -> read_rans_gguf ->
    CUDA decoder, bit-exact, with nothing but the file's contents."""
    import comp_inference_b200 as ci
    model = _Model()
    blk = model.model.layers[0]
    wq, wd = make_weight(160, 96, 21), make_weight(96, 160, 22)          # HF layout [out, in]
    with torch.no_grad():
        blk.self_attn.q_proj.weight.copy_(wq)
        blk.mlp.down_proj.weight.copy_(wd)
    ci.rans_compress_module_weight(blk.self_attn.q_proj, tile_height=64, tile_width=32)
    ci.rans_compress_module_weight(blk.mlp.down_proj, tile_height=128, tile_width=16)
    path = str(tmp_path / "gpu.gguf")
    rans_gguf.save_rans_model_gguf(model, None, path, arch="llama")
    got = rans_gguf.read_rans_gguf(path)
    dev = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a)).view(dt).cuda()
    for base, w in (("blk.0.attn_q", wq), ("blk.0.ffn_down", wd)):
        info = got[base + ".rans_info"].tolist()
        tn, tk, th, tw = info[7:11]
        K, N = info[11:13]
        out = ci.rans_decompress_bf16(dev(got[base + ".rans_exp_stream"], torch.uint8),
                                      dev(got[base + ".rans_exp_states"].view(np.int32), torch.int32),
                                      dev(got[base + ".rans_exp_tables"].view(np.int32), torch.int32),
                                      dev(got[base + ".rans_exp_slot_map"], torch.uint8), (K, N),
                                      dev(got[base + ".rans_exp_tile_offsets"].view(np.int32), torch.int32),
                                      dev(got[base + ".rans_exp_tile_max_lens"].view(np.int32), torch.int32), th, tw,
                                      dev(got[base + ".rans_man_raw"], torch.uint8))
        assert torch.equal(out.cpu().view(torch.uint16), w.t().contiguous().view(torch.uint16))     # stored [in, out]
        # and the fused linear straight from the file's arrays
        x = torch.randn(2, K, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16).cuda()
        y = ci.fused_rans_linear_triton(x, dev(got[base + ".rans_exp_stream"], torch.uint8),
                                        dev(got[base + ".rans_exp_states"].view(np.int32), torch.int32),
                                        dev(got[base + ".rans_exp_tables"].view(np.int32), torch.int32),
                                        dev(got[base + ".rans_exp_slot_map"], torch.uint8), (K, N),
                                        dev(got[base + ".rans_exp_tile_offsets"].view(np.int32), torch.int32),
                                        dev(got[base + ".rans_exp_tile_max_lens"].view(np.int32), torch.int32), th, tw,
                                        dev(got[base + ".rans_man_raw"], torch.uint8), SPLIT_K=0)
        ref = x.float().cpu() @ w.t().float()
        assert float((y.float().cpu() - ref).abs().max() / ref.abs().max()) <= 1e-2
