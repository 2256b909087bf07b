"""CPU: host-side logic around the kernels -- metadata validation, fused-projection packages, the shard
slicer for concatenated projections and vocabulary slices, the greedy-generation runner -- with the CPU
oracle standing in for the codec.  No kernel is launched."""
import numpy as np
import pytest
import torch
import torch.nn as nn

from conftest import bits, make_weight


def oracle_dict(oracle, W, th, tw):
    o = oracle.compress_bf16(bits(W), th, tw)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    K, N = W.shape
    return dict(rans_exp_stream=t(o.stream), rans_exp_states=t(o.states), rans_exp_tables=t(o.tables),
                rans_exp_slot_map=t(o.slot_map), rans_exp_tile_offsets=t(o.tile_offsets),
                rans_exp_tile_max_lens=t(o.tile_max_lens), rans_man_raw=t(o["mantissa"]), shape=(K, N),
                tile_height=o.tile_height, tile_width=o.tile_width)


def as_oracle(c):
    n = lambda k: c[k].numpy()
    return dict(stream=n("rans_exp_stream"), states=n("rans_exp_states"), tables=n("rans_exp_tables"),
                slot_map=n("rans_exp_slot_map"), tile_offsets=n("rans_exp_tile_offsets"),
                tile_max_lens=n("rans_exp_tile_max_lens"))


def test_validate_accepts_good_and_names_bad_metadata(oracle):
    from comp_inference_b200 import _lib
    W = make_weight(192, 96, seed=5)
    c = oracle_dict(oracle, W, 64, 32)
    _lib.validate_compressed(c)
    _lib.validate_compressed(c, max_tile_len=int(c["rans_exp_tile_max_lens"].view(torch.int32).max()))

    def corrupt(key, fn):
        d = dict(c)
        t = d[key].clone()
        fn(t.view(torch.int32) if t.dtype == torch.uint32 else t)
        d[key] = t
        return d

    cases = [
        (corrupt("rans_exp_tile_max_lens", lambda t: t.__setitem__(2, 65)), "tile 2.*exceeds"),          # > tile_h rows
        (corrupt("rans_exp_tile_offsets", lambda t: t.__setitem__(4, 0)), "tile 4.*overlaps"),
        (corrupt("rans_exp_tile_offsets", lambda t: t.__setitem__(8, 10 ** 8)), "tile 8.*run past"),
        (corrupt("rans_exp_tables", lambda t: t.__setitem__(7, int(t[7]) + (1 << 16))), "tables\\[7\\]: cumulative"),
        (corrupt("rans_exp_slot_map", lambda t: t.__setitem__(100, int(t[100]) ^ 1)), "slot_map\\[100\\]"),
        (dict(c, rans_exp_states=c["rans_exp_states"][:-1]), "initial states"),
        (dict(c, rans_man_raw=c["rans_man_raw"][:-1]), "mantissa"),
        (dict(c, rans_exp_stream=c["rans_exp_stream"][:-1]), "run past"),
    ]
    for bad, pattern in cases:
        with pytest.raises(RuntimeError, match=pattern):
            _lib.validate_compressed(bad)
    with pytest.raises(RuntimeError, match="above the declared maximum"):
        _lib.validate_compressed(c, max_tile_len=1)
    with pytest.raises(RuntimeError, match="entries"):
        _lib.validate_compressed(dict(c, rans_exp_tile_offsets=c["rans_exp_tile_offsets"][:-1]))


def test_status_word_address_is_plain_arithmetic():
    from comp_inference_b200 import _lib
    lib = _lib.load()
    assert lib.ci_workspace_status_word(0) is None
    assert lib.ci_workspace_status_word(1 << 20) == (1 << 20) + 4095 * 4
    assert lib.ci_status(None, None, 0, None) == -1 and b"null status word" in lib.ci_last_error()


@pytest.mark.parametrize("world", [2, 4])
def test_concatenated_projection_shards(oracle, world):
    """A rank's column shard of q|k|v is [q_r | k_r | v_r]: its slice of every block, not a slice of the whole."""
    from comp_inference_b200 import sharding
    parts = [128, 64, 64] if world == 2 else [256, 128, 128]
    K, N, th, tw = 128, sum(parts), 64, 32
    W = make_weight(K, N, seed=9)
    c = oracle_dict(oracle, W, th, tw)
    raw = bits(W)
    assert sharding.can_shard_cols(N, tw, world, parts)
    assert not sharding.can_shard_cols(96, 32, 2, [48, 48])
    for r in range(world):
        s = sharding.shard_cols(c, r, world, parts)
        k, n = s["shape"]
        assert n == N // world
        got = oracle.decode_bf16(as_oracle(s), s["rans_man_raw"].numpy(), k, n, th, tw)
        want, start = [], 0
        for p in parts:
            want.append(raw[:, start + r * (p // world):start + (r + 1) * (p // world)])
            start += p
        assert np.array_equal(got, np.concatenate(want, axis=1))


def test_tile_row_range_for_vocabulary_slices(oracle):
    """tile_rows cuts the tile rows that cover an arbitrary row range (a vocabulary slice that does not start on
    a tile row), including the partial last tile row."""
    from comp_inference_b200 import sharding
    K, N, th, tw = 300, 64, 64, 32                              # 5 tile rows, the last with 44 rows
    W = make_weight(K, N, seed=3)
    c = oracle_dict(oracle, W, th, tw)
    raw = bits(W)
    for k0, k1 in ((0, 2), (1, 4), (3, 5), (4, 5)):
        s = sharding.tile_rows(c, k0, k1)
        rows = min(k1 * th, K) - k0 * th
        assert s["shape"] == (rows, N)
        got = oracle.decode_bf16(as_oracle(s), s["rans_man_raw"].numpy(), rows, N, th, tw)
        assert np.array_equal(got, raw[k0 * th:k0 * th + rows])
    with pytest.raises(ValueError):
        sharding.tile_rows(c, 2, 6)


def _tiny():
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(hidden_size=128, intermediate_size=352, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=300, max_position_embeddings=128, rms_norm_eps=1e-5,
                      tie_word_embeddings=False)
    torch.manual_seed(0)
    return cfg, LlamaForCausalLM(cfg).eval()


def test_patch_model_builds_fused_modules_from_a_fused_package(oracle):
    """A package that stores q|k|v under q_proj and gate|up under gate_proj (rans_saving.py:52-60) loads as one
    RansFusedLinear per family plus slice modules; an unfused one as plain RansLinear."""
    import comp_inference_b200 as ci
    cfg, model = _tiny()
    model = model.to(torch.bfloat16)
    sd = {}

    def add(name, w_kn):
        c = oracle_dict(oracle, w_kn.contiguous(), 64, 32)
        for k, v in c.items():
            if torch.is_tensor(v):
                sd[f"{name}.{k}"] = v
        K, N = w_kn.shape
        sd[f"{name}.rans_info"] = torch.tensor([1, K * N, 1, 0, 0, 0, 2, -(-N // 32), -(-K // 64), 64, 32, K, N],
                                               dtype=torch.int32)

    for i, layer in enumerate(model.model.layers):
        a, m = layer.self_attn, layer.mlp
        add(f"model.layers.{i}.self_attn.q_proj", torch.cat([a.q_proj.weight, a.k_proj.weight, a.v_proj.weight]).t())
        add(f"model.layers.{i}.mlp.gate_proj", torch.cat([m.gate_proj.weight, m.up_proj.weight]).t())
        add(f"model.layers.{i}.self_attn.o_proj", a.o_proj.weight.t())
    ci.patch_model(model, sd, default_th=64, default_tw=32)
    a, m = model.model.layers[1].self_attn, model.model.layers[1].mlp
    assert isinstance(a.q_proj, ci.RansFusedLinear) and a.q_proj.parts == [128, 64, 64]       # 4 heads, 2 KV heads of 32
    assert isinstance(a.k_proj, ci.RansFusedSlice) and (a.k_proj.start, a.k_proj.end) == (128, 192)
    assert (a.v_proj.start, a.v_proj.end) == (192, 256) and a.v_proj.out_features == 64
    assert isinstance(m.gate_proj, ci.RansFusedLinear) and m.gate_proj.parts == [352, 352]
    assert isinstance(m.up_proj, ci.RansFusedSlice) and isinstance(m.down_proj, nn.Linear)
    assert type(a.o_proj) is ci.RansLinear and a.o_proj.rans_exp_stream.numel() > 0
    assert a.q_proj.rans_exp_states.numel() == 2 * 8 * 64      # 2 x 8 tiles of 64 streams
    names = set(model.state_dict())
    assert "model.layers.1.self_attn.q_proj.rans_exp_stream" in names
    assert not any(".k_proj." in n or ".up_proj." in n for n in names)
    # a damaged package is refused before anything is assigned
    bad = dict(sd)
    t = bad["model.layers.0.self_attn.o_proj.rans_exp_tile_offsets"].clone()
    t.view(torch.int32)[1] = 10 ** 7
    bad["model.layers.0.self_attn.o_proj.rans_exp_tile_offsets"] = t
    _, fresh = _tiny()
    with pytest.raises(RuntimeError, match="layers.0.self_attn.o_proj.*tile 1"):
        ci.patch_model(fresh.to(torch.bfloat16), bad, default_th=64, default_tw=32)


def test_greedy_runner_matches_hugging_face_generate():
    """The decode loop used for whole-model measurements (static KV cache, own rotary embedding and attention)
    produces the tokens Hugging Face's generate produces; grouped-query attention included."""
    from comp_inference_b200.generation import LlamaGreedyRunner
    cfg, model = _tiny()
    ids = torch.randint(0, cfg.vocab_size, (2, 12), generator=torch.Generator().manual_seed(1))
    runner = LlamaGreedyRunner(model, 2, 64)
    runner.cos, runner.sin = runner.cos.float(), runner.sin.float()
    runner.k_cache, runner.v_cache = runner.k_cache.float(), runner.v_cache.float()
    toks, first, timing = runner.generate(ids, 10, use_graph=False)
    with torch.no_grad():
        ref = model.generate(ids, max_new_tokens=10, do_sample=False, pad_token_id=0)
        ref_first = model(ids).logits[:, -1]
    assert torch.equal(toks, ref[:, 12:])
    assert float((first - ref_first).abs().max()) < 1e-3
    assert timing["decode_tok_s"] > 0
    all_logits = runner.prefill(ids, all_logits=True)
    assert all_logits.shape == (2, 12, cfg.vocab_size)
