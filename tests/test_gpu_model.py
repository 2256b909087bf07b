"""GPU: the reference's end-to-end procedure (tests/test_full_model_rans.py:19-266) on a small random-init
Llama: compress every linear / embedding / LM head (separately, and with q|k|v and gate|up concatenated),
save the package, load it back into compressed modules, and compare (a) every decompressed weight bit for
bit, (b) the logits of the compressed model with the dense model's, (c) greedy generation; then the same
model on 2 / 4 / 8 tensor-parallel ranks (as many as the box has GPUs)."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def tiny_llama(hidden=256, inter=704, heads=4, vocab=512, layers=2):
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(hidden_size=hidden, intermediate_size=inter, num_hidden_layers=layers,
                      num_attention_heads=heads, num_key_value_heads=heads, vocab_size=vocab,
                      max_position_embeddings=128, rms_norm_eps=1e-5, tie_word_embeddings=False)
    torch.manual_seed(0)
    model = LlamaForCausalLM(cfg).to(torch.bfloat16)
    return cfg, model


def assert_greedy_equivalent(dense, tokens, prompt_len, tol_rel=3e-2):
    """Greedy tokens of a model whose weights equal the dense model's bit for bit may still differ from the dense
    model's own greedy tokens where two candidates are closer than the rounding of the fused kernels.  What
    must hold: at every generated position the chosen token is the dense model's best candidate, or within
    ``tol_rel`` of the largest |logit| of it (the dense model is teacher-forced on the generated sequence).
    Returns the fraction of positions where the choice is exactly the dense argmax."""
    with torch.no_grad():
        logits = dense(tokens[:, :-1]).logits.float()
    exact = 0
    n = tokens.shape[1] - prompt_len
    for t in range(prompt_len, tokens.shape[1]):
        row = logits[:, t - 1]
        chosen = row.gather(1, tokens[:, t:t + 1]).squeeze(1)
        slack = tol_rel * row.abs().max(dim=1).values
        assert bool((chosen >= row.max(dim=1).values - slack).all()), f"position {t}: not a near-best token"
        exact += int((row.argmax(-1) == tokens[:, t]).all())
    return exact / n


def test_package_round_trip_and_logits(tmp_path):
    import comp_inference_b200 as ci
    cfg, dense = tiny_llama()
    dense_state = {k: v.clone() for k, v in dense.state_dict().items()}
    ids = torch.randint(0, cfg.vocab_size, (2, 24), generator=torch.Generator().manual_seed(4001))
    dense = dense.cuda().eval()
    with torch.no_grad():
        ref_logits = dense(ids.cuda()).logits.float()

    cfg2, model = tiny_llama()                      # same seed -> same weights
    ci.compress_model(model, tile_height=128, tile_width=32, layer_tiles={"model.layers.1.mlp.down_proj": (64, 32)})
    n_compressed = sum(getattr(m, "compressed", None) == "rans_bfloat16" for m in model.modules())
    assert n_compressed == 2 * 7 + 2                # 7 linears per layer + embedding + LM head
    out_dir = ci.save_rans_model_package(model, None, str(tmp_path / "pkg"), fuse=False)
    assert os.path.exists(os.path.join(out_dir, "model.safetensors"))

    # (a) decompress in place and compare with the dense weights
    for name, module in model.named_modules():
        if getattr(module, "compressed", None) == "rans_bfloat16":
            ci.rans_decompress_module_weight(module)
            want = dense_state[name + ".weight"]
            got = module.weight.detach()
            if not (name.endswith("lm_head") or name.endswith("embed_tokens")):
                got = got.t()                       # linears are stored transposed: [in, out]
            assert torch.equal(got.contiguous().view(torch.uint16), want.contiguous().view(torch.uint16)), name

    # (b) load the package into compressed modules and run it
    loaded = ci.load_compressed_model(out_dir).eval()
    kinds = {type(m).__name__ for m in loaded.modules()}
    assert {"RansLinear", "RansEmbedding", "RansLMHead"} <= kinds
    assert loaded.model.layers[1].mlp.down_proj.tile_k == 64
    assert loaded.lm_head._twin is not None         # the head's transposed twin is built at load, not in a forward
    with torch.no_grad():
        logits = loaded(ids.cuda()).logits.float()
    err = float((logits - ref_logits).abs().max() / ref_logits.abs().max())
    assert err <= 3e-2, err                         # 14 bf16 matmuls deep; each fused op is within 1e-2 of its own reference
    assert (logits.argmax(-1) == ref_logits.argmax(-1)).float().mean() > 0.9

    # (c) greedy decoding with a KV cache goes through the batch-1 path of every module
    with torch.no_grad():
        a = loaded.generate(ids[:1].cuda(), max_new_tokens=8, do_sample=False)
    assert a.shape == (1, 24 + 8) and torch.equal(a[:, :24].cpu(), ids[:1])
    assert_greedy_equivalent(dense, a, 24)
    ci.check_status()


def test_fused_projection_package(tmp_path):
    """q|k|v and gate|up concatenated before compression (rans_compress_qkv_fused / rans_compress_gate_up_fused,
    comp_inference/comp_inference.py:242-341), saved with fuse=True, loaded into RansFusedLinear + slices:
    one launch per family, results equal to the three (two) separate projections."""
    import comp_inference_b200 as ci
    cfg, dense = tiny_llama()
    ids = torch.randint(0, cfg.vocab_size, (2, 24), generator=torch.Generator().manual_seed(4002))
    dense = dense.cuda().eval()
    with torch.no_grad():
        ref_logits = dense(ids.cuda()).logits.float()
    _, model = tiny_llama()
    ci.compress_model(model, tile_height=128, tile_width=32, fuse=True)
    attn, mlp = model.model.layers[0].self_attn, model.model.layers[0].mlp
    assert attn.qkv_fused and not hasattr(attn, "k_proj") and not hasattr(attn, "v_proj")
    assert mlp.gate_up_fused and not hasattr(mlp, "up_proj")
    assert attn.q_proj.input_shape == [256, 3 * 256] and mlp.gate_proj.input_shape == [256, 2 * 704]
    n_compressed = sum(getattr(m, "compressed", None) == "rans_bfloat16" for m in model.modules())
    assert n_compressed == 2 * 4 + 2                # qkv, o, gate|up, down per layer + embedding + LM head
    out_dir = ci.save_rans_model_package(model, None, str(tmp_path / "pkg"), fuse=True)
    import json
    cfg_json = json.load(open(os.path.join(out_dir, "config.json")))
    names = set(cfg_json["quantization_config"]["layer_configs"])
    assert "model.layers.0.self_attn.qkv_proj" in names and "model.layers.1.mlp.gate_up_proj" in names
    loaded = ci.load_compressed_model(out_dir).eval()
    la = loaded.model.layers[0].self_attn
    assert type(la.q_proj).__name__ == "RansFusedLinear" and la.q_proj.parts == [256, 256, 256]
    assert type(la.k_proj).__name__ == "RansFusedSlice" and (la.v_proj.start, la.v_proj.end) == (512, 768)
    assert loaded.model.layers[1].mlp.gate_proj.parts == [704, 704]
    assert "model.layers.0.self_attn.k_proj.rans_exp_stream" not in loaded.state_dict()
    with torch.no_grad():
        logits = loaded(ids.cuda()).logits.float()
    err = float((logits - ref_logits).abs().max() / ref_logits.abs().max())
    assert err <= 3e-2, err
    # block by block against the dense projections
    x = torch.randn(3, 256, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).cuda()
    da = dense.model.layers[0].self_attn
    for mine, theirs in ((la.q_proj, da.q_proj), (la.k_proj, da.k_proj), (la.v_proj, da.v_proj)):
        ref = theirs(x).float()
        assert float((mine(x).float() - ref).abs().max() / ref.abs().max()) <= 1e-2
    with torch.no_grad():
        a = loaded.generate(ids[:1].cuda(), max_new_tokens=6, do_sample=False)
    assert_greedy_equivalent(dense, a, 24)
    # the graph-captured decode loop of this package against Hugging Face's own generate on the same modules
    from comp_inference_b200.generation import LlamaGreedyRunner
    runner = LlamaGreedyRunner(loaded, 2, 64)
    toks, first, t = runner.generate(ids.cuda(), 6)
    with torch.no_grad():
        b = loaded.generate(ids.cuda(), max_new_tokens=6, do_sample=False)
    full = torch.cat([ids.cuda(), toks], dim=1)
    assert_greedy_equivalent(dense, full, 24)
    assert (toks == b[:, 24:]).float().mean() >= 0.5, (toks, b[:, 24:])
    ci.check_status()


def test_corrupted_package_is_refused(tmp_path):
    """A package whose tile metadata was damaged is rejected at load (CI_E_INVALID, naming the module and the
    tile) instead of being handed to kernels that trust their metadata."""
    import comp_inference_b200 as ci
    from safetensors.torch import load_file, save_file
    _, model = tiny_llama(layers=1)
    ci.compress_model(model, tile_height=64, tile_width=32)
    out_dir = ci.save_rans_model_package(model, None, str(tmp_path / "pkg"), fuse=False)
    path = os.path.join(out_dir, "model.safetensors")
    state = load_file(path)
    key = "model.layers.0.mlp.down_proj.rans_exp_tile_max_lens"
    bad = state[key].clone().view(torch.int32)
    bad[3] = 60000                                              # a byte block that would run far past the stream
    state[key] = bad.view(torch.uint32)
    save_file(state, path, metadata={"format": "pt"})
    with pytest.raises(RuntimeError, match="down_proj.*tile 3"):
        ci.load_compressed_model(out_dir)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return str(s.getsockname()[1])


def _run_workers(script, world, extra_args, timeout=420):
    """One child process per rank.  The workers bound every wait themselves (kernel polls of about a second,
    a short process-group timeout) and always leave on their own; nothing here kills a rank that may still
    hold peer-mapped memory."""
    port = _free_port()
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, script), *extra_args, str(r), str(world), port],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = [p.communicate(timeout=timeout)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)
    return outs


def _worlds():
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    return [w for w in (2, 4, 8) if w <= n] or [2]


@pytest.mark.parametrize("kind,K,N,parts,th", [("col", 256, 768, [256, 256, 256], 128), ("row", 1024, 256, None, 128),
                                                ("row", 2752, 128, None, 128), ("col", 256, 512, None, 64)])
def test_shards_cut_and_retiled_at_load(kind, K, N, parts, th):
    """One rank's shard as the tensor-parallel loader makes it -- cut out of the compressed arrays, or decoded and
    re-encoded where the cut misses the tile grid -- with and without a new tile height: always the rank's slice
    of the dense weight, bit for bit."""
    import comp_inference_b200 as ci
    from comp_inference_b200 import pytorch_runtime as rt
    world = 4
    g = torch.Generator().manual_seed(K + N)
    W = (torch.randn(K, N, generator=g) * 0.02).to(torch.bfloat16).cuda()
    c = ci.compress_weight_cuda(W, th, 32)
    for rank in (0, world - 1):
        if kind == "col":
            cols, start = [], 0
            for p in (parts or [N]):
                cols.append(W[:, start + rank * (p // world):start + (rank + 1) * (p // world)])
                start += p
            want = torch.cat(cols, dim=1).contiguous()
        else:
            want = W[rank * (K // world):(rank + 1) * (K // world)].contiguous()
        for retile in (None, 32, 64):
            s = rt._shard(c, kind, rank, world, torch.device("cuda", 0), parts, retile=retile)
            assert s["tile_height"] == (retile or th) and tuple(s["shape"]) == tuple(want.shape)
            back = ci.rans_decompress_bf16(s["rans_exp_stream"].cuda(), s["rans_exp_states"].cuda(),
                                           s["rans_exp_tables"].cuda(), s["rans_exp_slot_map"].cuda(), s["shape"],
                                           s["rans_exp_tile_offsets"].cuda(), s["rans_exp_tile_max_lens"].cuda(),
                                           s["tile_height"], s["tile_width"], s["rans_man_raw"].cuda())
            assert torch.equal(back.view(torch.uint16), want.view(torch.uint16)), (kind, rank, retile)


@pytest.mark.parametrize("world", _worlds())
@pytest.mark.parametrize("fuse", [False, True])
def test_tensor_parallel_logits(tmp_path, world, fuse):
    """Every rank holds its column / row shards of every projection (cut out of the package's compressed arrays)
    and a slice of the LM head's vocabulary; together they reproduce the single-GPU logits; only activations
    cross the links."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import comp_inference_b200 as ci
    # 8 heads of 64, FFN 1024, vocabulary 1024: every cut of 2, 4 and 8 ranks falls on 32-column / 64-row tiles
    cfg, model = tiny_llama(hidden=512, inter=1024, heads=8, vocab=1024)
    ci.compress_model(model, tile_height=64, tile_width=32, fuse=fuse)
    out_dir = ci.save_rans_model_package(model, None, str(tmp_path / "pkg"), fuse=fuse)
    single = ci.load_compressed_model(out_dir).eval()
    ids = torch.randint(0, cfg.vocab_size, (2, 16), generator=torch.Generator().manual_seed(4001))
    with torch.no_grad():
        logits = single(ids.cuda()).logits.float().cpu()
        logits1 = single(ids[:, :1].cuda()).logits.float().cpu()
    ref_path = str(tmp_path / "ref.pt")
    torch.save({"ids": ids, "logits": logits, "logits1": logits1}, ref_path)
    del single
    torch.cuda.empty_cache()
    _run_workers("tp_worker.py", world, [out_dir, ref_path])


@pytest.mark.parametrize("world", _worlds())
def test_oneshot_allreduce(world):
    """The peer-memory all-reduce and all-gather against NCCL: several sizes, repeated calls, graph replay; the
    exchange fused into the row-parallel GEMV against the unsharded product, held to the same 1e-2 as every
    other fused linear."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _run_workers("ar_worker.py", world, [])
