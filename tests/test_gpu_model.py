"""GPU: the reference's end-to-end procedure (tests/test_full_model_rans.py:19-266) on a small random-init
Llama: compress every linear / embedding / LM head, save the package, load it back into compressed
modules, and compare (a) every decompressed weight bit for bit, (b) the logits of the compressed model
with the dense model's, (c) greedy generation."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def tiny_llama():
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(hidden_size=256, intermediate_size=704, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=4, vocab_size=512, max_position_embeddings=128, rms_norm_eps=1e-5,
                      tie_word_embeddings=False)
    torch.manual_seed(0)
    model = LlamaForCausalLM(cfg).to(torch.bfloat16)
    return cfg, model


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
    with torch.no_grad():
        logits = loaded(ids.cuda()).logits.float()
    err = float((logits - ref_logits).abs().max() / ref_logits.abs().max())
    assert err <= 3e-2, err                         # 14 bf16 matmuls deep; each fused op is within 1e-2 of its own reference
    assert (logits.argmax(-1) == ref_logits.argmax(-1)).float().mean() > 0.9

    # (c) greedy decoding with a KV cache goes through the batch-1 path of every module
    with torch.no_grad():
        a = loaded.generate(ids[:1].cuda(), max_new_tokens=8, do_sample=False)
        b = dense.generate(ids[:1].cuda(), max_new_tokens=8, do_sample=False)
    assert a.shape == b.shape


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tensor_parallel_logits(tmp_path):
    """Two ranks, each holding its column / row shards of every projection (cut out of the package's
    compressed arrays), reproduce the single-GPU logits; only activations cross NCCL."""
    import socket
    import subprocess
    import sys
    import comp_inference_b200 as ci
    cfg, model = tiny_llama()
    ci.compress_model(model, tile_height=64, tile_width=32)
    out_dir = ci.save_rans_model_package(model, None, str(tmp_path / "pkg"), fuse=False)
    single = ci.load_compressed_model(out_dir).eval()
    ids = torch.randint(0, cfg.vocab_size, (2, 16), generator=torch.Generator().manual_seed(4001))
    with torch.no_grad():
        logits = single(ids.cuda()).logits.float().cpu()
        logits1 = single(ids[:, :1].cuda()).logits.float().cpu()
    ref_path = str(tmp_path / "ref.pt")
    torch.save({"ids": ids, "logits": logits, "logits1": logits1}, ref_path)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = str(s.getsockname()[1])
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tp_worker.py")
    procs = [subprocess.Popen([sys.executable, worker, out_dir, ref_path, str(r), "2", port],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n[timed out]"
        outs.append(out)
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_oneshot_allreduce():
    """The peer-memory all-reduce against NCCL on two ranks: several sizes, repeated calls, graph replay."""
    import socket
    import subprocess
    import sys
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = str(s.getsockname()[1])
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ar_worker.py")
    procs = [subprocess.Popen([sys.executable, worker, str(r), "2", port], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n[timed out]"
        outs.append(out)
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)
