"""GPU: the one-kernel versions of the weightless decode-step stages (residual add + RMSNorm, rotary embedding
+ KV-cache write, single-query attention, SiLU * up) against the PyTorch operators they replace, and the
graph-captured decode loop with and without them."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def close(a, b, tol):
    a, b = a.float(), b.float()
    return float((a - b).abs().max()) <= tol * max(float(b.abs().max()), 1e-6)


def test_add_rmsnorm_matches_llama_rmsnorm():
    from comp_inference_b200 import ops
    from transformers.models.llama.modeling_llama import LlamaRMSNorm
    g = torch.Generator().manual_seed(0)
    for rows, cols in ((1, 4096), (8, 4096), (3, 512), (5, 11008)):
        norm = LlamaRMSNorm(cols, eps=1e-5).to(torch.bfloat16).cuda()
        with torch.no_grad():
            norm.weight.copy_(1 + 0.1 * torch.randn(cols, generator=g))
        x = torch.randn(rows, cols, generator=g).to(torch.bfloat16).cuda()
        r = torch.randn(rows, cols, generator=g).to(torch.bfloat16).cuda()
        y, h = ops.add_rmsnorm(x, r, norm.weight, 1e-5)
        assert torch.equal(h, x + r)                            # the residual stream: one bf16 rounding, as in PyTorch
        with torch.no_grad():
            want = norm(x + r)
        assert close(y, want, 2.0 ** -7)                        # at most one bf16 step apart
        assert float((y.float() - want.float()).abs().mean()) <= 1e-3 * float(want.float().abs().mean())
        y0, h0 = ops.add_rmsnorm(x, None, norm.weight, 1e-5)
        assert h0 is x
        with torch.no_grad():
            assert close(y0, norm(x), 2.0 ** -7)
    wide = torch.randn(4, 3 * 512, generator=g).to(torch.bfloat16).cuda()      # a column slice as input
    w = torch.ones(512, dtype=torch.bfloat16, device="cuda")
    ys, _ = ops.add_rmsnorm(wide[:, 512:1024], None, w, 1e-5)
    yc, _ = ops.add_rmsnorm(wide[:, 512:1024].contiguous(), None, w, 1e-5)
    assert torch.equal(ys, yc)


def rotate_ref(x, cos, sin):
    h = x.shape[-1] // 2
    rot = torch.cat((-x[..., h:], x[..., :h]), dim=-1)
    return x.float() * cos.float() + rot.float() * sin.float()


@pytest.mark.parametrize("B,n_q,n_kv,d,T,pos", [(1, 32, 32, 128, 648, 512), (8, 32, 32, 128, 648, 600), (2, 8, 2, 64, 96, 0),
                                                (3, 4, 4, 128, 64, 63)])
def test_rope_cache_write_and_attention(B, n_q, n_kv, d, T, pos):
    from comp_inference_b200 import ops
    g = torch.Generator().manual_seed(B * 100 + pos)
    qkv = torch.randn(B, (n_q + 2 * n_kv) * d, generator=g).to(torch.bfloat16).cuda()      # one fused projection output
    q, k, v = qkv[:, :n_q * d], qkv[:, n_q * d:(n_q + n_kv) * d], qkv[:, (n_q + n_kv) * d:]
    inv = 1.0 / (10000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    ang = torch.outer(torch.arange(T, dtype=torch.float32), inv)
    emb = torch.cat((ang, ang), -1)
    cos, sin = emb.cos().to(torch.bfloat16).cuda(), emb.sin().to(torch.bfloat16).cuda()
    k_cache = torch.randn(B, n_kv, T, d, generator=g).to(torch.bfloat16).cuda()
    v_cache = torch.randn(B, n_kv, T, d, generator=g).to(torch.bfloat16).cuda()
    k_before, v_before = k_cache.clone(), v_cache.clone()
    p = torch.tensor([pos], dtype=torch.int64, device="cuda")
    q_rot = ops.rope_kv(q, k, v, cos, sin, p, k_cache, v_cache, d)
    want_q = rotate_ref(q.view(B, n_q, d), cos[pos], sin[pos])
    want_k = rotate_ref(k.view(B, n_kv, d), cos[pos], sin[pos])
    assert close(q_rot, want_q, 2.0 ** -7) and close(k_cache[:, :, pos], want_k, 2.0 ** -7)
    assert torch.equal(v_cache[:, :, pos], v.view(B, n_kv, d))
    keep = torch.ones(T, dtype=torch.bool, device="cuda")
    keep[pos] = False
    assert torch.equal(k_cache[:, :, keep], k_before[:, :, keep]) and torch.equal(v_cache[:, :, keep], v_before[:, :, keep])
    out = ops.decode_attention(q_rot, k_cache, v_cache, p)
    rep = n_q // n_kv
    kk = k_cache[:, :, :pos + 1].repeat_interleave(rep, dim=1).float()
    vv = v_cache[:, :, :pos + 1].repeat_interleave(rep, dim=1).float()
    want = F.scaled_dot_product_attention(q_rot.float().unsqueeze(2), kk, vv).squeeze(2).reshape(B, n_q * d)
    assert out.shape == (B, n_q * d) and close(out, want, 1e-2)


def test_silu_mul_on_slices():
    from comp_inference_b200 import ops
    g = torch.Generator().manual_seed(3)
    gu = torch.randn(5, 2 * 11008, generator=g).to(torch.bfloat16).cuda()
    gate, up = gu[:, :11008], gu[:, 11008:]
    got = ops.silu_mul(gate, up)
    want = F.silu(gate) * up
    assert got.shape == want.shape and close(got, want, 2.0 ** -7)
    assert float((got.float() - want.float()).abs().mean()) <= 1e-3 * float(want.float().abs().mean())


def test_decode_loop_with_and_without_the_fused_stages():
    """The same dense model, the same graph-captured loop: the one-kernel stages change the logits by no more than
    bf16 rounding, and every generated token is a best or near-best token of the PyTorch-operator run."""
    from comp_inference_b200.generation import LlamaGreedyRunner
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(hidden_size=256, intermediate_size=704, num_hidden_layers=3, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=512, max_position_embeddings=128, rms_norm_eps=1e-5,
                      tie_word_embeddings=False)
    torch.manual_seed(0)
    model = LlamaForCausalLM(cfg).to(torch.bfloat16).cuda().eval()
    ids = torch.randint(0, 512, (2, 20), generator=torch.Generator().manual_seed(5)).cuda()
    plain = LlamaGreedyRunner(model, 2, 64, fused_glue=False)
    fused = LlamaGreedyRunner(model, 2, 64, fused_glue=True)
    t_plain, _, _ = plain.generate(ids, 8)
    t_fused, _, _ = fused.generate(ids, 8)
    assert t_fused.shape == (2, 8) and torch.equal(t_fused[:, 0], t_plain[:, 0])      # the first token comes from the prompt pass
    # teacher-force the plain runner on the fused runner's tokens: every choice is (near-)best there
    seq = torch.cat([ids, t_fused], dim=1)
    with torch.no_grad():
        logits = model(seq[:, :-1]).logits.float()[:, 19:]
    chosen = logits.gather(2, t_fused.unsqueeze(-1)).squeeze(-1)
    assert bool((chosen >= logits.max(-1).values - 3e-2 * logits.abs().max(-1).values).all())
    # one decode step from identical state: logits agree to bf16 rounding
    plain.prefill(ids)
    fused.prefill(ids)
    plain._decode_step(2)
    fused._decode_step(2)
    torch.cuda.synchronize()
    assert close(fused.logits, plain.logits, 3e-2)
