"""Greedy generation for Llama-architecture models whose projections, embedding table and LM head were
swapped for the compressed modules of this package (pytorch_runtime.patch_model /
patch_model_tensor_parallel): the caller on the other side of the fused decode-linear kernels.

The reference measures whole-model speed with Hugging Face's ``generate`` (greedy, KV cache, wall clock,
tests/test_rans_pytorch_runtime.py:89-118); every token there pays the host cost of a few thousand eager
kernel launches.  Here the prompt is processed once (eager), and one decode step -- embedding gather, all
layers, LM head, argmax, KV-cache update -- is captured in a CUDA graph with static buffers and replayed
per token, so that the measured time is the kernels' and, in a tensor-parallel group, the exchanges'.

The runner uses the model's own modules for everything that has weights (norms, projections, embedding,
head) and does the weightless part itself (rotary embedding, scaled-dot-product attention over a static
cache).  It therefore runs dense ``nn.Linear`` models too, which is how the dense baseline next to the
compressed model is produced with identical attention arithmetic.  Head counts are taken from the widths of
the projections it finds, so a rank of a tensor-parallel group simply sees fewer heads.
"""
import time

import torch
import torch.nn.functional as F


class LlamaGreedyRunner:
    """``fused_glue`` (default: on a CUDA device): the decode step runs residual add + RMSNorm, rotary
    embedding + cache write, single-query attention and SiLU * up as one kernel each (ops.add_rmsnorm, rope_kv,
    decode_attention, silu_mul) instead of some thirty element-wise PyTorch launches per layer; the prompt pass
    keeps the PyTorch operators."""

    def __init__(self, model, max_batch: int, max_len: int, fused_glue=None):
        cfg = model.config
        self.model, self.cfg = model, cfg
        self.layers = list(model.model.layers)
        self.head_dim = getattr(cfg, "head_dim", None) or cfg.hidden_size // cfg.num_attention_heads
        self.device = next(model.model.norm.parameters()).device
        attn = self.layers[0].self_attn
        self.n_q = attn.q_proj.out_features // self.head_dim if not hasattr(attn.q_proj, "parts") \
            else attn.q_proj.parts[0] // self.head_dim
        self.n_kv = attn.k_proj.out_features // self.head_dim
        self.B, self.T = int(max_batch), int(max_len)
        theta = float(getattr(cfg, "rope_theta", None) or (getattr(cfg, "rope_parameters", None) or {}).get(
            "rope_theta", 10000.0))
        inv = 1.0 / (theta ** (torch.arange(0, self.head_dim, 2, dtype=torch.float32, device=self.device) / self.head_dim))
        ang = torch.outer(torch.arange(self.T, dtype=torch.float32, device=self.device), inv)
        emb = torch.cat((ang, ang), dim=-1)
        self.cos, self.sin = emb.cos().to(torch.bfloat16), emb.sin().to(torch.bfloat16)      # [T, hd]
        L = len(self.layers)
        self.k_cache = torch.zeros(L, self.B, self.n_kv, self.T, self.head_dim, dtype=torch.bfloat16, device=self.device)
        self.v_cache = torch.zeros_like(self.k_cache)
        # static state of the captured decode step
        self.tok = torch.zeros(self.B, dtype=torch.int64, device=self.device)
        self.pos = torch.zeros(1, dtype=torch.int64, device=self.device)
        self.out = torch.zeros(self.B, self.T, dtype=torch.int64, device=self.device)
        self.steps_done = torch.zeros(1, dtype=torch.int64, device=self.device)
        self.logits = None
        self._graph = None
        self._graph_batch = None
        self.fused_glue = (self.device.type == "cuda") if fused_glue is None else bool(fused_glue)

    # ------------------------------------------------------------------ pieces
    @staticmethod
    def _rotate(x, cos, sin):
        h = x.shape[-1] // 2
        rot = torch.cat((-x[..., h:], x[..., :h]), dim=-1)
        return x * cos + rot * sin

    def _layer(self, i, layer, h, cos, sin, attend):
        """One decoder layer; ``attend(i, q, k, v)`` writes k/v into the cache and returns the attention output."""
        B, S, _ = h.shape
        x = layer.input_layernorm(h)
        a = layer.self_attn
        q = a.q_proj(x).view(B, S, self.n_q, self.head_dim).transpose(1, 2)
        k = a.k_proj(x).view(B, S, self.n_kv, self.head_dim).transpose(1, 2)
        v = a.v_proj(x).view(B, S, self.n_kv, self.head_dim).transpose(1, 2)
        q, k = self._rotate(q, cos, sin), self._rotate(k, cos, sin)
        o = attend(i, q, k, v).transpose(1, 2).reshape(B, S, self.n_q * self.head_dim)
        h = h + a.o_proj(o)
        x = layer.post_attention_layernorm(h)
        m = layer.mlp
        return h + m.down_proj(F.silu(m.gate_proj(x)) * m.up_proj(x))

    def _expand_kv(self, t):
        rep = self.n_q // self.n_kv
        return t if rep == 1 else t.repeat_interleave(rep, dim=1)

    # ------------------------------------------------------------------ prompt
    @torch.no_grad()
    def prefill(self, ids, all_logits=False):
        """Processes the prompt ids [B, S] (eager), fills the cache, returns the logits of the last position
        [B, V] (of every position [B, S, V] with ``all_logits``) and arms the decode step with the argmax."""
        B, S = ids.shape
        assert B <= self.B and S < self.T
        cos, sin = self.cos[:S][None, None], self.sin[:S][None, None]

        def attend(i, q, k, v):
            self.k_cache[i, :B, :, :S] = k
            self.v_cache[i, :B, :, :S] = v
            return F.scaled_dot_product_attention(q, self._expand_kv(k), self._expand_kv(v), is_causal=True)

        h = self.model.model.embed_tokens(ids)
        for i, layer in enumerate(self.layers):
            h = self._layer(i, layer, h, cos, sin, attend)
        h = self.model.model.norm(h if all_logits else h[:, -1:])
        logits = self.model.lm_head(h)
        last = logits[:, -1]
        self.tok[:B] = last.argmax(-1)
        self.pos.fill_(S)
        self.steps_done.zero_()
        self.out[:B, 0] = self.tok[:B]
        return logits if all_logits else last

    # ------------------------------------------------------------------ one token
    def _decode_step_fused(self, B):
        """The decode step with one kernel per weightless stage (see the class docstring)."""
        from . import ops
        pos, m, hd = self.pos, self.model.model, self.head_dim
        h = m.embed_tokens(self.tok[:B].view(B, 1)).view(B, -1)
        delta = None
        for i, layer in enumerate(self.layers):
            ln = layer.input_layernorm
            x, h = ops.add_rmsnorm(h if delta is None else delta, None if delta is None else h, ln.weight,
                                   ln.variance_epsilon)
            a = layer.self_attn
            q, k, v = a.q_proj(x), a.k_proj(x), a.v_proj(x)
            q = ops.rope_kv(q, k, v, self.cos, self.sin, pos, self.k_cache[i, :B], self.v_cache[i, :B], hd)
            o = ops.decode_attention(q, self.k_cache[i, :B], self.v_cache[i, :B], pos)
            delta = a.o_proj(o)
            ln = layer.post_attention_layernorm
            x, h = ops.add_rmsnorm(delta, h, ln.weight, ln.variance_epsilon)
            mlp = layer.mlp
            delta = mlp.down_proj(ops.silu_mul(mlp.gate_proj(x), mlp.up_proj(x)))
        x, h = ops.add_rmsnorm(delta, h, m.norm.weight, m.norm.variance_epsilon)
        self.logits = self.model.lm_head(x)
        self.tok[:B] = self.logits.argmax(-1)
        self.pos.add_(1)
        self.steps_done.add_(1)
        self.out[:B].index_copy_(1, self.steps_done, self.tok[:B].view(B, 1))

    def _decode_step(self, B):
        """Consumes self.tok (the token at position self.pos), produces the next one.  All shapes static."""
        if self.fused_glue:
            return self._decode_step_fused(B)
        pos = self.pos
        cos, sin = self.cos.index_select(0, pos)[None, None], self.sin.index_select(0, pos)[None, None]
        mask = (torch.arange(self.T, device=self.device) <= pos)[None, None, None, :]

        def attend(i, q, k, v):
            self.k_cache[i, :B].index_copy_(2, pos, k)
            self.v_cache[i, :B].index_copy_(2, pos, v)
            return F.scaled_dot_product_attention(q, self._expand_kv(self.k_cache[i, :B]),
                                                  self._expand_kv(self.v_cache[i, :B]), attn_mask=mask)

        h = self.model.model.embed_tokens(self.tok[:B].view(B, 1))
        for i, layer in enumerate(self.layers):
            h = self._layer(i, layer, h, cos, sin, attend)
        self.logits = self.model.lm_head(self.model.model.norm(h))[:, -1]
        self.tok[:B] = self.logits.argmax(-1)
        self.pos.add_(1)
        self.steps_done.add_(1)
        self.out[:B].index_copy_(1, self.steps_done, self.tok[:B].view(B, 1))

    @torch.no_grad()
    def capture(self, B):
        """Captures the decode step for batch B (after a prefill, so that every lazily built piece exists).
        The cache, position and token buffers are restored afterwards: warm-up and capture leave no trace."""
        saved = (self.tok.clone(), self.pos.clone(), self.steps_done.clone(), self.out.clone())
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            self._decode_step(B)                               # eager once on the capture stream: workspaces, tables
            torch.cuda.synchronize(self.device)
            self.pos.copy_(saved[1])
            self.steps_done.copy_(saved[2])
            self.tok.copy_(saved[0])
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                self._decode_step(B)
        torch.cuda.synchronize(self.device)
        self.tok.copy_(saved[0])
        self.pos.copy_(saved[1])
        self.steps_done.copy_(saved[2])
        self.out.copy_(saved[3])
        self._graph, self._graph_batch = graph, B
        return graph

    @torch.no_grad()
    def generate(self, ids, max_new_tokens: int, use_graph=True, barrier=None):
        """Greedy tokens [B, max_new_tokens] for the prompt ids [B, S]; returns (tokens, last-position prompt
        logits, timing dict).  Wall-clock times, the reference's definition: ``prefill_s`` prompt to first
        token, ``decode_s`` the remaining max_new_tokens - 1 steps.  ``barrier``: called before each timed
        section (a group barrier in tensor-parallel runs)."""
        B, S = ids.shape
        assert S + max_new_tokens < self.T
        sync = (lambda: torch.cuda.synchronize(self.device)) if self.device.type == "cuda" else (lambda: None)
        if barrier:
            barrier()
        sync()
        t0 = time.perf_counter()
        first_logits = self.prefill(ids)
        sync()
        t1 = time.perf_counter()
        if use_graph and (self._graph is None or self._graph_batch != B):
            self.capture(B)
        if barrier:
            barrier()
        sync()
        t2 = time.perf_counter()
        for _ in range(max_new_tokens - 1):
            if use_graph:
                self._graph.replay()
            else:
                self._decode_step(B)
        sync()
        t3 = time.perf_counter()
        return (self.out[:B, :max_new_tokens].clone(), first_logits,
                {"prefill_s": t1 - t0, "decode_s": t3 - t2, "prefill_tok_s": B * S / (t1 - t0),
                 "decode_tok_s": B * (max_new_tokens - 1) / (t3 - t2)})

    def release(self):
        """Drops the captured graph (it refers to the group's communicators in a tensor-parallel run)."""
        self._graph = None
        torch.cuda.synchronize(self.device)
