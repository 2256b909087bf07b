"""Benchmark of the compressed-weight hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--batch M]

Workload (named in the JSON line's ``config.workload``): the fused decode-GEMV of the linear layers of one
Llama-2-7B decoder block (q, k, v, o: 4096x4096; gate, up: 4096->11008; down: 11008->4096), weights seeded
N(0, 0.02) bf16, rANS-compressed in the reference's tiled stream layout (tile 128x32), activation batch M
(default 1).  q|k|v and gate|up are stored and run as one concatenated matrix each, which is what the
reference's rans_compress_qkv_fused / rans_compress_gate_up_fused produce, so a step is four launches over
the same seven weights.  One "step" is one token batch through the block; about 290 MB of compressed weights
are read per step, more than twice the L2, so every step streams from HBM.  ``value`` is tokens/s with all
inputs resident in HBM (one CUDA graph replay per step, timed with CUDA events; the ``steps`` replays are
repeated several times and the median is reported with the spread); ``e2e`` is the same work through the
public module API the way a serving loop runs a decode step: host-to-device copy of the activations from
pinned memory, the module calls and the copy of the result back to pinned host memory are captured once with
torch.cuda.graph and replayed, the host waiting for the result after every step.

With --gpus N > 1 (launched under torch.distributed.run) the block is tensor parallel: qkv and gate|up
are column shards, o/down row shards cut out of the compressed arrays, with an all-reduce of the
activations after o and down (inside the GEMV kernel over peer memory; a one-shot kernel or NCCL where that
is unavailable); every rank decodes only its own shard.  Total work is fixed as N grows ("strong" scaling).
Rank 0 also runs the unsharded block and the line carries the relative error of the N-rank result.

``extra.full_model`` (every N): the whole Llama-2-7B architecture (32 layers, random init from a seed), every
linear, the embedding table and the LM head compressed through the public API and loaded with patch_model /
patch_model_tensor_parallel; a 512-token prompt and 128 greedy tokens at batch 1 and 8, wall-clock tokens/s,
with the first-step logits and the greedy tokens compared against the dense bf16 model.

--impl reference times the CPU restatement of the reference's algorithm (the oracle; the reference
ships no CPU codec) on the host cores, on the same workload, metric and unit.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # peer buffers are never bound to a multicast object

import numpy as np
import torch

TILE_H, TILE_W = 128, 32
HIDDEN, FFN, VOCAB = 4096, 11008, 32000
# HF name, in_features (K), out_features (N), seed -- the seven weights of the block
WEIGHTS = {"q_proj": (HIDDEN, HIDDEN, 1001), "k_proj": (HIDDEN, HIDDEN, 1011), "v_proj": (HIDDEN, HIDDEN, 1021),
           "o_proj": (HIDDEN, HIDDEN, 1031), "gate_proj": (HIDDEN, FFN, 1002), "up_proj": (HIDDEN, FFN, 1012),
           "down_proj": (FFN, HIDDEN, 1003)}
# launch name, the weights concatenated along the output dimension, tensor-parallel kind
LAYERS = [("qkv_proj", ("q_proj", "k_proj", "v_proj"), "col"), ("o_proj", ("o_proj",), "row"),
          ("gate_up_proj", ("gate_proj", "up_proj"), "col"), ("down_proj", ("down_proj",), "row")]
METRIC = "fused decode-GEMV tok/s (one Llama-2-7B decoder block: 7 rANS-compressed linears)"
REPEATS = 7
# DRAM bytes (read + write) per launch of the fused kernel from the most recent ncu capture of the 4096x4096
# layer at tile 128x32 (24.06 MB of compressed bytes + activations); traffic grows in proportion to the
# compressed size, so a step's average launch is scaled by its compressed bytes.
NCU_TRAFFIC_4096 = 24.17e6
NCU_BYTES_4096 = 24.06e6
NCU_CAPTURE = "ncu --set full of k_linear_mma4 on the 4096x4096 layer (bench.py --kernels-once), scaled by compressed bytes"
ROUTES = {0: "k_linear (generic split-K)", 1: "k_linear_mma", 2: "k_linear_mma4", 3: "k_linear_gemm"}


def trace(msg):
    """Progress lines on stderr when CI_BENCH_TRACE is set (to locate a stall in a multi-rank run)."""
    if os.environ.get("CI_BENCH_TRACE"):
        print(f"[bench rank {os.environ.get('RANK', '0')} +{time.perf_counter() - _T0:.1f}s] {msg}", file=sys.stderr,
              flush=True)


_T0 = time.perf_counter()


def make_weight_kn(K, N, seed):
    """HF weight [out, in] = randn * 0.02 in bf16 from a CPU generator, returned as stored: [K=in, N=out]."""
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16).t().contiguous()


def make_fused_kn(names):
    """The named weights of the block side by side: [K, sum of N]."""
    return torch.cat([make_weight_kn(*WEIGHTS[n]) for n in names], dim=1).contiguous()


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops_sustained", 1377.6)), "measured"
    return 6650.0, 1400.0, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.rows, self.proc = index, [], None

    def run(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            for line in self.proc.stdout:
                self.rows.append([c.strip() for c in line.split(",")])
        except Exception:
            pass

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
        self.join(timeout=2)
        mhz = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(mhz)}


def timed(fn, iters, warm=3):
    """Mean milliseconds per call of fn over `iters` back-to-back calls (CUDA events, current stream)."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def graphed(fn):
    """fn captured in a CUDA graph on a side stream (after one eager run there); returns the graph."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        fn()
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=side):
            fn()
    torch.cuda.synchronize()
    return graph


# ------------------------------------------------------------------------------------------- ours

def compressed_bytes(c):
    return sum(c[key].numel() * c[key].element_size() for key in
               ("rans_exp_stream", "rans_exp_states", "rans_exp_tile_offsets", "rans_exp_tile_max_lens",
                "rans_man_raw")) + 1024 + 4096


def clone_block(mods, device):
    """A second set of modules with copies of the same compressed arrays at other addresses (for the rotation that
    keeps a rank's weights out of L2 between steps)."""
    import comp_inference_b200 as ci
    out = {}
    for name, m in mods.items():
        c = {k: (v.clone() if torch.is_tensor(v) else v) for k, v in m.bench_compressed.items()}
        if hasattr(m, "reducer"):
            new = ci.RansRowParallelLinear(m.in_features, m.out_features, m.tile_k, m.tile_n).load_compressed(c).to(device)
        else:
            new = ci.RansLinear(m.in_features, m.out_features, m.tile_k, m.tile_n).load_compressed(c).to(device)
        new.first_part, new.bench_compressed = m.first_part, c
        out[name] = new
    return out


def l2_bytes(device):
    return int(getattr(torch.cuda.get_device_properties(device), "L2_cache_size", 0)) or 126 * 1024 * 1024


def build_block(rank, world, device, keep_dense=False):
    """Compressed modules of this rank's part of the block, plus byte counts for the roofline."""
    import comp_inference_b200 as ci
    from comp_inference_b200 import sharding
    mods, wbytes, notes, dense = {}, 0, [], {}
    for name, members, kind in LAYERS:
        parts = [WEIGHTS[m][1] for m in members]
        K = WEIGHTS[members[0]][0]
        Wkn = make_fused_kn(members).to(device)
        if keep_dense:
            dense[name] = Wkn
        if world == 1:
            c = ci.compress_weight_cuda(Wkn, TILE_H, TILE_W)
        elif kind == "col":
            c = sharding.shard_cols(ci.compress_weight_cuda(Wkn, TILE_H, TILE_W), rank, world, parts)
        elif sharding.can_shard_rows(K, TILE_H, world):
            c = sharding.shard_rows(ci.compress_weight_cuda(Wkn, TILE_H, TILE_W), rank, world)
        else:
            # K/world is not a whole number of 128-row tiles (11008/8 = 10.75 tiles): this rank's rows are
            # compressed as a tensor of their own, which keeps the tile size of the other layers
            k = K // world
            c = ci.compress_weight_cuda(Wkn[rank * k:(rank + 1) * k].contiguous(), TILE_H, TILE_W)
            notes.append(f"{name}: per-rank compression (K/{world} not tile aligned)")
        del Wkn
        k, n = c["shape"]
        if world > 1 and kind == "row":     # multiplies its row shard and all-reduces the output (reducer set later)
            m = ci.RansRowParallelLinear(k, n, c["tile_height"], c["tile_width"]).load_compressed(c).to(device)
        else:
            m = ci.RansLinear(k, n, c["tile_height"], c["tile_width"]).load_compressed(c).to(device)
        m.first_part = parts[0] // world                        # width of the block that feeds the next layer
        m.bench_compressed = c
        mods[name] = m
        wbytes += compressed_bytes(c)
    return mods, wbytes, notes, dense


def block_step(mods, x):
    """One token batch through the block's linears (attention and the SwiGLU product are outside the hot
    path and left out; the data flow between the layers is real: the q block of qkv feeds o, the gate block of
    gate|up feeds down).  With N > 1, o_proj and down_proj are RansRowParallelLinear: they all-reduce their
    output themselves (inside the GEMV kernel for one or two rows, else with the one-shot kernel or NCCL)."""
    qkv = mods["qkv_proj"](x)
    h = mods["o_proj"](qkv[..., :mods["qkv_proj"].first_part])
    gu = mods["gate_up_proj"](h)
    return mods["down_proj"](gu[..., :mods["gate_up_proj"].first_part])


def block_routes(mods, M):
    from comp_inference_b200 import _lib
    lib = _lib.load()
    return sorted({ROUTES.get(lib.ci_linear_route(m._weight(m.in_features, m.out_features), M), "?")
                   for m in mods.values()})


def parity_table(mods, dense, device):
    """Per-shape error of the fused linear against fp32 matmul on the dense weight: the figures the parity
    tests assert, reported instead of thrown away.  max_rel = max|y - ref| / max|ref|; allclose = the
    reference's own criterion |y - ref| <= 1e-2 + 1e-2 |ref| (tests/test_mat_mul.py:220), as the fraction of
    elements that meet it."""
    rows = []
    for name, m in mods.items():
        m.prefill_policy = "fused"                              # the table is about this repository's kernels
        W = dense[name].float()
        for M in (1, 4, 16, 512):
            x = torch.randn(M, m.in_features, generator=torch.Generator().manual_seed(2000 + M)).to(torch.bfloat16).to(device)
            y = m(x).float()
            ref = x.float() @ W
            err = (y - ref).abs()
            rows.append({"layer": name, "K": m.in_features, "N": m.out_features, "M": M,
                         "max_rel": float(err.max() / ref.abs().max()),
                         "allclose_1e-2": float((err <= 1e-2 + 1e-2 * ref.abs()).float().mean())})
        m.prefill_policy = "auto"
        del W
    return rows


def secondary_metrics(mods, dense, device, peak_hbm, peak_tf, src):
    """The other parts of the headline metric on the same block, N = 1 only, short runs outside the timed
    region."""
    import comp_inference_b200 as ci
    from comp_inference_b200 import ops
    out = {}

    # ---- stand-alone rANS decode to bf16
    def decode_all():
        for m in mods.values():
            ci.rans_decompress_bf16(m.rans_exp_stream, m.rans_exp_states, m.rans_exp_tables, m.rans_exp_slot_map,
                                    (m.in_features, m.out_features), m.rans_exp_tile_offsets,
                                    m.rans_exp_tile_max_lens, m.tile_k, m.tile_n, m.rans_man_raw)

    dense_bytes = sum(2 * m.in_features * m.out_features for m in mods.values())
    ms = timed(decode_all, 10)
    out["decode_bf16"] = {"effective_uncompressed_GBs": dense_bytes / (ms * 1e-3) / 1e9, "ms_per_block": ms,
                          "frac_of_hbm_peak": dense_bytes / (ms * 1e-3) / 1e9 / peak_hbm, "peak_source": f"of {src}"}

    # ---- GPU encoder: whole pipeline (split, histogram, table, two encoder passes) and the encoder calls alone
    W = dense["gate_up_proj"]
    ms = timed(lambda: ci.compress_weight_cuda(W, TILE_H, TILE_W), 3, warm=1)
    e, _ = ci.extract_exp_and_mantissa(W)
    f, cdf = ci.get_rans_lut(e)
    mgr = ci.ccore.RansManager(e.numel())
    ms_enc = timed(lambda: mgr.compress_tiled(e, f, cdf, TILE_H, TILE_W, _keep_on_device=True), 3, warm=1)
    out["encode"] = {"shape_KN": list(W.shape), "pipeline_ms": ms, "pipeline_bf16_in_GBs": W.numel() * 2 / (ms * 1e-3) / 1e9,
                     "encoder_ms": ms_enc, "encoder_symbols_per_s": W.numel() / (ms_enc * 1e-3),
                     "note": "encoder_ms = both passes (sizes, write) + the host wait between them"}
    del e

    # ---- small batches through the block, ours and the dense library GEMV on the same rotation (> L2)
    dense7 = {}
    for name, members, _ in LAYERS:                             # the seven weights on their own, as the reference holds them
        start = 0
        for n in members:
            dense7[n] = dense[name][:, start:start + WEIGHTS[n][1]].contiguous()
            start += WEIGHTS[n][1]

    def dense_block7(x):
        q = torch.matmul(x, dense7["q_proj"])
        torch.matmul(x, dense7["k_proj"])
        torch.matmul(x, dense7["v_proj"])
        h = torch.matmul(q, dense7["o_proj"])
        g = torch.matmul(h, dense7["gate_proj"])
        torch.matmul(h, dense7["up_proj"])
        return torch.matmul(g, dense7["down_proj"])

    def dense_block4(x):
        qkv = torch.matmul(x, dense["qkv_proj"])
        h = torch.matmul(qkv[..., :HIDDEN], dense["o_proj"])
        gu = torch.matmul(h, dense["gate_up_proj"])
        return torch.matmul(gu[..., :FFN], dense["down_proj"])

    small = {}
    for M in (1, 4, 16):
        x = torch.randn(M, HIDDEN, generator=torch.Generator().manual_seed(2000 + M)).to(torch.bfloat16).to(device)
        g_ours = graphed(lambda: block_step(mods, x))
        g7 = graphed(lambda: dense_block7(x))
        g4 = graphed(lambda: dense_block4(x))
        t_ours, t7, t4 = (timed(g.replay, 50, warm=5) for g in (g_ours, g7, g4))
        small[f"batch{M}"] = {"ours_ms": t_ours, "cublas_7_matmuls_ms": t7, "cublas_4_fused_matmuls_ms": t4,
                              "ours_over_cublas7": t7 / t_ours, "ours_tok_s": M / (t_ours * 1e-3),
                              "kernels": block_routes(mods, M)}
        del g_ours, g7, g4
    out["block_small_batches"] = dict(small, note="one CUDA graph replay per step each; cuBLAS = torch.matmul on the "
                                      "dense bf16 weights [K,N] (the reference's baseline call, tests/test_split_k.py:153), "
                                      "405 MB per step, the same > L2 rotation")
    del dense7

    # ---- prefill: 512 and 2048 rows, split-K 1/2/4/8 and the library's own choice, and decode + cuBLAS
    flops_per_row = sum(2.0 * m.in_features * m.out_features for m in mods.values())

    def block_split(x, split_k):
        def lin(m, xx):
            x2 = ops._check_x(xx, m.in_features)
            return ops._linear_call(m._weight(m.in_features, m.out_features), x2, x2.shape[0], m.out_features, None,
                                    None, split_k, False)
        qkv = lin(mods["qkv_proj"], x)
        h = lin(mods["o_proj"], qkv[..., :HIDDEN])
        gu = lin(mods["gate_up_proj"], h)
        return lin(mods["down_proj"], gu[..., :FFN])

    from comp_inference_b200 import _lib
    _lib.reserve_workspace(device, (1 << 16) + 8 * 2048 * 2 * FFN * 4)   # room for 8 partial sums of the widest layer
    for m in mods.values():
        m.prefill_policy = "fused"
    prefill = {}
    for M in (512, 2048):
        x = torch.randn(M, HIDDEN, generator=torch.Generator().manual_seed(2000 + M)).to(torch.bfloat16).to(device)
        row = {}
        for sk in (0, 1, 2, 4, 8):
            ms = timed(lambda: block_split(x, sk), 5)
            row["auto" if sk == 0 else f"split_k{sk}"] = {
                "ms_per_block": ms, "tok_s": M / (ms * 1e-3), "TFLOPs": flops_per_row * M / (ms * 1e-3) / 1e12,
                "frac_of_bf16_peak": flops_per_row * M / (ms * 1e-3) / 1e12 / peak_tf}
        for m in mods.values():
            m.prefill_policy = "decode_then_gemm"
        ms = timed(lambda: block_step(mods, x), 5)
        for m in mods.values():
            m.prefill_policy = "fused"
        row["decode_then_gemm"] = {"ms_per_block": ms, "tok_s": M / (ms * 1e-3),
                                   "TFLOPs": flops_per_row * M / (ms * 1e-3) / 1e12,
                                   "kernel": "k_decode4 into a scratch buffer + cuBLAS bf16 GEMM"}
        prefill[f"M{M}"] = row
    # both routes at batch sizes between the GEMV kernels' 16 rows and a prompt: why the modules' default is 17
    small_rows = {}
    for M in (32, 128):
        x = torch.randn(M, HIDDEN, generator=torch.Generator().manual_seed(2000 + M)).to(torch.bfloat16).to(device)
        row = {}
        for pol in ("fused", "decode_then_gemm"):
            for m in mods.values():
                m.prefill_policy = pol
            row[pol + "_ms"] = timed(lambda: block_step(mods, x), 10)
        small_rows[f"M{M}"] = row
    out["prefill_rows_32_128"] = small_rows
    for m in mods.values():
        m.prefill_policy = "auto"
    out["prefill"] = dict(prefill, kernel="k_linear_gemm (tcgen05.mma, TMEM accumulators); 'auto' = the library's own split-K choice",
                          peak_source=f"of {src} sustained bf16")
    out["prefill_M512"] = dict(prefill["M512"]["auto"], kernel="k_linear_gemm (tcgen05.mma, TMEM accumulators)")
    out["prefill_M512_decode_then_gemm"] = prefill["M512"]["decode_then_gemm"]

    # ---- vocabulary table 32000 x 4096 stored [V, H]: row gather of 4096 ids by tile height; LM head at batch 1
    table = make_weight_kn(VOCAB, HIDDEN, 1004).to(device)           # generated as [H, V] -> stored [V, H]
    ids = torch.randint(0, VOCAB, (4096,), generator=torch.Generator().manual_seed(3001)).to(device)
    sweep, best = {}, None
    for th in (16, 32, 64, 128):
        c = ci.compress_weight_cuda(table, th, TILE_W)
        emb = ci.RansEmbedding(VOCAB, HIDDEN, c["tile_height"], c["tile_width"]).load_compressed(c).to(device)
        rows = emb(ids)
        exact = bool(torch.equal(rows.view(torch.int16), table[ids].view(torch.int16)))
        ms = timed(lambda: emb(ids), 10)
        half = th // 2
        sweep[f"tile_h{th}"] = {"ms": ms, "out_GBs": 4096 * HIDDEN * 2 / (ms * 1e-3) / 1e9, "bit_exact": exact,
                                "bytes_per_weight": compressed_bytes(c) / (VOCAB * HIDDEN),
                                "symbols_decoded_per_emitted": float(((ids % half) + 1).float().mean())}
        if best is None or ms < sweep[best]["ms"]:
            best = f"tile_h{th}"
        if th == TILE_H:
            head_c = c
        del emb
    out["embedding_tile_sweep"] = sweep
    out["embedding_4096_ids"] = dict(sweep[best], tile=best,
                                     note="the format stores the tile size per tensor; the table takes the height that "
                                          "minimises the gather (a stream cannot be entered in the middle)")
    head = ci.RansLMHead(HIDDEN, VOCAB, head_c["tile_height"], head_c["tile_width"]).load_compressed(head_c).to(device)
    head.prepare()
    x1 = torch.randn(1, HIDDEN, generator=torch.Generator().manual_seed(2001)).to(torch.bfloat16).to(device)
    ms = timed(lambda: head(x1), 10)
    out["lm_head_batch1"] = {"ms": ms, "effective_uncompressed_GBs": 2.0 * VOCAB * HIDDEN / (ms * 1e-3) / 1e9}
    del head, table

    out["parity"] = parity_table(mods, dense, device)
    return out


# ------------------------------------------------------------------------------ whole model

def full_model(rank, world, device, barrier):
    """BASELINE config 5: the Llama-2-7B architecture with random-init weights from a seed, every linear, the
    embedding table and the LM head rANS-compressed through the public API (compress_model with fused
    projections -> compressed_state_dict -> patch_model / patch_model_tensor_parallel), a 512-token prompt
    and 128 greedy tokens at batch 1 and 8.  Wall-clock tokens/s (the reference's definition,
    tests/test_rans_pytorch_runtime.py:89-118) of the prompt pass and of the decode steps; parity against the
    dense bf16 model (procedure of tests/test_full_model_rans.py:227-237): error of the first-step logits,
    agreement of the argmax over all prompt positions, and the fraction of identical greedy tokens."""
    import comp_inference_b200 as ci
    from comp_inference_b200.generation import LlamaGreedyRunner
    from transformers import LlamaConfig, LlamaForCausalLM
    t_start = time.perf_counter()
    cfg = LlamaConfig(hidden_size=HIDDEN, intermediate_size=FFN, num_hidden_layers=32, num_attention_heads=32,
                      num_key_value_heads=32, vocab_size=VOCAB, rms_norm_eps=1e-5, rope_theta=10000.0,
                      max_position_embeddings=4096, tie_word_embeddings=False)
    PROMPT, NEW = 512, 128
    ids = torch.randint(0, VOCAB, (8, PROMPT), generator=torch.Generator().manual_seed(4001)).to(device)

    def fresh():
        torch.manual_seed(0)                                    # same weights on every rank and for both models
        prev = torch.get_default_dtype()
        torch.set_default_dtype(torch.bfloat16)
        try:
            with torch.device(device):
                return LlamaForCausalLM(cfg).eval()
        finally:
            torch.set_default_dtype(prev)

    # Three copies of the same seeded model: the dense bf16 baseline (kept on rank 0 for the parity figures), the
    # one that is compressed in place, and the skeleton the compressed tensors are patched into.
    dense = fresh() if rank == 0 else None
    trace("dense model built")
    ref = {}
    if rank == 0:
        runner = LlamaGreedyRunner(dense, 8, PROMPT + NEW + 8)
        for B in (1, 8):
            if B == 1:
                ref["all1"] = runner.prefill(ids[:1], all_logits=True)[0].float()
            runner.prefill(ids[:B])                             # untimed: first-use allocations, library plans
            toks, first, t = runner.generate(ids[:B], NEW)
            ref[f"toks{B}"], ref[f"first{B}"], ref[f"t{B}"] = toks.cpu(), first.float().cpu(), t
        runner.release()
        del runner
        # the same prompt in fp32 (bf16 weights widened, fp32 activations and accumulation, no TF32): the yardstick
        # both bf16 pipelines are measured against, because a random-init model has near-tied logits everywhere
        tf32 = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = False
        dense.float()
        r32 = LlamaGreedyRunner(dense, 1, PROMPT + 8)
        r32.cos, r32.sin = r32.cos.float(), r32.sin.float()
        r32.k_cache, r32.v_cache = r32.k_cache.float(), r32.v_cache.float()
        ref["all1_fp32"] = r32.prefill(ids[:1], all_logits=True)[0].float()
        del r32
        dense.to(torch.bfloat16)
        torch.backends.cuda.matmul.allow_tf32 = tf32
        torch.cuda.empty_cache()
        trace("dense reference done")
    victim = fresh()
    ci.compress_model(victim, tile_height=TILE_H, tile_width=TILE_W, fuse=True, keep_on_device=True,
                      layer_tiles={"model.embed_tokens": (16, TILE_W)})     # per-layer tile: short streams for the row gather
    state = ci.compressed_state_dict(victim, to_cpu=False)
    del victim
    torch.cuda.empty_cache()
    n_comp = sum(1 for k in state if k.endswith(".rans_exp_stream"))
    comp_bytes = sum(v.numel() * v.element_size() for k, v in state.items() if ".rans_" in k)
    trace(f"compressed {n_comp} tensors")
    model = fresh()
    if world == 1:
        model = ci.prepare_model(ci.patch_model(model, state, default_th=TILE_H, default_tw=TILE_W).to(device))
    else:
        model = ci.patch_model_tensor_parallel(model, state, rank, world, default_th=TILE_H, default_tw=TILE_W,
                                               device=device)
    del state
    torch.cuda.empty_cache()
    kinds = sorted({type(m).__name__ for m in model.modules() if type(m).__name__.startswith("Rans")})
    trace("compressed model loaded")
    runner = LlamaGreedyRunner(model, 8, PROMPT + NEW + 8)
    res = {"model": "Llama-2-7B architecture, 32 layers, random init (seed 0), 6.74 G parameters",
           "prompt_tokens": PROMPT, "new_tokens": NEW, "tile": [TILE_H, TILE_W], "compressed_tensors": n_comp,
           "compressed_GB": comp_bytes / 1e9, "modules": kinds,
           "parallelism": "single GPU" if world == 1 else f"tp{world}: column/row shards, vocabulary-parallel LM head",
           "decode": "one CUDA graph replay per token (embedding gather, 32 layers, LM head, argmax, KV update)",
           "prefill": "module default: stand-alone decode + library GEMM above 16 rows (prefill_policy='auto'); one "
                      "untimed prompt pass per batch size comes first (first-use allocations, library plan selection)",
           "parity_note": "weights are bit-identical to the dense model's; a random-init model has near-tied logits, "
                          "so free-running greedy sequences part at the first near-tie.  near_best = share of "
                          "generated tokens whose dense-bf16 logit (dense model teacher-forced on that sequence) is "
                          "within 3e-2 of the largest |logit| of the best one; *_vs_fp32 = against the same model run "
                          "in fp32"}

    def rel(a, b):
        return float((a - b).abs().max() / b.abs().max())

    for B in (1, 8):
        mine_all = runner.prefill(ids[:1], all_logits=True)[0].float() if B == 1 else None
        runner.prefill(ids[:B])                                 # untimed, as for the dense model
        toks, first, t = runner.generate(ids[:B], NEW, barrier=barrier)
        row = {"prefill_tok_s": t["prefill_tok_s"], "decode_tok_s": t["decode_tok_s"],
               "decode_ms_per_token": 1e3 * t["decode_s"] / (NEW - 1), "prefill_s": t["prefill_s"]}
        if rank == 0:
            row["first_step_logits_rel_err"] = rel(first.float().cpu(), ref[f"first{B}"])
            if mine_all is not None:
                d16, d32 = ref["all1"], ref["all1_fp32"]
                row["prompt_logits_rel_err"] = rel(mine_all, d16)
                row["prompt_logits_rel_err_vs_fp32"] = rel(mine_all, d32)
                row["dense_bf16_prompt_logits_rel_err_vs_fp32"] = rel(d16, d32)
                row["prompt_argmax_agreement"] = float((mine_all.argmax(-1) == d16.argmax(-1)).float().mean())
                row["prompt_argmax_agreement_vs_fp32"] = float((mine_all.argmax(-1) == d32.argmax(-1)).float().mean())
                row["dense_bf16_prompt_argmax_agreement_vs_fp32"] = float((d16.argmax(-1) == d32.argmax(-1)).float().mean())
            same = (toks.cpu() == ref[f"toks{B}"])
            row["greedy_tokens_identical"] = float(same.float().mean())
            row["greedy_identical_prefix"] = float(same.long().cumprod(1).sum(1).float().mean())
            # the dense model teacher-forced on the sequence the compressed model generated
            drun = LlamaGreedyRunner(dense, B, PROMPT + NEW + 8)
            seq = torch.cat([ids[:B], toks], dim=1)
            near = []
            for b in range(B):                                  # one sequence at a time: [640, 32000] logits
                lg = drun.prefill(seq[b:b + 1, :-1], all_logits=True)[0, PROMPT - 1:].float()
                chosen = lg.gather(1, toks[b].view(-1, 1)).squeeze(1)
                near.append((chosen >= lg.max(-1).values - 3e-2 * lg.abs().max(-1).values).float().mean())
                del lg
            del drun
            row["greedy_tokens_near_best"] = float(torch.stack(near).mean())
            row["dense_bf16_decode_tok_s"] = ref[f"t{B}"]["decode_tok_s"]
            row["dense_bf16_prefill_tok_s"] = ref[f"t{B}"]["prefill_tok_s"]
        del mine_all
        res[f"batch{B}"] = row
        runner.release()
    ci.check_status()
    for e in getattr(model, "_ci_exchanges", []):
        e.check_status()
    res["setup_s"] = time.perf_counter() - t_start
    runner.release()
    del runner, dense, ref
    if world > 1:
        ci.close_tensor_parallel(model)
    del model
    torch.cuda.empty_cache()
    return res


def reference_triton(args):
    """The reference's own GPU kernel on this GPU, for the column next to ours: its Python package as installed
    under baseline/_ref (``pip install --target``; git-ignored, so present only where that install was made) and
    its Triton fused linear (comp_inference/linear_triton.py:229-314) through its public function, on the block's
    seven weights at batch 1.  The compressed arrays it reads are produced by this repository's encoder, whose
    bytes are identical to the reference encoder's (tests/test_gpu_parity.py::
    test_reference_encoder_produces_the_same_bytes); the reference's own compress call is not used here because
    its extension crashed (SIGSEGV on the host, inside RansManager.compress_tiled called from
    rans_compress_module_weight_bf16) on the first 4096x4096 weight at its default 1024x32 tile on this box.
    Runs in a process of its own and prints one JSON line; the caller treats any failure as "unavailable"."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isfile(os.path.join(ref_dir, "comp_inference", "linear_triton.py")):
        print(json.dumps({"unavailable": "the reference package is not installed under baseline/_ref"}))
        return
    import importlib.util
    import comp_inference_b200 as ci
    torch.cuda.set_device(0)
    # the op's module by file path: it imports only torch and triton (the package __init__ would load the extension)
    spec = importlib.util.spec_from_file_location("ref_linear_triton", os.path.join(ref_dir, "comp_inference", "linear_triton.py"))
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    out = {"kernel": "reference fused_rans_linear_triton (Triton JIT on this GPU) from baseline/_ref, stock code, "
                     "arrays from this repository's encoder (byte-identical to the reference encoder's)"}
    x = {K: torch.randn(1, K, generator=torch.Generator().manual_seed(2001)).to(torch.bfloat16).cuda() for K in (HIDDEN, FFN)}

    def run(tile_h, split_k):
        mods = {}
        for name, (K, N, seed) in WEIGHTS.items():
            mods[name] = ci.compress_weight_cuda(make_weight_kn(K, N, seed).cuda(), tile_h, TILE_W)

        def call(c, xx):
            return ref.fused_rans_linear_triton(
                xx, c["rans_exp_stream"], c["rans_exp_states"].view(torch.int32), c["rans_exp_tables"].view(torch.int32),
                c["rans_exp_slot_map"], c["shape"], c["rans_exp_tile_offsets"].view(torch.int32),
                c["rans_exp_tile_max_lens"].view(torch.int32), c["tile_height"], c["tile_width"], c["rans_man_raw"],
                SPLIT_K=split_k)

        def step():
            for name, (K, N, seed) in WEIGHTS.items():
                call(mods[name], x[K])

        step()                                                  # Triton compiles here
        torch.cuda.synchronize()
        K, N, seed = WEIGHTS["q_proj"]
        y = call(mods["q_proj"], x[K]).float()
        want = x[K].float() @ make_weight_kn(K, N, seed).cuda().float()
        ms = timed(step, 20, warm=3)
        return {"ms_per_block_7_launches": ms, "tok_s": 1.0 / (ms * 1e-3),
                "q_proj_rel_err": float((y - want).abs().max() / want.abs().max())}

    for label, th, sk in (("default_tile_1024x32_split_k8", 1024, 8), ("tile_128x32_split_k8", TILE_H, 8),
                          ("tile_128x32_split_k1", TILE_H, 1)):
        try:
            out[label] = run(th, sk)
        except Exception as e:
            out[label] = {"error": f"{type(e).__name__}: {str(e)[:300]}"}
    print(json.dumps(out))


def reference_triton_subprocess():
    """Runs reference_triton() in a child process (its Triton JIT and its prints stay out of this one)."""
    try:
        r = subprocess.run([sys.executable, "-X", "faulthandler", os.path.abspath(__file__), "--reference-triton"],
                           capture_output=True, text=True, timeout=600)
        for line in reversed(r.stdout.strip().splitlines()):
            if line.startswith("{"):
                return json.loads(line)
        return {"unavailable": f"no result (exit code {r.returncode}): {r.stderr.strip()[-1500:]}"}
    except Exception as e:
        return {"unavailable": f"{type(e).__name__}: {e}"}


def kernels_once(args):
    """One small invocation of each hot kernel on one 4096x4096 weight (24 MB compressed, nothing else resident):
    the case the ncu captures summarised under profiles/ are taken on.  Prints parity figures, no timing."""
    import comp_inference_b200 as ci
    torch.cuda.set_device(0)
    K = N = HIDDEN
    W = make_weight_kn(K, N, 1001).cuda()
    c = ci.compress_weight_cuda(W, TILE_H, TILE_W)
    m = ci.RansLinear(K, N, c["tile_height"], c["tile_width"], prefill_policy="fused").load_compressed(c).cuda()
    g = torch.Generator().manual_seed(7)
    x1 = torch.randn(1, K, generator=g).to(torch.bfloat16).cuda()
    x512 = torch.randn(512, K, generator=g).to(torch.bfloat16).cuda()
    ids = torch.randint(0, K, (4096,), generator=g).cuda()
    for _ in range(3):
        y1 = m(x1)                                                    # k_linear_mma4
        y512 = m(x512)                                                # k_linear_gemm + k_splitk_reduce
        w = ci.rans_decompress_bf16(m.rans_exp_stream, m.rans_exp_states, m.rans_exp_tables, m.rans_exp_slot_map,
                                    (K, N), m.rans_exp_tile_offsets, m.rans_exp_tile_max_lens, m.tile_k, m.tile_n,
                                    m.rans_man_raw)                   # k_decode4
        rows = ci.fused_rans_embedding_triton(ids, m.rans_exp_stream, m.rans_exp_states, m.rans_exp_tables,
                                              m.rans_exp_slot_map, (K, N), m.rans_exp_tile_offsets,
                                              m.rans_exp_tile_max_lens, m.tile_k, m.tile_n, m.rans_man_raw)  # k_embedding4
    torch.cuda.synchronize()
    ci.check_status()
    ref1, ref512 = x1.float() @ W.float(), x512.float() @ W.float()
    print(json.dumps({"kernels_once": True, "decode_bit_exact": bool(torch.equal(w.view(torch.int16), W.view(torch.int16))),
                      "embedding_bit_exact": bool(torch.equal(rows.view(torch.int16), W[ids].view(torch.int16))),
                      "gemv_rel_err": float((y1.float() - ref1).abs().max() / ref1.abs().max()),
                      "gemm_rel_err": float((y512.float() - ref512).abs().max() / ref512.abs().max())}))


def shards_once(args):
    """Rank 0's four shard launches of an N-way tensor-parallel block on ONE GPU, no exchange: what a rank of
    `--gpus N` runs between its exchanges.  A multi-rank command is never profiled; this single-process replay is
    the case the per-launch figures and ncu captures of the shard kernels are taken on.  Three eager steps at
    batch 1, the outputs checked against a dense product; with --shards-time also per-launch times (CUDA graphs of
    eight launches each, weights L2 resident for the small shards) and the step time over copies of the shards in
    rotation (weights from HBM)."""
    import comp_inference_b200 as ci
    from comp_inference_b200 import sharding, _lib
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    world = args.shards_once
    mods, dense, wbytes = {}, {}, 0
    for name, members, kind in LAYERS:
        parts = [WEIGHTS[m][1] for m in members]
        K = WEIGHTS[members[0]][0]
        Wkn = make_fused_kn(members).to(dev)
        if kind == "col":
            c = sharding.shard_cols(ci.compress_weight_cuda(Wkn, TILE_H, TILE_W), 0, world, parts)
            dense[name] = torch.cat([Wkn[:, sum(parts[:i]):sum(parts[:i]) + p // world] for i, p in enumerate(parts)], 1)
        elif sharding.can_shard_rows(K, TILE_H, world):
            c = sharding.shard_rows(ci.compress_weight_cuda(Wkn, TILE_H, TILE_W), 0, world)
            dense[name] = Wkn[:K // world]
        else:
            c = ci.compress_weight_cuda(Wkn[:K // world].contiguous(), TILE_H, TILE_W)
            dense[name] = Wkn[:K // world]
        del Wkn
        k, n = c["shape"]
        m = ci.RansLinear(k, n, c["tile_height"], c["tile_width"]).load_compressed(c).to(dev)
        m.first_part, m.bench_compressed = parts[0] // world, c
        wbytes += compressed_bytes(c)
        mods[name] = m.prepare()
    res = {"shards_once": world, "tile": [TILE_H, TILE_W], "layers": {}}
    for name, m in mods.items():
        x = torch.randn(1, m.in_features, generator=torch.Generator().manual_seed(11)).to(torch.bfloat16).to(dev)
        for _ in range(3):
            y = m(x)
        torch.cuda.synchronize()
        ref = x.float() @ dense[name].float()
        row = {"shape_in_out": [m.in_features, m.out_features],
               "kernel": ROUTES[_lib.load().ci_linear_route(m._weight(m.in_features, m.out_features), 1)],
               "rel_err": float((y.float() - ref).abs().max() / ref.abs().max())}
        if args.shards_time:
            def many():
                for _ in range(8):
                    m(x)
            row["us"] = timed(graphed(many).replay, 100, warm=10) * 1e3 / 8
        res["layers"][name] = row
    if args.shards_time:
        x = torch.randn(1, HIDDEN, generator=torch.Generator().manual_seed(12)).to(torch.bfloat16).to(dev)
        res["step_us_l2_resident"] = timed(graphed(lambda: block_step(mods, x)).replay, 200, warm=20) * 1e3
        # the step as a model with many layers sees it: copies of the shards in rotation, together larger than L2
        copies = max(2, -(-int(1.25 * l2_bytes(dev)) // int(wbytes)))
        sets = [mods] + [clone_block(mods, dev) for _ in range(copies - 1)]
        for ms in sets[1:]:
            for m in ms.values():
                m.prepare()

        def rotation():
            for ms in sets:
                block_step(ms, x)
        res["copies"] = copies
        res["step_us"] = timed(graphed(rotation).replay, 100, warm=10) * 1e3 / copies
    ci.check_status()
    print(json.dumps(res))


def cpu_baseline_run(M, steps, warmup):
    """Decode + matmul of the same block with the CPU oracle on all host cores; returns (tok/s, ms/step, cores)."""
    from oracle import oracle as O
    cores = O.default_threads()
    layers = []
    for name, members, kind in LAYERS:
        K = WEIGHTS[members[0]][0]
        raw = make_fused_kn(members).view(torch.uint16).numpy()
        N = raw.shape[1]
        r = O.compress_bf16(raw, TILE_H, TILE_W, cores)
        layers.append((name, K, N, r))
    x = {K: torch.randn(M, K, generator=torch.Generator().manual_seed(2000 + M)).to(torch.bfloat16)
            .view(torch.uint16).numpy() for K in (HIDDEN, FFN)}

    def step():
        for name, K, N, r in layers:
            O.linear(x[K], r, r["mantissa"], K, N, TILE_H, TILE_W, False, cores)

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    return M / dt, dt * 1e3, cores


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = max(1, min(args.steps, 50)), max(1, min(args.warmup, 3))
    val, ms, cores = cpu_baseline_run(args.batch, steps, warmup)
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": "tok/s", "n_gpus": args.gpus,
            "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "u8 rANS decode + bf16 x bf16 -> fp32", "data": "synthetic",
            "config": workload_config(args.batch, 1),
            "cpu_baseline": {"value": val, "unit": "tok/s", "cores": cores, "kind": "port",
                             "sample": f"{steps} full steps (the block's weights decoded and multiplied per step); the "
                                       "reference ships no CPU codec, this is the C restatement of its algorithm"},
            "e2e": {"value": val, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def workload_config(M, world, copies=1, rank_mb=290.0):
    if copies == 1:
        l2 = f"inputs larger than L2 (about {rank_mb:.0f} MB of compressed weights per GPU and step)"
    else:
        l2 = (f"inputs larger than L2: {copies} copies of the GPU's shards at different addresses, one per step in "
              f"rotation ({copies} x {rank_mb:.0f} MB per GPU)")
    return {"workload": "llama2-7b decoder block, 7 compressed linears, fused decode-GEMV", "batch": M,
            "shapes_out_in": [[4096, 4096]] * 4 + [[11008, 4096]] * 2 + [[4096, 11008]],
            "launches_per_step": 4,
            "fused_projections": "q|k|v as one [4096,12288] and gate|up as one [4096,22016] compressed matrix "
                                 "(rans_compress_qkv_fused / rans_compress_gate_up_fused): 4 launches over the 7 weights",
            "tile": [TILE_H, TILE_W], "weights": "N(0,0.02) bf16, seeded", "activations": "N(0,1) bf16",
            "l2": l2,
            "parallelism": "single GPU" if world == 1 else f"tp{world} (column/row shards of the compressed tiles)"}


def run_ours(args):
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU path for --impl ours")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    trace("start")
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")          # plain peer loads and stores only
        dist.init_process_group("nccl", device_id=device)
        trace("process group up")
    import comp_inference_b200 as ci
    M = args.batch
    peak_hbm, peak_tf, src = peaks()
    mods, wbytes, notes, dense = build_block(rank, world, device, keep_dense=(world == 1 and not args.no_extra))
    # A rank's shards shrink with N; below about one L2 size they would stay cached from step to step.  Steps then
    # rotate over several copies of the shards so that every step streams its weights from HBM, as a model with
    # many layers does.
    copies = max(1, -(-int(1.25 * l2_bytes(device)) // int(wbytes)))
    sets = [mods] + [clone_block(mods, device) for _ in range(copies - 1)]
    reducer = None
    if world > 1:
        from comp_inference_b200.collective import OneShotAllReduce
        reducer = OneShotAllReduce(capacity=16 * HIDDEN, device=device)
        row_mods = [m for ms in sets for m in ms.values() if hasattr(m, "reducer")]
        for m in row_mods:
            m.reducer = reducer
            m.fuse_exchange = not args.no_fuse_exchange
            m.prepare()                                         # collective: the group's verdict per layer
        fused = [m._fusable for m in row_mods]
        how = ("fused into the row-parallel GEMV" if all(fused) else
               "one-shot kernel behind the GEMV" if not any(fused) else "fused in some layers, one-shot kernel in others")
        notes.append(f"activation all-reduce over peer memory, {how}" if reducer.native
                     else f"activation all-reduce: NCCL ({reducer.why})")
    for ms in sets:
        for m in ms.values():
            if not hasattr(m, "reducer"):
                m.prepare()

    gen = torch.Generator().manual_seed(2000 + M)
    x_host = torch.randn(M, HIDDEN, generator=gen).to(torch.bfloat16).pin_memory()
    x_dev = x_host.to(device)
    y_host = torch.empty(M, HIDDEN, dtype=torch.bfloat16).pin_memory()

    # ---- N > 1: the N-rank result against the unsharded block on rank 0 ------------------------
    tp_err = None
    if world > 1:
        y_tp = block_step(mods, x_dev).float()
        torch.cuda.synchronize()
        if rank == 0:
            full, _, _, _ = build_block(0, 1, device)
            y_full = block_step(full, x_dev).float()
            tp_err = float((y_tp - y_full).abs().max() / y_full.abs().max())
            del full
            torch.cuda.empty_cache()
        dist.barrier()

    # ---- device-resident: one CUDA graph per step -------------------------------------------
    for _ in range(3):
        for ms in sets:
            block_step(ms, x_dev)
    torch.cuda.synchronize()
    trace("eager warm-up done")
    side = torch.cuda.Stream()
    graphs, y_graph = [], None
    with torch.cuda.stream(side):
        for ms in sets:
            block_step(ms, x_dev)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                y = block_step(ms, x_dev)
            graphs.append(g)
            y_graph = y if y_graph is None else y_graph
    torch.cuda.synchronize()
    trace(f"{len(graphs)} graph(s) captured")
    turn = [0]

    def device_step():                                          # one step = one replay, the copies taking turns
        graphs[turn[0] % len(graphs)].replay()
        turn[0] += 1

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed_region(fn):
        """`steps` calls bracketed by barriers, REPEATS times; the per-step milliseconds of every repeat (max
        over ranks)."""
        out = []
        for _ in range(REPEATS):
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.steps):
                fn()
            e1.record()
            barrier()
            out.append(e0.elapsed_time(e1) / args.steps)
        if world > 1:
            t = torch.tensor(out, device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            out = t.tolist()
        return out

    for _ in range(max(args.warmup, 3)):
        device_step()
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
        time.sleep(0.3)
    dev_runs = timed_region(device_step)
    dev_ms = statistics.median(dev_runs)
    trace(f"device loop done {dev_ms:.4f} ms/step")

    # ---- end to end: public module API, host buffers, copies inside the timed region ------
    # What a serving loop does per token: the step (copy of the pinned host activations to the device, the
    # module calls, copy of the result to pinned host memory) is captured once with torch.cuda.graph
    # and replayed; the caller waits for the result before the next token.
    x_in = torch.empty_like(x_dev)
    e2e_graphs, e2e_keep = [], []
    with torch.cuda.stream(side):
        for ms in sets:
            x_in.copy_(x_host, non_blocking=True)
            y_host.copy_(block_step(ms, x_in), non_blocking=True)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                x_in.copy_(x_host, non_blocking=True)
                y_e2e = block_step(ms, x_in)
                y_host.copy_(y_e2e, non_blocking=True)
            e2e_graphs.append(g)
            e2e_keep.append(y_e2e)
    torch.cuda.synchronize()

    def e2e_step():
        e2e_graphs[turn[0] % len(e2e_graphs)].replay()
        turn[0] += 1
        torch.cuda.current_stream().synchronize()              # the caller needs the result before the next token

    for _ in range(max(args.warmup, 3)):
        e2e_step()
    e2e_runs = timed_region(e2e_step)
    e2e_ms = statistics.median(e2e_runs)
    time.sleep(0.2)
    trace("e2e loop done")
    clocks = sampler.stop() if sampler else None

    if world > 1:
        wb = torch.tensor([float(wbytes)], device=device, dtype=torch.float64)
        dist.all_reduce(wb)
        wbytes_total = wb.item()
    else:
        wbytes_total = float(wbytes)

    assert torch.isfinite(y_graph.float()).all() and torch.equal(y_host, y_graph.cpu())
    ci.check_status()                                           # raises if any kernel reported an error
    if reducer is not None:
        reducer.check_status()
    routes = block_routes(mods, M)

    extra = {}
    if world == 1 and not args.no_extra:
        extra = secondary_metrics(mods, dense, device, peak_hbm, peak_tf, src)
        trace("secondary metrics done")
        if not args.no_reference_leg:
            extra["reference_triton_b200"] = reference_triton_subprocess()
            trace("reference Triton leg done")
    del dense
    # the block's graphs refer to the group's communicators; drop them before the model run sets up its own
    del graphs, y_graph, e2e_graphs, e2e_keep, y_e2e
    for ms in sets:
        for m in ms.values():
            m.reducer = None
    del mods, sets
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    if reducer is not None:
        reducer.close()
    failed = tp_err is not None and tp_err > 1e-2
    line = None
    if rank == 0:
        # algorithmic bytes of one step on one GPU: compressed weights + activations in + results out
        act = sum(2 * M * (WEIGHTS[members[0]][0] + sum(WEIGHTS[n][1] for n in members)) for _, members, _ in LAYERS)
        algo = wbytes_total / world + act / world
        launches = len(LAYERS)
        per_launch_s = dev_ms * 1e-3 / launches               # collectives included at N > 1 (noted in config)
        achieved = algo / launches / per_launch_s / 1e9
        traffic = (wbytes_total / world / launches) * (NCU_TRAFFIC_4096 / NCU_BYTES_4096)
        line = {"metric": METRIC, "value": M / (dev_ms * 1e-3), "unit": "tok/s", "n_gpus": world,
                "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": dev_ms,
                "repeats": REPEATS, "ms_per_step_min_max": [min(dev_runs), max(dev_runs)],
                "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "u8 rANS decode + bf16 x bf16 -> fp32 (mma.sync)",
                "data": "synthetic", "config": workload_config(M, world, copies, wbytes / 1e6),
                "e2e": {"value": M / (e2e_ms * 1e-3), "unit": "tok/s", "ms_per_step": e2e_ms,
                        "ms_per_step_min_max": [min(e2e_runs), max(e2e_runs)],
                        "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": y_host.numel() * 2},
                "gpu_launches": launches * args.steps,
                "roofline": {"bound": "hbm", "kernel": " + ".join(routes), "achieved": achieved, "peak": peak_hbm,
                             "unit": "GB/s", "frac": achieved / peak_hbm, "peak_source": f"of {src}",
                             "frac_of_nominal_8TBs": achieved / 8000.0, "traffic": traffic,
                             "traffic_source": NCU_CAPTURE,
                             "algorithmic_bytes_per_launch": algo / launches,
                             "effective_uncompressed_GBs": sum(2 * K * N for K, N, _ in WEIGHTS.values()) / world
                             / (dev_ms * 1e-3) / 1e9},
                "clocks": clocks, "notes": notes}
        if tp_err is not None:
            extra["tp_parity_rel_err"] = tp_err
        line["extra"] = extra

    def finish(code):
        """Prints the line (rank 0) and leaves.  Multi-rank runs leave through os._exit: communicator clean-up is
        left to process exit (tearing the process group down after graphs that referred to it blocked for
        minutes on a 2-GPU box); all graphs and peer buffers are gone by then."""
        if rank == 0:
            if not line["extra"]:
                del line["extra"]
            print(json.dumps(line))
            if failed:
                print(f"tensor-parallel result differs from the unsharded block by {tp_err:.3e} (> 1e-2)", file=sys.stderr)
        sys.stdout.flush()
        sys.stderr.flush()
        if world > 1:
            os._exit(code)
        if code:
            sys.exit(code)

    if not args.no_full_model:
        # The block's figures above are complete.  The whole-model run must not be able to lose them: if it raises
        # on some rank, or does not come back (a rank that failed leaves its peers inside a collective), every
        # rank gives up after a deadline, rank 0 prints the line with the reason, and the processes leave.
        def give_up():
            if rank == 0:
                extra["full_model"] = {"error": f"did not finish within {args.full_model_deadline} s"}
            finish(1 if failed else 0)
            os._exit(1 if failed else 0)

        watchdog = threading.Timer(args.full_model_deadline + (0 if rank == 0 else 10), give_up)
        watchdog.daemon = True
        watchdog.start()
        try:
            extra["full_model"] = full_model(rank, world, device, barrier if world > 1 else None)
            trace("full model done")
        except Exception as e:
            extra["full_model"] = {"error": f"{type(e).__name__}: {str(e)[:500]}"}
            trace(f"full model failed: {e}")
            if world > 1:                                       # the peers may be waiting for this rank: no more collectives
                watchdog.cancel()
                finish(1 if failed else 0)
        watchdog.cancel()

    if rank == 0 and world == 1 and not args.no_cpu:
        val, ms, cores = cpu_baseline_run(M, 1, 1)
        line["cpu_baseline"] = {"value": val, "unit": "tok/s", "cores": cores, "kind": "port",
                                "sample": "1 full step after 1 warm-up step (the block's weights decoded and "
                                          "multiplied), CPU restatement of the reference algorithm, all host cores"}
    if world > 1:
        trace("shutting down")
        torch.cuda.synchronize()
        dist.barrier()
    finish(1 if failed else 0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-extra", action="store_true", help="skip the secondary metrics (N = 1)")
    ap.add_argument("--no-full-model", action="store_true", help="skip the whole-model run")
    ap.add_argument("--no-reference-leg", action="store_true",
                    help="skip the child process that times the reference's own Triton kernel")
    ap.add_argument("--full-model-deadline", type=int, default=420,
                    help="seconds after which a whole-model run that has not come back is abandoned (the line is still printed)")
    ap.add_argument("--no-fuse-exchange", action="store_true",
                    help="N > 1: all-reduce with the one-shot kernel behind the row-parallel GEMV instead of inside it")
    ap.add_argument("--reference-triton", action="store_true",
                    help="time the reference's own Triton fused linear from baseline/_ref (if installed) and exit")
    ap.add_argument("--tile-height", type=int, default=0,
                    help="tile height of the compressed weights (default: 128 on one GPU, 64 for tensor-parallel shards)")
    ap.add_argument("--shards-once", type=int, default=0, metavar="N",
                    help="one GPU: rank 0's four shard launches of an N-way tensor-parallel block, checked against a "
                         "dense product (the case the shard kernels are profiled on)")
    ap.add_argument("--shards-time", action="store_true", help="with --shards-once: per-launch and per-step times")
    ap.add_argument("--kernels-once", action="store_true",
                    help="run each hot kernel three times on one 4096x4096 weight and exit (the ncu capture case)")
    args = ap.parse_args()
    # Tile height is a per-tensor parameter of the stored format.  One GPU: 128 rows (fewest bytes, longest
    # streams).  Tensor-parallel shards are small enough for a launch to be bounded by the length of one stream,
    # not by throughput, and finish sooner with 64-row tiles (measured per N with --shards-once N --shards-time).
    global TILE_H
    ways = args.shards_once or int(os.environ.get("WORLD_SIZE", "1"))
    TILE_H = args.tile_height or (128 if ways == 1 else 64)
    if args.reference_triton:
        reference_triton(args)
    elif args.kernels_once:
        kernels_once(args)
    elif args.shards_once:
        shards_once(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
