"""Benchmark of the compressed-weight hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--batch M]

Workload (named in the JSON line's ``config.workload``): the fused decode-GEMV of the seven linear
layers of one Llama-2-7B decoder block (q, k, v, o: 4096x4096; gate, up: 4096->11008; down:
11008->4096), weights seeded N(0, 0.02) bf16, rANS-compressed in the reference's tiled stream layout
(tile 128x32), activation batch M (default 1).  One "step" is one token batch through the seven
layers; about 290 MB of compressed weights are read per step, more than twice the L2, so every step
streams from HBM.  ``value`` is tokens/s with all inputs resident in HBM (one CUDA graph replay per
step, timed with CUDA events); ``e2e`` is the same work through the public module API
(RansLinear.forward) the way a serving loop runs a decode step: host-to-device copy of the activations
from pinned memory, the seven module calls and the copy of the result back to pinned host memory are
captured once with torch.cuda.graph and replayed, the host waiting for the result after every step.

With --gpus N > 1 (launched under torch.distributed.run) the block is tensor parallel: q/k/v/gate/up
are column shards, o/down row shards cut out of the compressed arrays, with an all-reduce of the
activations after o and down (a one-shot kernel over peer memory, NCCL where that is unavailable);
every rank decodes only its own shard.  Total work is fixed as N grows ("strong" scaling).

--impl reference times the CPU restatement of the reference's algorithm (the oracle; the reference
ships no CPU codec) on the host cores, on the same workload, metric and unit.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np
import torch

TILE_H, TILE_W = 128, 32
HIDDEN, FFN = 4096, 11008
# name, in_features (K), out_features (N), seed, tensor-parallel kind
LAYERS = [("q_proj", HIDDEN, HIDDEN, 1001, "col"), ("k_proj", HIDDEN, HIDDEN, 1011, "col"),
          ("v_proj", HIDDEN, HIDDEN, 1021, "col"), ("o_proj", HIDDEN, HIDDEN, 1031, "row"),
          ("gate_proj", HIDDEN, FFN, 1002, "col"), ("up_proj", HIDDEN, FFN, 1012, "col"),
          ("down_proj", FFN, HIDDEN, 1003, "row")]
METRIC = "fused decode-GEMV tok/s (one Llama-2-7B decoder block: 7 rANS-compressed linears)"
# DRAM bytes (read + write) per launch of the fused kernel from one ncu capture of the 4096x4096 layer
# (profiles/linear_mma4_4096x4096_tile128.md); traffic grows with the compressed size, so a step's
# average launch is scaled by its compressed bytes.
NCU_TRAFFIC_4096 = 24.17e6
NCU_BYTES_4096 = 24.06e6


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


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


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


# ------------------------------------------------------------------------------------------- ours

def build_block(rank, world, device):
    """Compressed modules of this rank's part of the block, plus byte counts for the roofline."""
    import comp_inference_b200 as ci
    from comp_inference_b200 import sharding
    mods, wbytes, notes = {}, 0, []
    for name, K, N, seed, kind in LAYERS:
        Wkn = make_weight_kn(K, N, seed).to(device)
        if world == 1:
            c = ci.compress_weight_cuda(Wkn, TILE_H, TILE_W)
        elif kind == "col":
            c = sharding.shard_cols(ci.compress_weight_cuda(Wkn, TILE_H, TILE_W), rank, world)
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
        mods[name] = m
        wbytes += sum(c[key].numel() * c[key].element_size() for key in
                      ("rans_exp_stream", "rans_exp_states", "rans_exp_tile_offsets", "rans_exp_tile_max_lens",
                       "rans_man_raw")) + 1024 + 4096
    return mods, wbytes, notes


def block_step(mods, x, world):
    """One token batch through the seven linears (attention and the SwiGLU product are outside the hot
    path and left out; the data flow between the layers is real).  With N > 1, o_proj and down_proj are
    RansRowParallelLinear: they all-reduce their output themselves (inside the GEMV kernel for one or two
    rows, else with the one-shot kernel or NCCL)."""
    q = mods["q_proj"](x)
    mods["k_proj"](x)
    mods["v_proj"](x)
    h = mods["o_proj"](q)                       # column shard of q feeds the row shard of o
    g = mods["gate_proj"](h)
    mods["up_proj"](h)
    return mods["down_proj"](g)


def secondary_metrics(mods, device):
    """The other two halves of the headline metric on the same block, N = 1 only, short runs outside the
    timed region: stand-alone rANS decode (effective uncompressed GB/s) and prefill through the tcgen05
    decode-GEMM (tokens/s at 512 activation rows)."""
    import comp_inference_b200 as ci

    def timed(fn, iters):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    def decode_all():
        for m in mods.values():
            ci.rans_decompress_bf16(m.rans_exp_stream, m.rans_exp_states, m.rans_exp_tables, m.rans_exp_slot_map,
                                    (m.in_features, m.out_features), m.rans_exp_tile_offsets,
                                    m.rans_exp_tile_max_lens, m.tile_k, m.tile_n, m.rans_man_raw)

    dense_bytes = sum(2 * m.in_features * m.out_features for m in mods.values())
    ms = timed(decode_all, 10)
    peak, src = peaks()
    out = {"decode_bf16": {"effective_uncompressed_GBs": dense_bytes / (ms * 1e-3) / 1e9, "ms_per_block": ms,
                           "frac_of_hbm_peak": dense_bytes / (ms * 1e-3) / 1e9 / peak, "peak_source": f"of {src}"}}
    x = torch.randn(512, HIDDEN, generator=torch.Generator().manual_seed(2512)).to(torch.bfloat16).to(device)
    ms = timed(lambda: block_step(mods, x, 1), 10)
    flops = sum(2.0 * 512 * m.in_features * m.out_features for m in mods.values())
    out["prefill_M512"] = {"tok_s": 512 / (ms * 1e-3), "ms_per_block": ms, "TFLOPs": flops / (ms * 1e-3) / 1e12,
                           "kernel": "k_linear_gemm (tcgen05.mma, TMEM accumulators)"}
    # the same 512 rows through the reference's other prefill route: stand-alone decode into a scratch buffer,
    # then a library GEMM (RansLinear(prefill_policy="decode_then_gemm"))
    for m in mods.values():
        m.prefill_policy = "decode_then_gemm"
    ms = timed(lambda: block_step(mods, x, 1), 10)
    for m in mods.values():
        m.prefill_policy = "fused"
    out["prefill_M512_decode_then_gemm"] = {"tok_s": 512 / (ms * 1e-3), "ms_per_block": ms,
                                            "TFLOPs": flops / (ms * 1e-3) / 1e12,
                                            "kernel": "k_decode4 into an L2-sized scratch + cuBLAS bf16 GEMM"}
    # vocabulary table 32000 x 4096 stored [V, H]: row gather of 4096 ids, and the LM head at batch 1
    V = 32000
    table = make_weight_kn(V, HIDDEN, 1004).to(device)
    c = ci.compress_weight_cuda(table, TILE_H, TILE_W)
    emb = ci.RansEmbedding(V, HIDDEN, c["tile_height"], c["tile_width"]).load_compressed(c).to(device)
    head = ci.RansLMHead(HIDDEN, V, c["tile_height"], c["tile_width"]).load_compressed(c).to(device)
    ids = torch.randint(0, V, (4096,), generator=torch.Generator().manual_seed(3001)).to(device)
    rows = emb(ids)
    exact = bool(torch.equal(rows.view(torch.int16), table[ids].view(torch.int16)))
    ms = timed(lambda: emb(ids), 10)
    out["embedding_4096_ids"] = {"ms": ms, "out_GBs": 4096 * HIDDEN * 2 / (ms * 1e-3) / 1e9, "bit_exact": exact,
                                 "symbols_decoded_per_emitted": (TILE_H // 2 + 1) / 2.0}
    x1 = torch.randn(1, HIDDEN, generator=torch.Generator().manual_seed(2001)).to(torch.bfloat16).to(device)
    head(x1)                                                       # builds the transposed twin
    ms = timed(lambda: head(x1), 10)
    out["lm_head_batch1"] = {"ms": ms, "effective_uncompressed_GBs": 2.0 * V * HIDDEN / (ms * 1e-3) / 1e9}
    return out


def kernels_once(args):
    """One small invocation of each hot kernel on one 4096x4096 weight (24 MB compressed, nothing else resident):
    the case the ncu captures summarised under profiles/ are taken on.  Prints parity figures, no timing."""
    import comp_inference_b200 as ci
    torch.cuda.set_device(0)
    K = N = HIDDEN
    W = make_weight_kn(K, N, 1001).cuda()
    c = ci.compress_weight_cuda(W, TILE_H, TILE_W)
    m = ci.RansLinear(K, N, c["tile_height"], c["tile_width"]).load_compressed(c).cuda()
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
    ref1, ref512 = x1.float() @ W.float(), x512.float() @ W.float()
    print(json.dumps({"kernels_once": True, "decode_bit_exact": bool(torch.equal(w.view(torch.int16), W.view(torch.int16))),
                      "embedding_bit_exact": bool(torch.equal(rows.view(torch.int16), W[ids].view(torch.int16))),
                      "gemv_rel_err": float((y1.float() - ref1).abs().max() / ref1.abs().max()),
                      "gemm_rel_err": float((y512.float() - ref512).abs().max() / ref512.abs().max())}))


def cpu_baseline_run(M, steps, warmup):
    """Decode + matmul of the same block with the CPU oracle on all host cores; returns (tok/s, ms/step, cores)."""
    from oracle import oracle as O
    cores = O.default_threads()
    layers = []
    for name, K, N, seed, kind in LAYERS:
        raw = make_weight_kn(K, N, seed).view(torch.uint16).numpy()
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
                             "sample": f"{steps} full steps (7 layers decoded and multiplied per step); the reference "
                                       "ships no CPU codec, this is the C restatement of its algorithm"},
            "e2e": {"value": val, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def workload_config(M, world):
    return {"workload": "llama2-7b decoder block, 7 compressed linears, fused decode-GEMV", "batch": M,
            "shapes_out_in": [[4096, 4096]] * 4 + [[11008, 4096]] * 2 + [[4096, 11008]],
            "tile": [TILE_H, TILE_W], "weights": "N(0,0.02) bf16, seeded", "activations": "N(0,1) bf16",
            "l2": "inputs larger than L2 (about 290 MB of compressed weights per step)",
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
        dist.init_process_group("nccl", device_id=device)
        trace("process group up")
    M = args.batch
    mods, wbytes, notes = build_block(rank, world, device)
    if world > 1:
        from comp_inference_b200.collective import OneShotAllReduce
        reducer = OneShotAllReduce(capacity=16 * HIDDEN, device=device)
        row_mods = [m for m in mods.values() if hasattr(m, "reducer")]
        for m in row_mods:
            m.reducer = reducer
            m._fusable = False
        fuse = reducer.native and not args.no_fuse_exchange
        if fuse:
            # one step each way before anything is timed: the fused exchange must reproduce the separate one on
            # every rank, else all ranks drop it together
            xt = torch.randn(M, HIDDEN, generator=torch.Generator().manual_seed(77)).to(torch.bfloat16).to(device)
            y_sep = block_step(mods, xt, world).float()
            for m in row_mods:
                m._fusable = True
            y_fused = block_step(mods, xt, world).float()
            torch.cuda.synchronize()
            from comp_inference_b200 import _lib as _cl
            good = (float((y_fused - y_sep).abs().max()) <= 3e-2 * max(float(y_sep.abs().max()), 1e-6)
                    and reducer.status() == 0 and _cl.kernel_status(device) == 0)
            verdict = torch.tensor([1 if good else 0], device=device, dtype=torch.int32)
            dist.all_reduce(verdict, op=dist.ReduceOp.MIN)
            fuse = bool(verdict.item())
            for m in row_mods:
                m._fusable = fuse
            if not fuse:
                notes.append("fused exchange failed its check against the separate one: not used")
        how = "fused into the row-parallel GEMV" if fuse else "one-shot kernel behind the GEMV"
        notes.append(f"activation all-reduce over peer memory, {how}" if reducer.native
                     else f"activation all-reduce: NCCL ({reducer.why})")

    gen = torch.Generator().manual_seed(2000 + M)
    x_host = torch.randn(M, HIDDEN, generator=gen).to(torch.bfloat16).pin_memory()
    x_dev = x_host.to(device)
    y_host = torch.empty(M, HIDDEN, dtype=torch.bfloat16).pin_memory()

    # ---- device-resident: one CUDA graph per step -------------------------------------------
    for _ in range(3):
        y = block_step(mods, x_dev, world)
    torch.cuda.synchronize()
    trace("eager warm-up done")
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        block_step(mods, x_dev, world)
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=side):
            y_graph = block_step(mods, x_dev, world)
    torch.cuda.synchronize()
    trace("graph captured")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        graph.replay()
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
        time.sleep(0.3)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        graph.replay()
    e1.record()
    barrier()
    dev_ms = e0.elapsed_time(e1) / args.steps
    trace(f"device loop done {dev_ms:.3f} ms/step")

    # ---- end to end: public module API, host buffers, copies inside the timed region ------
    # What a serving loop does per token: the step (copy of the pinned host activations to the device, the
    # seven module calls, copy of the result to pinned host memory) is captured once with torch.cuda.graph
    # and replayed; the caller waits for the result before the next token.
    x_in = torch.empty_like(x_dev)
    e2e_graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        x_in.copy_(x_host, non_blocking=True)
        y_host.copy_(block_step(mods, x_in, world), non_blocking=True)
        torch.cuda.synchronize()
        with torch.cuda.graph(e2e_graph, stream=side):
            x_in.copy_(x_host, non_blocking=True)
            y_e2e = block_step(mods, x_in, world)
            y_host.copy_(y_e2e, non_blocking=True)
    torch.cuda.synchronize()
    for _ in range(max(args.warmup, 3)):
        e2e_graph.replay()
        torch.cuda.current_stream().synchronize()
    barrier()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    for _ in range(args.steps):
        e2e_graph.replay()
        torch.cuda.current_stream().synchronize()          # the caller needs the result before the next token
    e3.record()
    barrier()
    e2e_ms = e2.elapsed_time(e3) / args.steps
    trace("e2e loop done")
    clocks = sampler.stop() if sampler else None

    if world > 1:
        t = torch.tensor([dev_ms, e2e_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms, e2e_ms = t.tolist()
        wb = torch.tensor([float(wbytes)], device=device, dtype=torch.float64)
        dist.all_reduce(wb)
        wbytes_total = wb.item()
    else:
        wbytes_total = float(wbytes)

    # parity spot check of the graph's result against a dense matmul on decoded weights happens in tests;
    # here only sanity: finite output
    assert torch.isfinite(y_graph.float()).all() and torch.equal(y_host, y_graph.cpu())

    if rank == 0:
        peak, src = peaks()
        # algorithmic bytes of one step on one GPU: compressed weights + activations in + results out
        act = sum(2 * M * (K + N) for _, K, N, _, _ in LAYERS)
        algo = wbytes_total / world + act / world
        launches = len(LAYERS)
        per_launch_s = dev_ms * 1e-3 / launches               # collectives included at N > 1 (noted in config)
        achieved = algo / launches / per_launch_s / 1e9
        traffic = (wbytes_total / world / launches) * (NCU_TRAFFIC_4096 / NCU_BYTES_4096)
        line = {"metric": METRIC, "value": M / (dev_ms * 1e-3), "unit": "tok/s", "n_gpus": world,
                "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": dev_ms, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "u8 rANS decode + bf16 x bf16 -> fp32 (mma.sync)",
                "data": "synthetic", "config": workload_config(M, world),
                "e2e": {"value": M / (e2e_ms * 1e-3), "unit": "tok/s", "ms_per_step": e2e_ms,
                        "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": y_host.numel() * 2},
                "gpu_launches": launches * args.steps,
                "roofline": {"bound": "hbm", "kernel": "k_linear_mma4", "achieved": achieved, "peak": peak,
                             "unit": "GB/s", "frac": achieved / peak, "peak_source": f"of {src}",
                             "frac_of_nominal_8TBs": achieved / 8000.0, "traffic": traffic,
                             "algorithmic_bytes_per_launch": algo / launches,
                             "effective_uncompressed_GBs": sum(2 * K * N for _, K, N, _, _ in LAYERS) / world
                             / (dev_ms * 1e-3) / 1e9},
                "clocks": clocks, "notes": notes}
        if world == 1:
            line["extra"] = secondary_metrics(mods, device)
        if world == 1 and not args.no_cpu:
            val, ms, cores = cpu_baseline_run(M, 1, 1)
            line["cpu_baseline"] = {"value": val, "unit": "tok/s", "cores": cores, "kind": "port",
                                    "sample": "1 full step after 1 warm-up step (7 layers decoded and multiplied), "
                                              "CPU restatement of the reference algorithm, all host cores"}
        print(json.dumps(line))
    if world > 1:
        # The captured graph still refers to the NCCL communicator; tearing the process group down while
        # it exists blocked for minutes on the 2-GPU box.  Drop the graph, line the ranks up, and leave
        # communicator clean-up to process exit.
        trace("shutting down")
        del graph, y_graph, e2e_graph, y_e2e
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-fuse-exchange", action="store_true",
                    help="N > 1: all-reduce with the one-shot kernel behind the row-parallel GEMV instead of inside it")
    ap.add_argument("--kernels-once", action="store_true",
                    help="run each hot kernel three times on one 4096x4096 weight and exit (the ncu capture case)")
    args = ap.parse_args()
    if args.kernels_once:
        kernels_once(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
