"""Child process of test_gpu_model.py::test_oneshot_allreduce: one rank.
usage: python ar_worker.py <rank> <world> <port>"""
import datetime
import os
import sys

os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"           # peer buffers are never bound to a multicast object
os.environ["NCCL_NVLS_ENABLE"] = "0"

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world, port = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"),
                            timeout=datetime.timedelta(seconds=120))
    from comp_inference_b200.collective import OneShotAllGather, OneShotAllReduce
    ar = OneShotAllReduce(capacity=1 << 16)
    ag = OneShotAllGather(capacity=1 << 14)
    print(f"rank {rank}: all-reduce native={ar.native} {ar.why}; all-gather native={ag.native} {ag.why}", flush=True)
    ok = ar.native and ag.native
    # all-gather: [M, cols] blocks side by side, against NCCL (exact: nothing is added); the last shape takes the NCCL route
    for (M, cols) in ((1, 2), (1, 4000), (2, 126), (8, 2000), (16, 1024), (3, 50000)):
        for rep in range(2):
            x = (torch.arange(M * cols, dtype=torch.float32).view(M, cols) % 251 + rank).to(torch.bfloat16).cuda()
            got = ag(x)
            want = ag._nccl(x)
            torch.cuda.synchronize()
            if got.shape != (M, world * cols) or not torch.equal(got, want):
                ok = False
                print(f"rank {rank}: all-gather {M}x{cols} rep {rep} mismatch", flush=True)
    g = torch.Generator().manual_seed(100 + rank)
    for n in (1, 7, 8, 4096, 4100, 11008, 65536, 70000):       # the last one exceeds the capacity: NCCL route
        for rep in range(3):
            x = torch.randn(n, generator=g).to(torch.bfloat16).cuda()
            want = x.clone()
            dist.all_reduce(want)
            got = ar(x.clone())
            torch.cuda.synchronize()
            # both sum bf16 inputs in fp32 and round once; only the order of the additions may differ
            err = float((got.float() - want.float()).abs().max())
            tol = 2.0 ** -6 * max(float(want.float().abs().max()), 1.0)
            if err > tol:
                ok = False
                print(f"rank {rank}: n={n} rep={rep} err {err}", flush=True)
    # replayed from a CUDA graph: the call counter lives on the device
    x = torch.randn(4096, generator=g).to(torch.bfloat16).cuda()
    y = torch.empty_like(x)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        y.copy_(x)
        ar(y)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            y.copy_(x)
            ar(y)
    want = x.clone()
    dist.all_reduce(want)
    for _ in range(5):
        graph.replay()
    torch.cuda.synchronize()
    if float((y.float() - want.float()).abs().max()) > 2.0 ** -6 * max(float(want.float().abs().max()), 1.0):
        ok = False
        print(f"rank {rank}: graph replay mismatch", flush=True)
    # the exchange fused into the row-parallel GEMV: each rank holds a row shard of W, both kernels
    # (small matrix -> one-tile units, large matrix -> two-tile units), one and two activation rows, repeated
    import comp_inference_b200 as ci
    from comp_inference_b200 import _lib
    # (the third shape: one unit per column group and N = 6 mod 8, so the single-owner route of the four-streams
    # kernel pushes a short last quad)
    for (K, N) in ((1024, 256), (4096, 4096), (256 * world, 28422)):
        gw = torch.Generator().manual_seed(7)
        W = (torch.randn(K, N, generator=gw) * 0.02).to(torch.bfloat16)
        k = K // world
        c = ci.compress_weight_cuda(W[rank * k:(rank + 1) * k].contiguous().cuda(), 128 if k % 128 == 0 else 64, 32)
        lin = ci.RansRowParallelLinear(k, N, c["tile_height"], c["tile_width"], reducer=ar,
                                       fuse_exchange=True).load_compressed(c).cuda()
        lin.prepare()                                           # collective: the group's verdict on the fused route
        for M in (1, 2):
            xs = torch.randn(M, K, generator=gw).to(torch.bfloat16)
            ref = xs.double() @ W.double()
            for rep in range(3):
                y = lin(xs[:, rank * k:(rank + 1) * k].contiguous().cuda())
                torch.cuda.synchronize()
                err = float((y.double().cpu() - ref).abs().max() / ref.abs().max())
                if err > 1e-2 or not lin._fusable:
                    ok = False
                    print(f"rank {rank}: fused K={K} N={N} M={M} rep={rep} err {err} fusable {lin._fusable}", flush=True)
        # every rank must hold the same result
        mine = y.float().clone()
        other = mine.clone()
        dist.broadcast(other, src=0)
        if not torch.equal(mine, other):
            ok = False
            print(f"rank {rank}: ranks disagree on the fused result", flush=True)
    if ar.status() != 0 or ag.status() != 0 or _lib.kernel_status(f"cuda:{rank}") != 0:
        ok = False
        print(f"rank {rank}: status {ar.status()} / {ag.status()} / {_lib.kernel_status(f'cuda:{rank}')}", flush=True)
    del graph, lin
    torch.cuda.synchronize()
    ar.close()                                # barrier + release of the peer-mapped buffers, nothing in flight
    ag.close()
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    os._exit(0 if ok else 1)


if __name__ == "__main__":
    main()
