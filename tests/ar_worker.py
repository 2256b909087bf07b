"""Child process of test_gpu_model.py::test_oneshot_allreduce: one rank.
usage: python ar_worker.py <rank> <world> <port>"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world, port = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=port, NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
    from comp_inference_b200.collective import OneShotAllReduce
    ar = OneShotAllReduce(capacity=1 << 16)
    print(f"rank {rank}: native={ar.native} {ar.why}", flush=True)
    ok = ar.native
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
    if ar.status() != 0:
        ok = False
        print(f"rank {rank}: status {ar.status()}", flush=True)
    del graph
    dist.barrier()
    torch.cuda.synchronize()
    os._exit(0 if ok else 1)


if __name__ == "__main__":
    main()
