"""CPU: tensor-parallel shards cut out of the compressed arrays decode to the matching slices of the
weight, and a 2-rank gloo group reproduces the full fused-linear result (all-gather for column
shards, all-reduce for row shards).  The codec side is the CPU oracle, so no GPU is needed."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import bits, make_weight


def to_dict(o):
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    return dict(rans_exp_stream=t(o.stream), rans_exp_states=t(o.states), rans_exp_tables=t(o.tables),
                rans_exp_slot_map=t(o.slot_map), rans_exp_tile_offsets=t(o.tile_offsets),
                rans_exp_tile_max_lens=t(o.tile_max_lens), rans_man_raw=t(o["mantissa"]),
                shape=(int(o["K"]), int(o["N"])), tile_height=o.tile_height, tile_width=o.tile_width)


def as_oracle(c):
    n = lambda k: c[k].numpy()
    return dict(stream=n("rans_exp_stream"), states=n("rans_exp_states"), tables=n("rans_exp_tables"),
                slot_map=n("rans_exp_slot_map"), tile_offsets=n("rans_exp_tile_offsets"),
                tile_max_lens=n("rans_exp_tile_max_lens"))


def compress(oracle, K, N, th, tw, seed):
    W = make_weight(K, N, seed)
    o = oracle.compress_bf16(bits(W), th, tw)
    o["K"], o["N"] = K, N
    return W, to_dict(o)


@pytest.mark.parametrize("K,N,th,tw,world", [(256, 128, 64, 32, 2), (512, 256, 128, 32, 4), (192, 96, 32, 16, 3),
                                             (1024, 64, 128, 32, 8)])
def test_shards_decode_to_slices(oracle, K, N, th, tw, world):
    from comp_inference_b200 import sharding
    W, c = compress(oracle, K, N, th, tw, seed=K + N)
    raw = bits(W)
    for r in range(world):
        if sharding.can_shard_rows(K, th, world):
            s = sharding.shard_rows(c, r, world)
            k, n = s["shape"]
            got = oracle.decode_bf16(as_oracle(s), s["rans_man_raw"].numpy(), k, n, th, tw)
            assert np.array_equal(got, raw[r * k:(r + 1) * k])
        if sharding.can_shard_cols(N, tw, world):
            s = sharding.shard_cols(c, r, world)
            k, n = s["shape"]
            got = oracle.decode_bf16(as_oracle(s), s["rans_man_raw"].numpy(), k, n, th, tw)
            assert np.array_equal(got, raw[:, r * n:(r + 1) * n])
            assert s["rans_exp_stream"].numel() == int((s["rans_exp_tile_max_lens"].view(torch.int32).long() * 2 * tw).sum())


def test_misaligned_shards_are_refused(oracle):
    from comp_inference_b200 import sharding
    W, c = compress(oracle, 11008 // 8, 64, 128, 32, seed=3)        # 1376 rows = 10.75 tiles of 128
    with pytest.raises(ValueError):
        sharding.shard_rows(c, 0, 2 * 43)
    assert not sharding.can_shard_rows(11008, 128, 8) and sharding.can_shard_rows(11008, 32, 8)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from comp_inference_b200 import sharding
        from oracle import oracle as O
        K, N, th, tw, M = 512, 256, 64, 32, 3
        W = make_weight(K, N, seed=77)
        o = O.compress_bf16(bits(W), th, tw)
        o["K"], o["N"] = K, N
        c = to_dict(o)
        x = torch.randn(M, K, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16)
        full = torch.from_numpy(O.linear(bits(x), o, o["mantissa"], K, N, th, tw))
        # column parallel: every rank multiplies the whole x by its slice of the outputs, then all-gather
        s = sharding.shard_cols(c, rank, world)
        yc = torch.from_numpy(O.linear(bits(x), as_oracle(s), s["rans_man_raw"].numpy(), K, N // world, th, tw))
        parts = [torch.empty_like(yc) for _ in range(world)]
        dist.all_gather(parts, yc)
        assert torch.equal(torch.cat(parts, dim=1), full)
        # row parallel: every rank multiplies its slice of x by its rows, then all-reduce
        s = sharding.shard_rows(c, rank, world)
        k = K // world
        yr = torch.from_numpy(O.linear(bits(x[:, rank * k:(rank + 1) * k].contiguous()), as_oracle(s),
                                       s["rans_man_raw"].numpy(), k, N, th, tw))
        dist.all_reduce(yr)
        assert torch.allclose(yr, full, rtol=1e-5, atol=1e-6)
        if rank == 0:
            open(out_path, "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_two_rank_tensor_parallel_linear(oracle, tmp_path):
    out = str(tmp_path / "done")
    mp.spawn(_rank_main, args=(2, _free_port(), out), nprocs=2, join=True)
    assert open(out).read() == "ok"
