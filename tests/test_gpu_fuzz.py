"""GPU: seeded random shapes through the four-streams-per-lane kernels (and their fall-backs) against plain
torch arithmetic on the original weight: decode and embedding bit-exact, fused linear within tolerance, status
word clean.  Complements the oracle parity cases with shapes nobody picked by hand."""
import random

import pytest
import torch

from conftest import make_weight

pytestmark = pytest.mark.gpu
REL_TOL = 1e-2


def _cases():
    rng = random.Random(20240611)
    out = []
    for i in range(36):
        th = rng.choice([16, 32, 64, 128, 128, 128])
        tiles_k = rng.choice([1, 2, 3, 4, 6, 8, 12])
        K = th * tiles_k + (rng.choice([0, 0, 0, th // 2, 5]) if i % 5 == 4 else 0)      # every fifth case: ragged K
        N = rng.choice([32, 64, 96, 100, 128, 130, 160, 200, 256, 288, 36, 4, 1024])
        M = rng.choice([1, 1, 2, 3, 5, 8, 9, 16])
        out.append((K, N, th, M, 1000 + i))
    return out


@pytest.mark.parametrize("K,N,th,M,seed", _cases())
def test_random_shapes(K, N, th, M, seed):
    import comp_inference_b200 as ci
    from comp_inference_b200 import _lib
    W = make_weight(K, N, seed)
    c = ci.compress_weight_cuda(W.cuda(), th, 32)
    a = dict(compressed_data=c["rans_exp_stream"], initial_states=c["rans_exp_states"], tables=c["rans_exp_tables"],
             slot_map=c["rans_exp_slot_map"], tile_offsets=c["rans_exp_tile_offsets"],
             tile_max_lens=c["rans_exp_tile_max_lens"], tile_k=c["tile_height"], tile_n=c["tile_width"],
             mantissas=c["rans_man_raw"])
    w = ci.rans_decompress_bf16(a["compressed_data"], a["initial_states"], a["tables"], a["slot_map"], (K, N),
                                a["tile_offsets"], a["tile_max_lens"], a["tile_k"], a["tile_n"], a["mantissas"])
    assert torch.equal(w.view(torch.int16).cpu(), W.view(torch.int16))
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(-2, K + 2, (37,), generator=g)
    rows = ci.fused_rans_embedding_triton(ids.cuda(), weight_shape=(K, N), **a).cpu()
    valid = (ids >= 0) & (ids < K)
    want = torch.zeros(37, N, dtype=torch.bfloat16)
    want[valid] = W[ids[valid]]
    assert torch.equal(rows.view(torch.int16), want.view(torch.int16))
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    ref = x.double() @ W.double()
    y = ci.fused_rans_linear_triton(x.cuda(), weight_shape=(K, N), SPLIT_K=0, **a).double().cpu()
    err = float((y - ref).abs().max() / max(float(ref.abs().max()), 1e-30))
    assert err <= REL_TOL, err
    y2 = ci.fused_rans_linear_triton(x.cuda(), weight_shape=(K, N), SPLIT_K=0, **a).double().cpu()
    assert torch.equal(y, y2)                                   # deterministic, workspace left clean
    assert _lib.kernel_status("cuda:0") == 0


# Matrices with at least six two-tile units per multiprocessor take the four-streams-per-lane GEMV kernel
# (smaller ones take the two-streams kernel): every batch size of both of its instantiations (weights as
# the A operand up to 8 rows, as the B operand for 9..16), a ragged last column tile, a bias, and several
# warps sharing a column group (partials + ticket).
@pytest.mark.parametrize("K,N,th", [(1024, 2048, 16), (2048, 1056, 32), (4096, 1000, 64), (8192, 1024, 128)])
@pytest.mark.parametrize("M", [1, 2, 3, 4, 5, 7, 8, 9, 12, 16])
def test_four_stream_gemv_all_batches(K, N, th, M):
    import comp_inference_b200 as ci
    from comp_inference_b200 import _lib
    W = make_weight(K, N, 7000 + K + N)
    c = ci.compress_weight_cuda(W.cuda(), th, 32)
    a = dict(compressed_data=c["rans_exp_stream"], initial_states=c["rans_exp_states"], tables=c["rans_exp_tables"],
             slot_map=c["rans_exp_slot_map"], tile_offsets=c["rans_exp_tile_offsets"],
             tile_max_lens=c["rans_exp_tile_max_lens"], tile_k=c["tile_height"], tile_n=c["tile_width"],
             mantissas=c["rans_man_raw"])
    g = torch.Generator().manual_seed(M * 31 + N)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    bias = torch.randn(N, generator=g).to(torch.bfloat16)
    ref = x.double() @ W.double() + bias.double()
    y = ci.fused_rans_linear_triton(x.cuda(), weight_shape=(K, N), SPLIT_K=0, bias=bias.cuda(), **a).double().cpu()
    assert y.shape == (M, N)
    err = float((y - ref).abs().max() / float(ref.abs().max()))
    assert err <= REL_TOL, err
    # every row on its own, so that a row landing in another row's place cannot hide in the maximum
    for m in range(M):
        e = float((y[m] - ref[m]).abs().max() / float(ref[m].abs().max()))
        assert e <= 2 * REL_TOL, (m, e)
    y2 = ci.fused_rans_linear_triton(x.cuda(), weight_shape=(K, N), SPLIT_K=0, bias=bias.cuda(), **a).double().cpu()
    assert torch.equal(y, y2)
    assert _lib.kernel_status("cuda:0") == 0
