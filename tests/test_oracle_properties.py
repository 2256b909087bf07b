"""CPU: size-independent properties of the oracle (round trips, layout invariants, edge cases)."""
import numpy as np
import pytest
import torch

from conftest import bits, make_weight

SHAPES = [
    (96, 64, 64, 32), (100, 70, 32, 16), (256, 128, 1024, 32), (48, 33, 16, 32), (16, 8, 16, 8),
    (130, 200, 64, 64), (64, 256, 32, 128), (1000, 96, 128, 32), (33, 5, 16, 8),
]


@pytest.mark.parametrize("K,N,th,tw", SHAPES)
def test_round_trip(oracle, K, N, th, tw):
    W = make_weight(K, N, seed=K * 7 + N)
    raw = bits(W)
    r = oracle.compress_bf16(raw, th, tw)
    th2, tw2 = r.tile_height, r.tile_width
    assert th2 <= max(K, 1) * 2 and th2 % 16 == 0 or th2 < 16
    e, m = oracle.split_bf16(raw)
    assert np.array_equal(oracle.decode_plane(r, K, N, th2, tw2), e)
    assert np.array_equal(oracle.decode_bf16(r, r["mantissa"], K, N, th2, tw2), raw)
    # layout invariants of src/cuda/rans_ops.cu:328-370
    W2 = 2 * tw2
    assert r.stream_len == int((r.tile_max_lens.astype(np.int64) * W2).sum())
    assert np.array_equal(r.tile_offsets.astype(np.int64),
                          np.concatenate([[0], np.cumsum(r.tile_max_lens.astype(np.int64) * W2)[:-1]]))
    sizes = r.output_sizes.reshape(-1, W2)
    assert np.array_equal(sizes.max(axis=1), r.tile_max_lens)
    # zero prefix above short streams
    t = int(np.argmax(r.tile_max_lens))
    tile = r.stream[r.tile_offsets[t]: r.tile_offsets[t] + r.tile_max_lens[t] * W2].reshape(-1, W2)
    for j in range(W2):
        pad = int(r.tile_max_lens[t] - sizes[t, j])
        assert not tile[:pad, j].any()


@pytest.mark.parametrize("K,N,th,tw", SHAPES[:5])
def test_dense_round_trip(oracle, K, N, th, tw):
    raw = bits(make_weight(K, N, seed=3 + K))
    e, _ = oracle.split_bf16(raw)
    f, c = oracle.rans_lut(e)
    d = oracle.encode_dense(e, f, c, th, tw)
    assert d.stream_len == int(d.output_sizes.astype(np.int64).sum())
    assert np.array_equal(oracle.decode_plane_dense(d, K, N, d.tile_height, d.tile_width), e)


def test_partial_tiles_have_empty_streams(oracle):
    # K = 96 with 64-row tiles: the last tile has 32 rows, all in the top halves; bottom-half streams are empty
    raw = bits(make_weight(96, 64, seed=5))
    r = oracle.compress_bf16(raw, 64, 32)
    sizes = r.output_sizes.reshape(2, 2, 2, 32)          # [tk][tn][A/B][col]
    assert (sizes[1, :, 1, :] == 0).all()
    assert (r.states.reshape(2, 2, 2, 32)[1, :, 1, :] == 1 << 16).all()


def test_skewed_flat_and_single_symbol_planes(oracle):
    rng = np.random.default_rng(0)
    for plane in (rng.integers(0, 256, (64, 32), dtype=np.uint8),            # flat: ~8 bit / symbol
                  np.full((64, 32), 7, np.uint8),                              # one symbol
                  (rng.zipf(1.2, (128, 64)) % 256).astype(np.uint8)):          # heavy tail, rare symbols need 2 bytes
        f, c = oracle.rans_lut(plane)
        r = oracle.encode_tiled(plane, f, c, 32, 32)
        assert np.array_equal(oracle.decode_plane(r, *plane.shape, 32, 32), plane)
        d = oracle.encode_dense(plane, f, c, 32, 32)
        assert np.array_equal(oracle.decode_plane_dense(d, *plane.shape, 32, 32), plane)


def test_embedding_and_linear_semantics(oracle):
    K, N, th, tw = 200, 96, 64, 32
    W = make_weight(K, N, seed=9)
    r = oracle.compress_bf16(bits(W), th, tw)
    ids = np.array([0, 199, 200, -5, 63, 64, 31, 32, 100])
    emb = oracle.embedding(ids, r, r["mantissa"], K, N, th, tw)
    for i, t in enumerate(ids):
        want = bits(W[t]) if 0 <= t < K else np.zeros(N, np.uint16)
        assert np.array_equal(emb[i], want)
    x = torch.randn(5, K, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16)
    y = oracle.linear(bits(x), r, r["mantissa"], K, N, th, tw)
    assert np.allclose(y, (x.double() @ W.double()).numpy(), rtol=1e-6, atol=1e-7)
    xt = torch.randn(3, N, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16)
    yt = oracle.linear(bits(xt), r, r["mantissa"], K, N, th, tw, transposed=True)
    assert np.allclose(yt, (xt.double() @ W.double().t()).numpy(), rtol=1e-6, atol=1e-7)


def test_baseline_config_one_round_trip(oracle):
    """The CPU round trip BASELINE names: 4096x4096 N(0,0.02) bf16, default tile, bit-exact."""
    W = make_weight(4096, 4096, seed=1001)
    raw = bits(W)
    r = oracle.compress_bf16(raw, 1024, 32)
    assert np.array_equal(oracle.decode_bf16(r, r["mantissa"], 4096, 4096, 1024, 32), raw)
    stored = r.stream_len + r["mantissa"].size + 4 * r.num_streams + 8 * r.tile_offsets.size + 1024 + 4096
    assert 0.66 < stored / (2 * 4096 * 4096) < 0.70
