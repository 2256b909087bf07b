"""Tensor-parallel shards of a compressed weight, cut out of the compressed arrays
themselves: tiles are self-contained (own states, own byte block) and share only
the per-tensor tables, so a shard is a re-indexing of existing bytes, never a
re-encode, and a rank only ever holds and decodes its own part.

The reference has no multi-GPU code; the layout facts used here are those of
src/cuda/rans_ops.cu:328-370 (tile t = tk * tiles_n + tn owns states
[t*2*tw, (t+1)*2*tw) and the bytes [tile_offsets[t], + tile_max_lens[t]*2*tw))
and comp_inference/comp_inference.py:35-64 (mantissa plane [tk][tn][th][tw]).

  column shard  (split N = output features: q/k/v, gate, up, LM-head vocabulary when stored [H,V])
  row shard     (split K = input features:  o_proj, down_proj; partial sums need an all-reduce)
"""
import torch

_KEYS = ("rans_exp_stream", "rans_exp_states", "rans_exp_tables", "rans_exp_slot_map", "rans_exp_tile_offsets",
         "rans_exp_tile_max_lens", "rans_man_raw")


def _geom(c):
    K, N = c["shape"]
    th, tw = c["tile_height"], c["tile_width"]
    return K, N, th, tw, -(-K // th), -(-N // tw)


def _i64(t):
    return t.view(torch.int32).to(torch.int64) if t.dtype == torch.uint32 else t.to(torch.int64)


def _u32(t):
    return t.to(torch.int32).view(torch.uint32)


def _finish(c, stream, states, lens, man, K, N, Tk, Tn):
    th, tw = c["tile_height"], c["tile_width"]
    lens64 = _i64(lens).reshape(-1)
    sizes = lens64 * (2 * tw)
    offs = torch.cumsum(sizes, 0) - sizes
    out = dict(c)
    out.update(rans_exp_stream=stream.contiguous(), rans_exp_states=states.reshape(-1).contiguous(),
               rans_exp_tile_offsets=_u32(offs), rans_exp_tile_max_lens=lens.reshape(-1).contiguous(),
               rans_man_raw=man.reshape(-1).contiguous(), shape=(K, N), num_tiles_k=Tk, num_tiles_n=Tn,
               num_streams=Tk * Tn * 2 * tw)
    out.pop("output_sizes", None)
    return out


def shard_rows(c, rank, world):
    """Rows (K, the reduction dimension) [rank*K/world, (rank+1)*K/world) of a compressed [K,N] weight.
    K/world must be a multiple of the tile height, so every shard starts on a tile row."""
    K, N, th, tw, Tk, Tn = _geom(c)
    if K % world or (K // world) % th:
        raise ValueError(f"K={K} cannot be cut into {world} row shards on {th}-row tile boundaries")
    per = K // world // th
    k0, k1 = rank * per, (rank + 1) * per
    offs, lens = _i64(c["rans_exp_tile_offsets"]), c["rans_exp_tile_max_lens"]
    lens64 = _i64(lens)
    t0, t1 = k0 * Tn, k1 * Tn
    b0 = int(offs[t0])
    b1 = int(offs[t1 - 1] + lens64[t1 - 1] * 2 * tw)
    stream = c["rans_exp_stream"][b0:b1]
    states = c["rans_exp_states"].reshape(Tk * Tn, 2 * tw)[t0:t1]
    man = c["rans_man_raw"].reshape(Tk * Tn, th * tw)[t0:t1]
    return _finish(c, stream, states, lens.reshape(-1)[t0:t1], man, K // world, N, per, Tn)


def shard_cols(c, rank, world):
    """Columns (N, output features) [rank*N/world, (rank+1)*N/world); N/world must be a multiple of the tile width."""
    K, N, th, tw, Tk, Tn = _geom(c)
    if N % world or (N // world) % tw:
        raise ValueError(f"N={N} cannot be cut into {world} column shards on {tw}-column tile boundaries")
    per = N // world // tw
    n0, n1 = rank * per, (rank + 1) * per
    offs = _i64(c["rans_exp_tile_offsets"]).reshape(Tk, Tn)
    lens = c["rans_exp_tile_max_lens"].reshape(Tk, Tn)
    lens64 = _i64(lens)
    begin = offs[:, n0].tolist()
    end = (offs[:, n1 - 1] + lens64[:, n1 - 1] * 2 * tw).tolist()
    src = c["rans_exp_stream"]
    pieces = [src[int(b):int(e)] for b, e in zip(begin, end)]       # one contiguous run per tile row
    stream = torch.cat(pieces) if pieces else src[:0]
    states = c["rans_exp_states"].reshape(Tk, Tn, 2 * tw)[:, n0:n1]
    man = c["rans_man_raw"].reshape(Tk, Tn, th * tw)[:, n0:n1]
    return _finish(c, stream, states, lens[:, n0:n1], man, K, N // world, Tk, per)


def can_shard_rows(K, th, world):
    return K % world == 0 and (K // world) % th == 0


def can_shard_cols(N, tw, world):
    return N % world == 0 and (N // world) % tw == 0
