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


def tile_rows(c, k0, k1):
    """Tile rows [k0, k1) of a compressed [K,N] weight as a compressed weight of its own: one contiguous
    slice of every array.  The result covers rows [k0*th, min(k1*th, K))."""
    K, N, th, tw, Tk, Tn = _geom(c)
    if not (0 <= k0 < k1 <= Tk):
        raise ValueError(f"tile rows [{k0}, {k1}) outside [0, {Tk})")
    offs, lens = _i64(c["rans_exp_tile_offsets"]), c["rans_exp_tile_max_lens"]
    lens64 = _i64(lens)
    t0, t1 = k0 * Tn, k1 * Tn
    b0 = int(offs[t0])
    b1 = int(offs[t1 - 1] + lens64[t1 - 1] * 2 * tw)
    stream = c["rans_exp_stream"][b0:b1]
    states = c["rans_exp_states"].reshape(Tk * Tn, 2 * tw)[t0:t1]
    man = c["rans_man_raw"].reshape(Tk * Tn, th * tw)[t0:t1]
    rows = min(k1 * th, K) - k0 * th
    return _finish(c, stream, states, lens.reshape(-1)[t0:t1], man, rows, N, k1 - k0, Tn)


def tile_cols(c, ranges):
    """The tile columns of the given [n0, n1) ranges (in units of tiles), concatenated in that order, as a
    compressed weight of its own.  Every range must end on a whole tile (only the matrix's last tile column
    may be partial, and then it must come last)."""
    K, N, th, tw, Tk, Tn = _geom(c)
    ranges = [(int(a), int(b)) for a, b in ranges]
    for a, b in ranges:
        if not (0 <= a < b <= Tn):
            raise ValueError(f"tile columns [{a}, {b}) outside [0, {Tn})")
    offs = _i64(c["rans_exp_tile_offsets"]).reshape(Tk, Tn)
    lens = c["rans_exp_tile_max_lens"].reshape(Tk, Tn)
    lens64 = _i64(lens)
    src = c["rans_exp_stream"]
    begins = [offs[:, a].tolist() for a, _ in ranges]
    ends = [(offs[:, b - 1] + lens64[:, b - 1] * 2 * tw).tolist() for _, b in ranges]
    pieces = [src[int(begins[j][k]):int(ends[j][k])] for k in range(Tk) for j in range(len(ranges))]
    stream = torch.cat(pieces) if pieces else src[:0]
    st = c["rans_exp_states"].reshape(Tk, Tn, 2 * tw)
    mn = c["rans_man_raw"].reshape(Tk, Tn, th * tw)
    states = torch.cat([st[:, a:b] for a, b in ranges], dim=1)
    man = torch.cat([mn[:, a:b] for a, b in ranges], dim=1)
    new_lens = torch.cat([lens[:, a:b] for a, b in ranges], dim=1)
    cols = sum(min(b * tw, N) - a * tw for a, b in ranges)
    return _finish(c, stream, states, new_lens, man, K, cols, Tk, sum(b - a for a, b in ranges))


def shard_rows(c, rank, world):
    """Rows (K, the reduction dimension) [rank*K/world, (rank+1)*K/world) of a compressed [K,N] weight.
    K/world must be a multiple of the tile height, so every shard starts on a tile row."""
    K, N, th, tw, Tk, Tn = _geom(c)
    if K % world or (K // world) % th:
        raise ValueError(f"K={K} cannot be cut into {world} row shards on {th}-row tile boundaries")
    per = K // world // th
    return tile_rows(c, rank * per, (rank + 1) * per)


def shard_cols(c, rank, world, parts=None):
    """Columns (N, output features) [rank*N/world, (rank+1)*N/world); N/world must be a multiple of the tile
    width.  ``parts``: widths of the blocks a concatenated projection consists of (q|k|v, gate|up); the shard
    is then the rank's slice of every block, concatenated in the same order, so that each rank holds whole
    heads of q, k and v (or matching gate and up columns)."""
    K, N, th, tw, Tk, Tn = _geom(c)
    parts = [N] if parts is None else [int(p) for p in parts]
    if sum(parts) != N:
        raise ValueError(f"parts {parts} do not add up to N={N}")
    ranges, start = [], 0
    for p in parts:
        if p % world or (p // world) % tw or start % tw:
            raise ValueError(f"a block of {p} columns cannot be cut into {world} column shards on {tw}-column tile boundaries")
        per = p // world // tw
        ranges.append((start // tw + rank * per, start // tw + (rank + 1) * per))
        start += p
    return tile_cols(c, ranges)


def can_shard_rows(K, th, world):
    return K % world == 0 and (K // world) % th == 0


def can_shard_cols(N, tw, world, parts=None):
    parts = [N] if parts is None else parts
    return all(p % world == 0 and (p // world) % tw == 0 for p in parts) and all(
        sum(parts[:i]) % tw == 0 for i in range(len(parts)))
