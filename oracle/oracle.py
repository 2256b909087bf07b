"""numpy-facing wrapper around the CPU oracle (librans_oracle.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke test and by the CPU
legs of bench.py -- never by the product package.  Each function names the
reference code the C routine behind it follows; see rans_oracle.c.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "librans_oracle.so")
_lib = None

u8p = C.POINTER(C.c_uint8)
u16p = C.POINTER(C.c_uint16)
u32p = C.POINTER(C.c_uint32)


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            from . import build as _b
            _b.build_oracle()
        _lib = C.CDLL(_SO)
        _lib.orc_rans_lut.restype = C.c_int
        _lib.orc_encode_tiled.restype = C.c_int
        _lib.orc_encode_dense.restype = C.c_int
        _lib.orc_linear.restype = C.c_int
    return _lib


def _p(a, t):
    return a.ctypes.data_as(t)


def _c(a, dt):
    a = np.ascontiguousarray(a)
    if a.dtype != dt:
        a = a.astype(dt)
    return a


def default_threads():
    return len(os.sched_getaffinity(0))


def split_bf16(raw_u16):
    """extract_exp_and_mantissa (comp_inference/comp_inference.py:10-32) on raw bf16 bits."""
    raw = _c(raw_u16, np.uint16)
    e = np.empty(raw.shape, np.uint8)
    m = np.empty(raw.shape, np.uint8)
    lib().orc_split_bf16(_p(raw, u16p), C.c_uint64(raw.size), _p(e, u8p), _p(m, u8p))
    return e, m


def merge_bf16(exp, man):
    """reconstruct_from_exp_and_mantissa (comp_inference/comp_inference.py:156-180) -> raw bf16 bits."""
    e = _c(exp, np.uint8)
    m = _c(man, np.uint8)
    out = np.empty(e.shape, np.uint16)
    lib().orc_merge_bf16(_p(e, u8p), _p(m, u8p), C.c_uint64(e.size), _p(out, u16p))
    return out


def rans_lut(plane):
    """get_rans_lut (comp_inference/comp_inference.py:183-239) -> (freqs u16[256], cdf u16[256])."""
    d = _c(plane, np.uint8).reshape(-1)
    f = np.empty(256, np.uint16)
    c = np.empty(256, np.uint16)
    rc = lib().orc_rans_lut(_p(d, u8p), C.c_uint64(d.size), _p(f, u16p), _p(c, u16p))
    if rc != 0:
        raise RuntimeError(f"orc_rans_lut failed ({rc})")
    return f, c


def build_tables(freqs, cdf):
    """Packed tables u32[256] and slot map u8[4096] (src/cuda/rans_host.cuh:476-488)."""
    f = _c(freqs, np.uint16)
    c = _c(cdf, np.uint16)
    t = np.empty(256, np.uint32)
    s = np.empty(4096, np.uint8)
    lib().orc_build_tables(_p(f, u16p), _p(c, u16p), _p(t, u32p), _p(s, u8p))
    return t, s


def effective_tile(K, N, th, tw):
    a, b = C.c_uint32(th), C.c_uint32(tw)
    lib().orc_effective_tile(C.c_uint32(K), C.c_uint32(N), C.byref(a), C.byref(b))
    return a.value, b.value


def interleave_mantissa(man, th, tw):
    """interleave_mantissas (comp_inference/comp_inference.py:35-64)."""
    m = _c(man, np.uint8)
    K, N = m.shape
    tk, tn = -(-K // th), -(-N // tw)
    out = np.empty(tk * tn * th * tw, np.uint8)
    lib().orc_interleave_mantissa(_p(m, u8p), C.c_uint32(K), C.c_uint32(N), C.c_uint32(th), C.c_uint32(tw), _p(out, u8p))
    return out


def uninterleave_mantissa(tiled, K, N, th, tw):
    """uninterleave_mantissas (comp_inference/comp_inference.py:67-93)."""
    t = _c(tiled, np.uint8).reshape(-1)
    out = np.empty((K, N), np.uint8)
    lib().orc_uninterleave_mantissa(_p(t, u8p), C.c_uint64(t.size), C.c_uint32(K), C.c_uint32(N),
                                    C.c_uint32(th), C.c_uint32(tw), _p(out, u8p))
    return out


class Tiled(dict):
    """Result of encode_tiled; keys mirror TiledTensorCompressResult (src/python_bindings.cpp:150-165)."""
    __getattr__ = dict.__getitem__


def encode_tiled(plane, freqs, cdf, th, tw, nthreads=None):
    """RansManager.compress_tiled, ILP2 layout (src/cuda/rans_ops.cu:205-410)."""
    p = _c(plane, np.uint8)
    K, N = p.shape
    th, tw = effective_tile(K, N, th, tw)
    tk, tn = -(-K // th), -(-N // tw)
    T = tk * tn
    S = T * 2 * tw
    f = _c(freqs, np.uint16)
    c = _c(cdf, np.uint16)
    states = np.empty(S, np.uint32)
    sizes = np.empty(S, np.uint32)
    offs = np.empty(T, np.uint32)
    lens = np.empty(T, np.uint32)
    sp = u8p()
    sl = C.c_uint64(0)
    rc = lib().orc_encode_tiled(_p(p, u8p), C.c_uint32(K), C.c_uint32(N), _p(f, u16p), _p(c, u16p),
                                C.c_uint32(th), C.c_uint32(tw), _p(states, u32p), _p(sizes, u32p),
                                _p(offs, u32p), _p(lens, u32p), C.byref(sp), C.byref(sl),
                                C.c_int(nthreads or default_threads()))
    if rc != 0:
        raise RuntimeError(f"orc_encode_tiled failed ({rc})")
    stream = np.ctypeslib.as_array(sp, shape=(max(sl.value, 1),))[: sl.value].copy()
    lib().orc_free(sp)
    tables, slot_map = build_tables(f, c)
    return Tiled(success=True, stream=stream, states=states, output_sizes=sizes, tables=tables, slot_map=slot_map,
                 num_streams=S, stream_len=sl.value, tile_offsets=offs, tile_max_lens=lens,
                 num_tiles_n=tn, num_tiles_k=tk, tile_height=th, tile_width=tw)


def encode_dense(plane, freqs, cdf, th, tw, nthreads=None):
    """RansManager.compress_tiled_uncoalesced (src/cuda/rans_ops.cu:74-203)."""
    p = _c(plane, np.uint8)
    K, N = p.shape
    th, tw = effective_tile(K, N, th, tw)
    tk, tn = -(-K // th), -(-N // tw)
    S = tk * tn * tw
    f = _c(freqs, np.uint16)
    c = _c(cdf, np.uint16)
    states = np.empty(S, np.uint32)
    sizes = np.empty(S, np.uint32)
    offs = np.empty(S, np.uint32)
    sp = u8p()
    sl = C.c_uint64(0)
    rc = lib().orc_encode_dense(_p(p, u8p), C.c_uint32(K), C.c_uint32(N), _p(f, u16p), _p(c, u16p),
                                C.c_uint32(th), C.c_uint32(tw), _p(states, u32p), _p(sizes, u32p),
                                _p(offs, u32p), C.byref(sp), C.byref(sl), C.c_int(nthreads or default_threads()))
    if rc != 0:
        raise RuntimeError(f"orc_encode_dense failed ({rc})")
    stream = np.ctypeslib.as_array(sp, shape=(max(sl.value, 1),))[: sl.value].copy()
    lib().orc_free(sp)
    tables, slot_map = build_tables(f, c)
    return Tiled(success=True, stream=stream, states=states, output_sizes=sizes, tables=tables, slot_map=slot_map,
                 num_streams=S, stream_len=sl.value, stream_offsets=offs,
                 num_tiles_n=tn, num_tiles_k=tk, tile_height=th, tile_width=tw)


def _dec_args(r):
    return (_p(_c(r["stream"], np.uint8), u8p), _p(_c(r["states"], np.uint32), u32p),
            _p(_c(r["tables"], np.uint32), u32p), _p(_c(r["slot_map"], np.uint8), u8p),
            _p(_c(r["tile_offsets"], np.uint32), u32p), _p(_c(r["tile_max_lens"], np.uint32), u32p))


def _keep(r):
    """Contiguous, correctly typed copies that stay alive for the duration of a call."""
    return dict(stream=_c(r["stream"], np.uint8), states=_c(r["states"], np.uint32),
                tables=_c(r["tables"], np.uint32), slot_map=_c(r["slot_map"], np.uint8),
                tile_offsets=_c(r["tile_offsets"], np.uint32), tile_max_lens=_c(r["tile_max_lens"], np.uint32))


def decode_plane(r, K, N, th, tw, nthreads=None):
    """rans_decomp_triton_tiled (comp_inference/rans_triton.py:34-168) -> u8 [K,N]."""
    k = _keep(r)
    out = np.zeros((K, N), np.uint8)
    lib().orc_decode_plane(*_dec_args(k), C.c_uint32(K), C.c_uint32(N), C.c_uint32(th), C.c_uint32(tw),
                           _p(out, u8p), C.c_int(nthreads or default_threads()))
    return out


def decode_bf16(r, mantissa_tiled, K, N, th, tw, nthreads=None):
    """rans_decompress_module_weight_bf16 (comp_inference/comp_inference.py:573-713) -> raw bf16 bits [K,N]."""
    k = _keep(r)
    m = _c(mantissa_tiled, np.uint8)
    out = np.zeros((K, N), np.uint16)
    lib().orc_decode_bf16(*_dec_args(k), _p(m, u8p), C.c_uint32(K), C.c_uint32(N), C.c_uint32(th), C.c_uint32(tw),
                          _p(out, u16p), C.c_int(nthreads or default_threads()))
    return out


def decode_plane_dense(r, K, N, th, tw, nthreads=None):
    """Dense-layout decode (comp_inference/linear_triton.py:1044-1186 stream walk) -> u8 [K,N]."""
    stream = _c(r["stream"], np.uint8)
    states = _c(r["states"], np.uint32)
    sizes = _c(r["output_sizes"], np.uint32)
    offs = _c(r["stream_offsets"], np.uint32)
    tables = _c(r["tables"], np.uint32)
    sm = _c(r["slot_map"], np.uint8)
    out = np.zeros((K, N), np.uint8)
    lib().orc_decode_plane_dense(_p(stream, u8p), _p(states, u32p), _p(sizes, u32p), _p(offs, u32p),
                                 _p(tables, u32p), _p(sm, u8p), C.c_uint32(K), C.c_uint32(N),
                                 C.c_uint32(th), C.c_uint32(tw), _p(out, u8p), C.c_int(nthreads or default_threads()))
    return out


def embedding(ids, r, mantissa_tiled, K, N, th, tw, nthreads=None):
    """fused_rans_embedding_triton (comp_inference/embedding_triton.py:170-330) -> raw bf16 bits [n, N]."""
    k = _keep(r)
    m = _c(mantissa_tiled, np.uint8)
    i = _c(np.asarray(ids).reshape(-1), np.int64)
    out = np.zeros((i.size, N), np.uint16)
    lib().orc_embedding(_p(i, C.POINTER(C.c_int64)), C.c_uint64(i.size), *_dec_args(k), _p(m, u8p),
                        C.c_uint32(K), C.c_uint32(N), C.c_uint32(th), C.c_uint32(tw), _p(out, u16p),
                        C.c_int(nthreads or default_threads()))
    return out


def linear(x_bf16_bits, r, mantissa_tiled, K, N, th, tw, transposed=False, nthreads=None):
    """decompress-then-matmul in fp32 (tests/test_mat_mul.py:186-238).

    transposed=False: x [M,K] -> y [M,N] (linear_triton.py:229-552 semantics);
    transposed=True:  x [M,N] -> y [M,K] (transposed_linear_triton.py:187-435 semantics).
    """
    k = _keep(r)
    m = _c(mantissa_tiled, np.uint8)
    x = _c(x_bf16_bits, np.uint16)
    M = x.shape[0]
    y = np.zeros((M, K if transposed else N), np.float32)
    rc = lib().orc_linear(_p(x, u16p), C.c_uint32(M), *_dec_args(k), _p(m, u8p), C.c_uint32(K), C.c_uint32(N),
                          C.c_uint32(th), C.c_uint32(tw), C.c_int(1 if transposed else 0),
                          _p(y, C.POINTER(C.c_float)), C.c_int(nthreads or default_threads()))
    if rc != 0:
        raise RuntimeError("orc_linear failed")
    return y


def compress_bf16(raw_u16_KN, th, tw, nthreads=None):
    """Whole rans_compress_module_weight_bf16 path on raw bf16 bits already laid out [K,N]
    (comp_inference/comp_inference.py:344-502): split, LUT, ILP2 encode, mantissa tiling."""
    e, m = split_bf16(raw_u16_KN)
    f, c = rans_lut(e)
    r = encode_tiled(e, f, c, th, tw, nthreads)
    r["mantissa"] = interleave_mantissa(m, r.tile_height, r.tile_width)
    r["freqs"], r["cdf"] = f, c
    return r


# ---- legacy flat layout, the reference encoder's 512-row segments (pure numpy, small cases) -----------------
def encode_legacy_segments(plane, freqs, cdf, seg_rows=512):
    """Stream g = seg * cols + col codes rows [seg * seg_rows, + seg_rows) of column col, last row first, so
    that the decoder (comp_inference/rans_triton.py:171-241) meets them first row first; byte j of stream g
    sits at j * num_streams + g and the decoder reads from sizes[g] - 1 downwards.  Encoder step as in
    src/cuda/rans_kernels.cuh:393-509: renormalise while x >= ((L >> 12) << 8) * freq, then
    x = (x // freq << 12) + x % freq + cdf.  Returns (stream u8, states u32, sizes u32)."""
    p = _c(plane, np.uint8)
    rows, cols = p.shape
    f = np.asarray(freqs, np.uint64)
    c = np.asarray(cdf, np.uint64)
    segs = -(-rows // seg_rows)
    S = segs * cols
    x = np.full(S, 1 << 16, np.uint64)
    emitted = [[] for _ in range(S)]
    for i in range(seg_rows - 1, -1, -1):
        for seg in range(segs):
            r = seg * seg_rows + i
            if r >= rows:
                continue
            for col in range(cols):
                g = seg * cols + col
                s = int(p[r, col])
                fs, cs, xs = int(f[s]), int(c[s]), int(x[g])
                lim = ((1 << 16) >> 12 << 8) * fs
                while xs >= lim:
                    emitted[g].append(xs & 0xFF)
                    xs >>= 8
                x[g] = ((xs // fs) << 12) + xs % fs + cs
    sizes = np.array([len(e) for e in emitted], np.uint32)
    stream = np.zeros(int(sizes.max(initial=0)) * S, np.uint8)
    for g, e in enumerate(emitted):
        if e:
            stream[np.arange(len(e)) * S + g] = e
    return stream, x.astype(np.uint32), sizes


def decode_legacy_segments(stream, states, sizes, rows, cols, freqs, cdf, seg_rows=512):
    """Inverse of encode_legacy_segments, following the reference's decoder loop
    (comp_inference/rans_triton.py:199-241): symbol from the 12 low bits of the state, state update from the
    symbol's frequency and cumulative count, at most two bytes per symbol while the state is below 2^16."""
    t, slot_map = build_tables(freqs, cdf)
    S = len(states)
    out = np.zeros((rows, cols), np.uint8)
    for g in range(S):
        seg, col = divmod(g, cols)
        x, off = int(states[g]), int(sizes[g]) - 1
        for i in range(min(seg_rows, rows - seg * seg_rows)):
            slot = x & 4095
            s = int(slot_map[slot])
            out[seg * seg_rows + i, col] = s
            fs, cs = int(t[s]) & 0xFFFF, int(t[s]) >> 16
            x = fs * (x >> 12) + slot - cs
            for _ in range(2):
                if x < (1 << 16) and off >= 0:
                    x = (x << 8) | int(stream[off * S + g])
                    off -= 1
    return out
