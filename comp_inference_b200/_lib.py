"""ctypes binding of libci_b200.so (the C ABI declared in include/comp_inference_b200.h).

The shared library is the only compute backend of this package.  If it is
missing or cannot be loaded, every operation raises; nothing falls back to
PyTorch or to the CPU.
"""
import ctypes as C
import os
import weakref

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "csrc", "libci_b200.so")

u8p = C.POINTER(C.c_uint8)
u16p = C.POINTER(C.c_uint16)
u32p = C.POINTER(C.c_uint32)
u64p = C.POINTER(C.c_uint64)
i64p = C.POINTER(C.c_int64)


class TiledWeight(C.Structure):
    """struct ci_tiled_weight"""
    _fields_ = [("stream", C.c_void_p), ("states", C.c_void_p), ("tables", C.c_void_p), ("slot_map", C.c_void_p),
                ("tile_offsets", C.c_void_p), ("tile_max_lens", C.c_void_p), ("mantissa", C.c_void_p),
                ("lut", C.c_void_p), ("stream_len", C.c_uint64), ("K", C.c_uint32), ("N", C.c_uint32),
                ("tile_h", C.c_uint32), ("tile_w", C.c_uint32), ("max_tile_len", C.c_uint32), ("reserved", C.c_uint32)]


class DenseWeight(C.Structure):
    """struct ci_dense_weight"""
    _fields_ = [("stream", C.c_void_p), ("states", C.c_void_p), ("stream_sizes", C.c_void_p),
                ("stream_offsets", C.c_void_p), ("tables", C.c_void_p), ("slot_map", C.c_void_p),
                ("mantissa", C.c_void_p), ("lut", C.c_void_p), ("stream_len", C.c_uint64), ("K", C.c_uint32),
                ("N", C.c_uint32), ("tile_h", C.c_uint32), ("tile_w", C.c_uint32)]


# Every entry point of the header, with its argument types.  tests check this
# table against the header and against the symbols the library exports.
_V, _S = C.c_void_p, C.c_void_p
SIGNATURES = {
    "ci_abi_version": (C.c_int, []),
    "ci_last_error": (C.c_char_p, []),
    "ci_device_info": (C.c_int, [C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "ci_workspace_status_word": (C.c_void_p, [_V]),
    "ci_status": (C.c_int, [_V, u32p, C.c_int, _S]),
    "ci_validate_tiled_metadata": (C.c_int, [_V, _V, _V, _V, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint32,
                                             C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32]),
    "ci_build_tables": (C.c_int, [_V, _V, _V, _V]),
    "ci_prepare_lut": (C.c_int, [_V, _V, _V, _S]),
    "ci_split_bf16": (C.c_int, [_V, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, _V, _V, _V, _V, _S]),
    "ci_histogram_u8": (C.c_int, [_V, C.c_uint64, _V, _S]),
    "ci_normalize_freqs": (C.c_int, [_V, _V, _V]),
    "ci_untile_mantissa": (C.c_int, [_V, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, _V, _S]),
    "ci_encode_tiled_sizes": (C.c_int, [_V, C.c_uint32, C.c_uint32, _V, _V, C.c_uint32, C.c_uint32, _V, _V, _V, _V,
                                        u64p, _S]),
    "ci_encode_tiled_write": (C.c_int, [_V, C.c_uint32, C.c_uint32, _V, _V, C.c_uint32, C.c_uint32, _V, _V, _V, _V,
                                        C.c_uint64, _S]),
    "ci_encode_dense_sizes": (C.c_int, [_V, C.c_uint32, C.c_uint32, _V, _V, C.c_uint32, C.c_uint32, _V, _V, _V,
                                        u64p, _S]),
    "ci_encode_dense_write": (C.c_int, [_V, C.c_uint32, C.c_uint32, _V, _V, C.c_uint32, C.c_uint32, _V, _V,
                                        C.c_uint64, _S]),
    "ci_decode_plane": (C.c_int, [C.POINTER(TiledWeight), _V, _S]),
    "ci_decode_bf16": (C.c_int, [C.POINTER(TiledWeight), _V, _S]),
    "ci_decode_plane_dense": (C.c_int, [C.POINTER(DenseWeight), _V, _S]),
    "ci_decode_bf16_dense": (C.c_int, [C.POINTER(DenseWeight), _V, _S]),
    "ci_linear_workspace_bytes": (C.c_size_t, [C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32]),
    "ci_linear": (C.c_int, [C.POINTER(TiledWeight), _V, C.c_int64, C.c_uint32, _V, _V, C.c_int64, _V, C.c_size_t,
                            C.c_uint32, _S]),
    "ci_linear_route": (C.c_int, [C.POINTER(TiledWeight), C.c_uint32]),
    "ci_linear_static_max_bytes": (C.c_size_t, []),
    "ci_linear_static": (C.c_int, [C.POINTER(TiledWeight), _V, C.c_int64, C.c_uint32, _V, _V, C.c_int64, _S]),
    "ci_linear_static_status": (C.c_int, [u32p, C.c_int, _S]),
    "ci_linear_transposed": (C.c_int, [C.POINTER(TiledWeight), _V, C.c_int64, C.c_uint32, _V, _V, C.c_int64, _V,
                                       C.c_size_t, _S]),
    "ci_embedding": (C.c_int, [C.POINTER(TiledWeight), _V, C.c_uint64, _V, C.c_int64, _S]),
    "ci_linear_dense": (C.c_int, [C.POINTER(DenseWeight), _V, C.c_int64, C.c_uint32, _V, _V, C.c_int64, _V,
                                  C.c_size_t, C.c_uint32, _S]),
    "ci_embedding_dense": (C.c_int, [C.POINTER(DenseWeight), _V, C.c_uint64, _V, C.c_int64, _S]),
    "ci_linear_transposed_dense": (C.c_int, [C.POINTER(DenseWeight), _V, C.c_int64, C.c_uint32, _V, _V, C.c_int64, _V,
                                             C.c_size_t, _S]),
    "ci_decode_legacy": (C.c_int, [_V, C.c_uint64, _V, _V, C.c_uint32, C.c_uint64, _V, _V, _V, _S]),
    "ci_encode_legacy_sizes": (C.c_int, [_V, C.c_uint64, C.c_uint32, _V, _V, _V, _V, _S]),
    "ci_encode_legacy_write": (C.c_int, [_V, C.c_uint64, C.c_uint32, _V, _V, _V, C.c_uint64, _S]),
    "ci_decode_legacy_segments": (C.c_int, [_V, C.c_uint64, _V, _V, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, _V,
                                            _V, _V, _S]),
    "ci_encode_legacy_segments_sizes": (C.c_int, [_V, C.c_uint32, C.c_uint32, C.c_uint32, _V, _V, _V, _V, _S]),
    "ci_encode_legacy_segments_write": (C.c_int, [_V, C.c_uint32, C.c_uint32, C.c_uint32, _V, _V, _V, C.c_uint64, _S]),
    "ci_add_rmsnorm": (C.c_int, [_V, C.c_int64, _V, C.c_int64, _V, C.c_float, C.c_uint32, C.c_uint32, _V, C.c_int64, _V,
                                 C.c_int64, _S]),
    "ci_rope_kv": (C.c_int, [_V, C.c_int64, _V, C.c_int64, _V, C.c_int64, _V, _V, _V, C.c_uint32, C.c_uint32, C.c_uint32,
                             C.c_uint32, C.c_uint32, _V, _V, _V, _S]),
    "ci_decode_attention_workspace_bytes": (C.c_size_t, [C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32]),
    "ci_decode_attention": (C.c_int, [_V, _V, _V, _V, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
                                      C.c_float, _V, C.c_size_t, _V, C.c_int64, _S]),
    "ci_silu_mul": (C.c_int, [_V, C.c_int64, _V, C.c_int64, C.c_uint32, C.c_uint32, _V, C.c_int64, _S]),
    "ci_allreduce_buffer_bytes": (C.c_size_t, [C.c_uint32, C.c_uint32]),
    "ci_allreduce_counter_bytes": (C.c_size_t, []),
    "ci_linear_allreduce_counter_bytes": (C.c_size_t, []),
    "ci_linear_allreduce_qualifies": (C.c_int, [C.POINTER(TiledWeight), C.c_uint32]),
    "ci_allreduce_set_poll_limit": (None, [C.c_uint32]),
    "ci_linear_allreduce": (C.c_int, [C.POINTER(TiledWeight), _V, C.c_int64, C.c_uint32, _V, _V, _V, C.c_size_t, _V,
                                      C.c_uint32, _V, C.c_uint32, C.c_uint32, _V, _S]),
    "ci_allgather_oneshot": (C.c_int, [_V, _V, C.c_uint32, C.c_uint32, C.c_uint32, _V, _V, C.c_uint32, C.c_uint32, _V, _S]),
    "ci_allreduce_oneshot": (C.c_int, [_V, _V, C.c_uint32, C.c_uint32, _V, _V, C.c_uint32, C.c_uint32, _V, _S]),
}

_lib = None


def load():
    """Returns the loaded library; raises RuntimeError if it is not there."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python comp_inference_b200/csrc/build.py` "
            "(needs nvcc with sm_100a support). This package has no other backend.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError here = library older than the header
        fn.restype = res
        fn.argtypes = args
    if lib.ci_abi_version() != 1:
        raise RuntimeError(f"libci_b200.so has ABI version {lib.ci_abi_version()}, expected 1")
    _lib = lib
    return lib


def check(rc):
    if rc != 0:
        msg = load().ci_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"comp_inference_b200: {msg} (code {rc})")


def stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


def require_cuda(t, name):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: this package has no CPU path")
    return t


def as_u32(t, name):
    """32-bit metadata arrives as uint32 or int32 (the reference casts back and forth); same bits."""
    if t.dtype not in (torch.uint32, torch.int32):
        raise RuntimeError(f"{name} must be uint32 or int32, got {t.dtype}")
    return t.contiguous()


def as_u8(t, name):
    if t.dtype != torch.uint8:
        raise RuntimeError(f"{name} must be uint8, got {t.dtype}")
    return t.contiguous()


# ---- prepared decode tables, one per (tables, slot_map) pair -----------------
_lut_cache = {}


def prepared_lut(tables, slot_map):
    """Device uint32[4096] merged decode table for this tables/slot_map pair (cached per tensor object)."""
    key = (tables.data_ptr(), slot_map.data_ptr())
    hit = _lut_cache.get(key)
    if hit is not None:
        ref_t, ref_s, ver, lut = hit
        if ref_t() is tables and ref_s() is slot_map and ver == (tables._version, slot_map._version):
            return lut
    lut = torch.empty(4096, dtype=torch.int32, device=tables.device)
    check(load().ci_prepare_lut(ptr(tables), ptr(slot_map), ptr(lut), stream()))
    if len(_lut_cache) > 4096:
        _lut_cache.clear()
    _lut_cache[key] = (weakref.ref(tables), weakref.ref(slot_map), (tables._version, slot_map._version), lut)
    return lut


_maxlen_cache = {}


def max_tile_len(tile_max_lens):
    """Largest entry of tile_max_lens (one device->host read per tensor object, then cached); the
    staged kernels size their shared-memory byte window with it."""
    key = tile_max_lens.data_ptr()
    hit = _maxlen_cache.get(key)
    if hit is not None and hit[0]() is tile_max_lens and hit[1] == tile_max_lens._version:
        return hit[2]
    v = int(tile_max_lens.view(torch.int32).max().item()) if tile_max_lens.numel() else 0
    if len(_maxlen_cache) > 4096:
        _maxlen_cache.clear()
    _maxlen_cache[key] = (weakref.ref(tile_max_lens), tile_max_lens._version, v)
    return v


# ---- split-K / stream-K workspaces ---------------------------------------------------------
# One zero-initialised buffer per (device, CUDA stream): kernels of one stream run in order and leave the
# ticket counters zeroed, so they can share; two streams may overlap on the GPU and must not (the
# reference keeps one global buffer for every layer and stream, comp_inference/pytorch_runtime.py:386-394).
# A buffer that was handed out is never freed: a CUDA graph captured earlier keeps replaying into the
# address it saw, so when a larger one is needed the old tensor is retired, not dropped.
_workspaces = {}
_retired = []
_MIN_WORKSPACE = 8 << 20


def workspace(device, nbytes):
    device = torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        if ws is not None:
            _retired.append((key[0], ws))
        ws = torch.zeros(max(int(nbytes), _MIN_WORKSPACE), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def reserve_workspace(device, nbytes):
    """Sizes the current stream's workspace up front (e.g. for the largest M x N a model will see) so that
    no later call has to replace it."""
    return workspace(device, nbytes)


def _status_words(device):
    device = torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    bufs = [ws for (dev, _), ws in _workspaces.items() if dev == device]
    bufs += [ws for dev, ws in _retired if dev == device]
    return bufs


def kernel_status(device):
    """First non-zero status word among this device's workspaces (0 = fine): set by the staged kernels when a
    bounded wait ran out or tile metadata contradicted the descriptor.  Reading it synchronises with the device."""
    for ws in _status_words(device):
        v = int(ws[4095 * 4:4096 * 4].view(torch.int32).item())
        if v:
            return v
    return 0


def check_status(device=None, clear=True):
    """Raises RuntimeError (CI_E_DEVICE) if any kernel that used one of this device's workspaces reported an
    error through its status word; call it wherever the host waits for results anyway.  Goes through the C ABI
    (ci_status), which waits for the current stream."""
    lib = load()
    device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
    for ws in _status_words(device):
        word = lib.ci_workspace_status_word(ptr(ws))
        check(lib.ci_status(C.c_void_p(word), None, 1 if clear else 0, stream()))


def validate_compressed(c, K=None, N=None, th=None, tw=None, max_tile_len=0):
    """ci_validate_tiled_metadata on a dict of package tensors (any device; copied to the host here).
    Raises RuntimeError naming the first inconsistent entry."""
    import numpy as np
    if K is None:
        K, N = c["shape"]
        th, tw = c["tile_height"], c["tile_width"]
    host = lambda t, dt: np.ascontiguousarray(t.detach().cpu().contiguous().view(dt).numpy())
    off = host(c["rans_exp_tile_offsets"], torch.int32).view(np.uint32)
    lens = host(c["rans_exp_tile_max_lens"], torch.int32).view(np.uint32)
    tables = host(c["rans_exp_tables"], torch.int32).view(np.uint32) if "rans_exp_tables" in c else None
    slot = host(c["rans_exp_slot_map"], torch.uint8) if "rans_exp_slot_map" in c else None
    tiles = -(-int(K) // int(th)) * -(-int(N) // int(tw))
    if off.size != tiles or lens.size != tiles:
        raise RuntimeError(f"comp_inference_b200: tile_offsets / tile_max_lens have {off.size} / {lens.size} "
                           f"entries, {tiles} expected (code -1)")
    man = c.get("rans_man_raw")
    check(load().ci_validate_tiled_metadata(
        off.ctypes.data, lens.ctypes.data, tables.ctypes.data if tables is not None else None,
        slot.ctypes.data if slot is not None else None, int(c["rans_exp_stream"].numel()),
        int(c["rans_exp_states"].numel()), int(man.numel()) if man is not None else 0, int(K), int(N), int(th),
        int(tw), int(max_tile_len)))


def tiled_weight(stream_t, states, tables, slot_map, tile_offsets, tile_max_lens, mantissa, K, N, th, tw, lut=None,
                 keep=None, want_max=False):
    """Fills a ci_tiled_weight from CUDA tensors; returns (struct, tensors that must stay alive)."""
    require_cuda(stream_t, "compressed stream")
    st = as_u8(stream_t, "compressed stream")
    sts = as_u32(require_cuda(states, "states"), "states")
    tb = as_u32(require_cuda(tables, "tables"), "tables")
    sm = as_u8(require_cuda(slot_map, "slot_map"), "slot_map")
    off = as_u32(require_cuda(tile_offsets, "tile_offsets"), "tile_offsets")
    ml = as_u32(require_cuda(tile_max_lens, "tile_max_lens"), "tile_max_lens")
    man = as_u8(require_cuda(mantissa, "mantissas"), "mantissas") if mantissa is not None else None
    tiles = -(-K // th) * -(-N // tw)
    if sts.numel() != tiles * 2 * tw:
        raise ValueError(f"Initial states size mismatch. Expected {tiles * 2 * tw}")     # rans_triton.py:141-144
    if off.numel() != tiles or ml.numel() != tiles:
        raise ValueError(f"tile_offsets / tile_max_lens must have {tiles} entries")
    if man is not None and man.numel() < tiles * th * tw:
        raise ValueError(f"mantissa plane has {man.numel()} bytes, {tiles * th * tw} expected")
    if lut is None:
        lut = prepared_lut(tb, sm) if (tb is tables and sm is slot_map) else None
    deepest = max_tile_len(tile_max_lens) if (want_max and ml is tile_max_lens) else 0
    w = TiledWeight(ptr(st), ptr(sts), ptr(tb), ptr(sm), ptr(off), ptr(ml), ptr(man), ptr(lut), st.numel(),
                    K, N, th, tw, deepest, 0)
    return w, (st, sts, tb, sm, off, ml, man, lut, keep)


def dense_weight(stream_t, states, sizes, offsets, tables, slot_map, mantissa, K, N, th, tw):
    require_cuda(stream_t, "compressed stream")
    st = as_u8(stream_t, "compressed stream")
    sts = as_u32(require_cuda(states, "states"), "states")
    sz = as_u32(require_cuda(sizes, "stream_sizes"), "stream_sizes")
    off = as_u32(require_cuda(offsets, "stream_offsets"), "stream_offsets")
    tb = as_u32(require_cuda(tables, "tables"), "tables")
    sm = as_u8(require_cuda(slot_map, "slot_map"), "slot_map")
    man = as_u8(require_cuda(mantissa, "mantissas"), "mantissas") if mantissa is not None else None
    n = -(-K // th) * -(-N // tw) * tw
    if sts.numel() != n or sz.numel() != n or off.numel() != n:
        raise ValueError(f"dense layout needs {n} states / sizes / offsets")
    lut = prepared_lut(tb, sm) if (tb is tables and sm is slot_map) else None
    w = DenseWeight(ptr(st), ptr(sts), ptr(sz), ptr(off), ptr(tb), ptr(sm), ptr(man), ptr(lut), st.numel(), K, N, th, tw)
    return w, (st, sts, sz, off, tb, sm, man, lut)
