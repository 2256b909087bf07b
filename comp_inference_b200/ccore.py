"""Drop-in for the reference's extension module ``comp_inference.ccore``
(src/python_bindings.cpp): same names, argument meaning, result attributes and
error behaviour, served by the C ABI in libci_b200.so.

Differences that matter to a caller:
  * the encoder runs wholly on the GPU and writes the packed stream directly;
    there is no host-side repack (src/cuda/rans_ops.cu:328-370);
  * tile sizes larger than the matrix are halved *before* encoding (the
    reference halves them afterwards, src/cuda/rans_ops.cu:219-223, which leaves
    a result no decoder can read);
  * lanes of a partial last column tile get state 2^16 / size 0 instead of
    uninitialised memory (src/cuda/rans_kernels.cuh:99-100).
"""
import ctypes as C

import numpy as np
import torch

from . import _lib


def _device():
    if not torch.cuda.is_available():
        raise RuntimeError("comp_inference_b200.ccore needs a CUDA device: the rANS encoder has no CPU path")
    return torch.device("cuda", torch.cuda.current_device())


def _as_u16_host(t, name):
    if isinstance(t, torch.Tensor):
        t = t.detach().cpu()
        if t.dtype != torch.uint16:
            t = t.to(torch.int32).to(torch.uint16) if t.dtype != torch.int16 else t.view(torch.uint16)
        a = t.contiguous().numpy()
    else:
        a = np.ascontiguousarray(t)
    a = a.astype(np.uint16, copy=False).reshape(-1)
    if a.size != 256:
        raise RuntimeError(f"{name} must have 256 entries, got {a.size}")
    return np.ascontiguousarray(a)


def effective_tile(K, N, tile_height, tile_width):
    while tile_height > K and tile_height > 1:
        tile_height //= 2
    while tile_width > N and tile_width > 1:
        tile_width //= 2
    return tile_height, tile_width


class TiledTensorCompressResult:
    """Mirror of TiledTensorCompressResult (src/python_bindings.cpp:150-165): CPU tensors, owned copies."""

    def __init__(self, **kw):
        self.__dict__.update(kw)


class UncoalescedTiledTensorCompressResult(TiledTensorCompressResult):
    """Mirror of UncoalescedTiledTensorCompressResult (src/python_bindings.cpp:167-190)."""


class TensorCompressResult(TiledTensorCompressResult):
    """Mirror of TensorCompressResult (src/python_bindings.cpp:140-148), legacy flat layout."""


def _tables_host(freqs, cdf):
    tables = np.empty(256, np.uint32)
    slot_map = np.empty(4096, np.uint8)
    _lib.check(_lib.load().ci_build_tables(freqs.ctypes.data, cdf.ctypes.data, tables.ctypes.data, slot_map.ctypes.data))
    return torch.from_numpy(tables), torch.from_numpy(slot_map)


class RansManager:
    """ccore.RansManager (src/python_bindings.cpp:222-471, src/cpp/rans.hpp:9-96)."""

    def __init__(self, max_data_hint: int = 0):
        self.max_data_hint = int(max_data_hint)
        _lib.load()

    # -- ILP2 tiled layout ------------------------------------------------------
    def compress_tiled(self, data, freqs, cdf, tile_height, tile_width, _keep_on_device=False):
        """data: uint8 [K,N] (CPU or CUDA); freqs/cdf: uint16[256]; returns TiledTensorCompressResult."""
        dev = _device()
        if data.dtype != torch.uint8:
            raise RuntimeError("expected scalar type Byte")                    # data_ptr<uint8_t>() in the reference
        K = int(data.shape[0])
        N = int(data.shape[1]) if data.dim() > 1 else 1
        if data.numel() != K * N:
            raise RuntimeError("Input size mismatch in tiled compression")   # src/cuda/rans_host.cuh:462-467
        if tile_height % 16 != 0:
            raise RuntimeError("Invalid tile height")                        # src/cuda/rans_host.cuh:440-445
        f = _as_u16_host(freqs, "freqs")
        c = _as_u16_host(cdf, "cdf")
        th, tw = effective_tile(K, N, int(tile_height), int(tile_width))
        plane = data.to(dev, non_blocking=True).contiguous()
        tk, tn = -(-K // th), -(-N // tw)
        T, S = tk * tn, tk * tn * 2 * tw
        states = torch.empty(S, dtype=torch.uint32, device=dev)
        sizes = torch.empty(S, dtype=torch.uint32, device=dev)
        offs = torch.empty(T, dtype=torch.uint32, device=dev)
        lens = torch.empty(T, dtype=torch.uint32, device=dev)
        n = C.c_uint64(0)
        lib = _lib.load()
        _lib.check(lib.ci_encode_tiled_sizes(_lib.ptr(plane), K, N, f.ctypes.data, c.ctypes.data, th, tw,
                                             _lib.ptr(states), _lib.ptr(sizes), _lib.ptr(offs), _lib.ptr(lens),
                                             C.byref(n), _lib.stream()))
        stream = torch.empty(n.value, dtype=torch.uint8, device=dev)
        _lib.check(lib.ci_encode_tiled_write(_lib.ptr(plane), K, N, f.ctypes.data, c.ctypes.data, th, tw,
                                             _lib.ptr(sizes), _lib.ptr(offs), _lib.ptr(lens), _lib.ptr(stream),
                                             n.value, _lib.stream()))
        tables, slot_map = _tables_host(f, c)
        mv = (lambda t: t) if _keep_on_device else (lambda t: t.cpu())
        if _keep_on_device:
            tables, slot_map = tables.to(dev), slot_map.to(dev)
        return TiledTensorCompressResult(
            success=True, stream=mv(stream), states=mv(states), tables=tables, slot_map=slot_map,
            output_sizes=mv(sizes), num_streams=S, stream_len=int(n.value), tile_offsets=mv(offs),
            tile_max_lens=mv(lens), num_tiles_n=tn, num_tiles_k=tk, tile_height=th, tile_width=tw)

    # -- dense ("uncoalesced") layout ----------------------------------------------
    def compress_tiled_uncoalesced(self, data, freqs, cdf, tile_height, tile_width, _keep_on_device=False):
        dev = _device()
        if data.dtype != torch.uint8:
            raise RuntimeError("expected scalar type Byte")
        K = int(data.shape[0])
        N = int(data.shape[1]) if data.dim() > 1 else 1
        if tile_height % 16 != 0:
            raise RuntimeError("Invalid tile height")
        f = _as_u16_host(freqs, "freqs")
        c = _as_u16_host(cdf, "cdf")
        th, tw = effective_tile(K, N, int(tile_height), int(tile_width))
        plane = data.to(dev, non_blocking=True).contiguous()
        tk, tn = -(-K // th), -(-N // tw)
        S = tk * tn * tw
        states = torch.empty(S, dtype=torch.uint32, device=dev)
        sizes = torch.empty(S, dtype=torch.uint32, device=dev)
        offs = torch.empty(S, dtype=torch.uint32, device=dev)
        n = C.c_uint64(0)
        lib = _lib.load()
        _lib.check(lib.ci_encode_dense_sizes(_lib.ptr(plane), K, N, f.ctypes.data, c.ctypes.data, th, tw,
                                             _lib.ptr(states), _lib.ptr(sizes), _lib.ptr(offs), C.byref(n),
                                             _lib.stream()))
        stream = torch.empty(n.value, dtype=torch.uint8, device=dev)
        _lib.check(lib.ci_encode_dense_write(_lib.ptr(plane), K, N, f.ctypes.data, c.ctypes.data, th, tw,
                                             _lib.ptr(offs), _lib.ptr(stream), n.value, _lib.stream()))
        tables, slot_map = _tables_host(f, c)
        mv = (lambda t: t) if _keep_on_device else (lambda t: t.cpu())
        if _keep_on_device:
            tables, slot_map = tables.to(dev), slot_map.to(dev)
        return UncoalescedTiledTensorCompressResult(
            success=True, stream=mv(stream), states=mv(states), tables=tables, slot_map=slot_map,
            output_sizes=mv(sizes), num_streams=S, stream_len=int(n.value), stream_offsets=mv(offs),
            num_tiles_n=tn, num_tiles_k=tk, tile_height=th, tile_width=tw)


def _legacy_compress(self, data, freqs, cdf, min_block_size=512):
    """RansManager.compress (src/python_bindings.cpp:225-299): legacy flat layout.  Accepts a numpy array or
    a tensor (CPU or CUDA), returns CPU tensors like the reference.  Stream count as the reference chooses it
    (src/cuda/rans_host.cuh:167-186): ceil(rows / min_block_size) * columns; symbol g + i * num_streams belongs
    to stream g, the assignment its decoder inverts."""
    import numpy as np
    dev = _device()
    t = torch.from_numpy(np.ascontiguousarray(data)) if isinstance(data, np.ndarray) else data
    if t.dtype != torch.uint8:
        raise RuntimeError("expected scalar type Byte")
    rows = int(t.shape[0]) if t.dim() > 0 else 1
    cols = int(t.shape[1]) if t.dim() > 1 else 1
    n = t.numel()
    if n == 0:
        raise RuntimeError("empty input")
    f = _as_u16_host(freqs, "freqs")
    c = _as_u16_host(cdf, "cdf")
    S = max(1, -(-rows // max(1, int(min_block_size))) * cols)
    flat = t.to(dev).contiguous().view(-1)
    states = torch.empty(S, dtype=torch.uint32, device=dev)
    sizes = torch.empty(S, dtype=torch.uint32, device=dev)
    lib = _lib.load()
    _lib.check(lib.ci_encode_legacy_sizes(_lib.ptr(flat), n, S, f.ctypes.data, c.ctypes.data, _lib.ptr(states),
                                          _lib.ptr(sizes), _lib.stream()))
    max_len = int(sizes.view(torch.int32).max().item())
    stream = torch.empty(max_len * S, dtype=torch.uint8, device=dev)
    _lib.check(lib.ci_encode_legacy_write(_lib.ptr(flat), n, S, f.ctypes.data, c.ctypes.data, _lib.ptr(stream),
                                          stream.numel(), _lib.stream()))
    tables, slot_map = _tables_host(f, c)
    return TensorCompressResult(success=True, stream=stream.cpu(), states=states.cpu().view(torch.int32),
                                sizes=sizes.cpu().view(torch.int32), tables=tables, slot_map=slot_map,
                                checkpoints=torch.empty(0, dtype=torch.uint64), num_streams=S,
                                stream_len=int(stream.numel()))


def _legacy_decompress_into(self, stream, states, sizes, num_streams, freqs, cdf, output_buffer):
    """RansManager.decompress_into (src/python_bindings.cpp:438-470): decodes into the caller's buffer
    (numpy array or tensor, CPU or CUDA); returns the kernel time in milliseconds."""
    import numpy as np
    dev = _device()
    as_t = lambda a: torch.from_numpy(np.ascontiguousarray(a)) if isinstance(a, np.ndarray) else a
    f = _as_u16_host(freqs, "freqs")
    c = _as_u16_host(cdf, "cdf")
    tables, slot_map = _tables_host(f, c)
    out_t = as_t(output_buffer) if not isinstance(output_buffer, np.ndarray) else torch.from_numpy(output_buffer)
    d_out = out_t if out_t.is_cuda else torch.empty(out_t.numel(), dtype=torch.uint8, device=dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    decompress(as_t(stream).to(dev), as_t(states).to(dev), as_t(sizes).to(dev), int(num_streams), tables.to(dev),
               slot_map.to(dev), d_out.view(-1))
    e1.record()
    e1.synchronize()
    if not out_t.is_cuda:
        out_t.view(-1).copy_(d_out.cpu())
    return e0.elapsed_time(e1)


def _legacy_decompress(self, stream, states, sizes, num_streams, output_len, freqs, cdf):
    """RansManager.decompress (src/python_bindings.cpp:399-436): returns (output, kernel ms); the output is a
    numpy array for numpy input, else a uint8 tensor on the stream's device."""
    import numpy as np
    if isinstance(stream, np.ndarray):
        out = np.empty(int(output_len), dtype=np.uint8)
    else:
        out = torch.empty(int(output_len), dtype=torch.uint8, device=stream.device)
    ms = _legacy_decompress_into(self, stream, states, sizes, num_streams, freqs, cdf, out)
    return out, ms


def _legacy_compress_segments(self, data, freqs, cdf, seg_rows=512):
    """The legacy layout with the stream assignment of the reference's own legacy encoder
    (src/cuda/rans_kernels.cuh:393-509): stream seg * width + col codes rows [seg * seg_rows, + seg_rows) of
    column col of a 2-D uint8 tensor; this is what ``rans_decomp_triton`` (comp_inference/rans_triton.py:243-271,
    fixed seg_rows = 512) decodes.  Same result type as ``compress``."""
    dev = _device()
    t = torch.from_numpy(np.ascontiguousarray(data)) if isinstance(data, np.ndarray) else data
    if t.dtype != torch.uint8 or t.dim() != 2 or t.numel() == 0:
        raise RuntimeError("expected a non-empty 2-D uint8 tensor")
    rows, cols = int(t.shape[0]), int(t.shape[1])
    f = _as_u16_host(freqs, "freqs")
    c = _as_u16_host(cdf, "cdf")
    S = -(-rows // int(seg_rows)) * cols
    plane = t.to(dev).contiguous()
    states = torch.empty(S, dtype=torch.uint32, device=dev)
    sizes = torch.empty(S, dtype=torch.uint32, device=dev)
    lib = _lib.load()
    _lib.check(lib.ci_encode_legacy_segments_sizes(_lib.ptr(plane), rows, cols, int(seg_rows), f.ctypes.data,
                                                   c.ctypes.data, _lib.ptr(states), _lib.ptr(sizes), _lib.stream()))
    max_len = int(sizes.view(torch.int32).max().item())
    stream = torch.empty(max_len * S, dtype=torch.uint8, device=dev)
    _lib.check(lib.ci_encode_legacy_segments_write(_lib.ptr(plane), rows, cols, int(seg_rows), f.ctypes.data,
                                                   c.ctypes.data, _lib.ptr(stream), stream.numel(), _lib.stream()))
    tables, slot_map = _tables_host(f, c)
    return TensorCompressResult(success=True, stream=stream.cpu(), states=states.cpu().view(torch.int32),
                                sizes=sizes.cpu().view(torch.int32), tables=tables, slot_map=slot_map,
                                checkpoints=torch.empty(0, dtype=torch.uint64), num_streams=S,
                                stream_len=int(stream.numel()))


RansManager.compress = _legacy_compress
RansManager.compress_segments = _legacy_compress_segments
RansManager.decompress = _legacy_decompress
RansManager.decompress_into = _legacy_decompress_into


def decompress(stream, states, sizes, num_streams, tables, slot_map, output):
    """ccore.decompress (src/python_bindings.cpp:61-78): legacy flat layout, all CUDA tensors,
    writes into `output` on the current stream, does not synchronise."""
    if not stream.is_cuda:
        raise RuntimeError("Stream must be on GPU")
    if not output.is_cuda:
        raise RuntimeError("Output buffer must be on GPU")
    _lib.check(_lib.load().ci_decode_legacy(
        _lib.ptr(stream), stream.numel(), _lib.ptr(_lib.as_u32(states, "states")),
        _lib.ptr(_lib.as_u32(sizes, "sizes")), int(num_streams), output.numel(),
        _lib.ptr(_lib.as_u32(tables, "tables")), _lib.ptr(_lib.as_u8(slot_map, "slot_map")),
        _lib.ptr(output), _lib.stream()))


def allocate_pinned_tensor(size):
    """ccore.allocate_pinned_tensor (src/python_bindings.cpp:110-135): pinned uint8 CPU tensor."""
    return torch.empty(int(size), dtype=torch.uint8, pin_memory=True)


def allocate_pinned_memory(size):
    """ccore.allocate_pinned_memory (src/python_bindings.cpp:91-108): pinned uint8 numpy array."""
    return allocate_pinned_tensor(size).numpy()
