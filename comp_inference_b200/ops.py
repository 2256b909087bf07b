"""The reference's Python ops, same names and keyword arguments, on the CUDA
kernels of libci_b200.so.  (The names still say "triton" because they are the
public API of the reference; nothing here is Triton.)

    rans_decomp_triton_tiled                  comp_inference/rans_triton.py:122-168
    rans_decomp_triton                        comp_inference/rans_triton.py:243-271 (legacy flat layout)
    fused_rans_linear_triton                  comp_inference/linear_triton.py:229-314
    fused_rans_linear_transposed_triton       comp_inference/transposed_linear_triton.py:361-435
    fused_rans_embedding_triton               comp_inference/embedding_triton.py:278-330
    *_uncoalesced variants                    linear_triton.py:1189-1265, embedding_triton.py:431-483,
                                              transposed_linear_triton.py:813-883
    triton_matmul                             comp_inference/triton_gemm.py:324-337

All tensor arguments must already be CUDA tensors; inputs are borrowed for the
call, outputs are fresh tensors or the caller's ``out``.  Everything is queued on
the current torch CUDA stream and nothing synchronises.
"""
import torch

from . import _lib


def _check_x(x, K):
    if x.dtype != torch.bfloat16:
        raise RuntimeError(f"activations must be bfloat16, got {x.dtype}")
    _lib.require_cuda(x, "x")
    x2 = x.reshape(-1, K)
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    return x2


def _bias(bias, n):
    if bias is None:
        return None
    if bias.dtype != torch.bfloat16 or bias.numel() != n:
        raise RuntimeError("bias must be bfloat16 with one entry per output feature")
    return bias.contiguous()


def rans_decomp_triton_tiled(compressed_streams, initial_states, tables, slot_map, output_shape, tile_offsets,
                             tile_max_lens, tile_k=1024, tile_n=32):
    """Exponent plane uint8 [K,N] of a tiled stream."""
    K, N = int(output_shape[0]), int(output_shape[1])
    w, keep = _lib.tiled_weight(compressed_streams, initial_states, tables, slot_map, tile_offsets, tile_max_lens,
                                None, K, N, int(tile_k), int(tile_n), want_max=True)
    out = torch.empty((K, N), device=compressed_streams.device, dtype=torch.uint8)
    _lib.check(_lib.load().ci_decode_plane(w, _lib.ptr(out), _lib.stream()))
    return out


def rans_decomp_triton(compressed_streams, initial_states, tables, slot_map, stream_sizes, output_shape):
    """Legacy flat layout: stream g = seg * width + col holds rows [512 * seg, 512 * (seg + 1)) of column col,
    its bytes at stride len(initial_states) read from index stream_sizes[g] - 1 downwards; returns the uint8
    plane of ``output_shape`` (comp_inference/rans_triton.py:171-271; the order RansManager.compress of the
    reference writes, src/cuda/rans_kernels.cuh:393-509)."""
    rows, cols = int(output_shape[0]), int(output_shape[1])
    _lib.require_cuda(compressed_streams, "compressed stream")
    n = int(initial_states.numel())
    out = torch.empty((rows, cols), device=compressed_streams.device, dtype=torch.uint8)
    if rows * cols == 0:
        return out
    st = _lib.as_u8(compressed_streams, "compressed stream")
    states = _lib.as_u32(_lib.require_cuda(initial_states, "states"), "states")
    sizes = _lib.as_u32(_lib.require_cuda(stream_sizes, "stream_sizes"), "stream_sizes")
    tb = _lib.as_u32(_lib.require_cuda(tables, "tables"), "tables")
    sm = _lib.as_u8(_lib.require_cuda(slot_map, "slot_map"), "slot_map")
    _lib.check(_lib.load().ci_decode_legacy_segments(_lib.ptr(st), st.numel(), _lib.ptr(states), _lib.ptr(sizes), n,
                                                     rows, cols, 512, _lib.ptr(tb), _lib.ptr(sm), _lib.ptr(out),
                                                     _lib.stream()))
    return out


def rans_decompress_bf16(compressed_streams, initial_states, tables, slot_map, weight_shape, tile_offsets,
                         tile_max_lens, tile_k, tile_n, mantissas):
    """Whole weight as bfloat16 [K,N] in one kernel: the decode + uninterleave + reconstruct
    chain of rans_decompress_module_weight_bf16 (comp_inference/comp_inference.py:633-711)."""
    K, N = int(weight_shape[0]), int(weight_shape[1])
    w, keep = _lib.tiled_weight(compressed_streams, initial_states, tables, slot_map, tile_offsets, tile_max_lens,
                                mantissas, K, N, int(tile_k), int(tile_n), want_max=True)
    out = torch.empty((K, N), device=compressed_streams.device, dtype=torch.bfloat16)
    _lib.check(_lib.load().ci_decode_bf16(w, _lib.ptr(out), _lib.stream()))
    return out


def _linear_call(w, x2, M, n_out, bias, out, split_k, transposed):
    dev = x2.device
    lib = _lib.load()
    y = out.view(M, n_out) if out is not None else torch.empty((M, n_out), device=dev, dtype=torch.bfloat16)
    if y.dtype != torch.bfloat16 or y.stride(1) != 1:
        raise RuntimeError("out must be a bfloat16 tensor with unit inner stride")
    nbytes = lib.ci_linear_workspace_bytes(M, n_out, 0 if transposed else w.K, 0 if transposed else w.tile_h)
    if M > 16 and not transposed and split_k > 1:               # an explicit split-K of the prefill GEMM: room for its partials
        nbytes = max(nbytes, (1 << 14) + min(int(split_k), 8) * M * n_out * 4)
    ws = _lib.workspace(dev, nbytes)
    b = _bias(bias, n_out)
    if transposed:
        _lib.check(lib.ci_linear_transposed(w, _lib.ptr(x2), x2.stride(0), M, _lib.ptr(b), _lib.ptr(y), y.stride(0),
                                            _lib.ptr(ws), ws.numel(), _lib.stream()))
    else:
        _lib.check(lib.ci_linear(w, _lib.ptr(x2), x2.stride(0), M, _lib.ptr(b), _lib.ptr(y), y.stride(0),
                                 _lib.ptr(ws), ws.numel(), int(split_k), _lib.stream()))
    return y


def fused_rans_linear_triton(x, compressed_data, initial_states, tables, slot_map, weight_shape, tile_offsets,
                             tile_max_lens, tile_k, tile_n, mantissas, accum_block_size=32, bias=None, out=None,
                             SPLIT_K=8, workspace=None):
    """y[..., N] = x[..., K] . W[K, N] (+ bias) with W decoded on the fly.

    ``accum_block_size`` and ``workspace`` are accepted for source compatibility: blocking is internal,
    and split-K partials live in this package's own fp32 workspace (the reference's is a bf16 buffer
    of another size).  ``SPLIT_K`` is honoured up to 16; 0 lets the library choose.
    """
    K, N = int(weight_shape[0]), int(weight_shape[1])
    x2 = _check_x(x, K)
    M = x2.shape[0]
    w, keep = _lib.tiled_weight(compressed_data, initial_states, tables, slot_map, tile_offsets, tile_max_lens,
                                mantissas, K, N, int(tile_k), int(tile_n), want_max=True)
    y = _linear_call(w, x2, M, N, bias, out, SPLIT_K, False)
    return out if out is not None else y.view(*x.shape[:-1], N)


def fused_rans_linear_transposed_triton(x, compressed_data, initial_states, tables, slot_map, weight_shape,
                                        tile_offsets, tile_max_lens, tile_k, tile_n, mantissas, workspace=None,
                                        bias=None, out=None, SPLIT_K=8):
    """y[..., V] = x[..., H] . W[V, H]^T for a weight stored [V, H] (LM head / tied embedding)."""
    V, H = int(weight_shape[0]), int(weight_shape[1])
    x2 = _check_x(x, H)
    M = x2.shape[0]
    w, keep = _lib.tiled_weight(compressed_data, initial_states, tables, slot_map, tile_offsets, tile_max_lens,
                                mantissas, V, H, int(tile_k), int(tile_n))
    y = _linear_call(w, x2, M, V, bias, out, 0, True)
    return out if out is not None else y.view(*x.shape[:-1], V)


def fused_rans_embedding_triton(x, compressed_data, initial_states, tables, slot_map, weight_shape, tile_offsets,
                                tile_max_lens, tile_k, tile_n, mantissas, out=None):
    """out[..., :] = W[x[...], :]; ids outside [0, K) give zero rows."""
    K, N = int(weight_shape[0]), int(weight_shape[1])
    _lib.require_cuda(x, "x")
    ids = x.reshape(-1).to(torch.int64).contiguous()
    n = ids.numel()
    w, keep = _lib.tiled_weight(compressed_data, initial_states, tables, slot_map, tile_offsets, tile_max_lens,
                                mantissas, K, N, int(tile_k), int(tile_n), want_max=True)
    o = out.view(n, N) if out is not None else torch.empty((n, N), device=x.device, dtype=torch.bfloat16)
    if o.dtype != torch.bfloat16 or (n > 0 and o.stride(1) != 1):
        raise RuntimeError("out must be a bfloat16 tensor with unit inner stride")
    _lib.check(_lib.load().ci_embedding(w, _lib.ptr(ids), n, _lib.ptr(o), o.stride(0) if n else N, _lib.stream()))
    return o.view(*x.shape, N)


# ---- dense ("uncoalesced") layout ------------------------------------------------

def rans_decomp_uncoalesced(compressed_streams, initial_states, tables, slot_map, output_shape, stream_offsets,
                            stream_sizes, tile_k, tile_n):
    """Exponent plane of a dense-layout stream (no reference counterpart as a stand-alone op)."""
    K, N = int(output_shape[0]), int(output_shape[1])
    w, keep = _lib.dense_weight(compressed_streams, initial_states, stream_sizes, stream_offsets, tables, slot_map,
                                None, K, N, int(tile_k), int(tile_n))
    out = torch.empty((K, N), device=compressed_streams.device, dtype=torch.uint8)
    _lib.check(_lib.load().ci_decode_plane_dense(w, _lib.ptr(out), _lib.stream()))
    return out


def fused_rans_linear_triton_uncoalesced(x, compressed_data, initial_states, tables, slot_map, weight_shape,
                                         stream_offsets, stream_sizes, tile_k, tile_n, mantissas,
                                         accum_block_size=32, bias=None, out=None, SPLIT_K=8, workspace=None):
    K, N = int(weight_shape[0]), int(weight_shape[1])
    x2 = _check_x(x, K)
    M = x2.shape[0]
    w, keep = _lib.dense_weight(compressed_data, initial_states, stream_sizes, stream_offsets, tables, slot_map,
                                mantissas, K, N, int(tile_k), int(tile_n))
    lib = _lib.load()
    y = out.view(M, N) if out is not None else torch.empty((M, N), device=x2.device, dtype=torch.bfloat16)
    ws = _lib.workspace(x2.device, lib.ci_linear_workspace_bytes(M, N, 0, 0))
    b = _bias(bias, N)
    _lib.check(lib.ci_linear_dense(w, _lib.ptr(x2), x2.stride(0), M, _lib.ptr(b), _lib.ptr(y), y.stride(0),
                                   _lib.ptr(ws), ws.numel(), int(SPLIT_K), _lib.stream()))
    return out if out is not None else y.view(*x.shape[:-1], N)


def fused_rans_linear_transposed_triton_uncoalesced(x, compressed_data, initial_states, tables, slot_map,
                                                    weight_shape, stream_offsets, stream_sizes, tile_k, tile_n,
                                                    mantissas, workspace=None, bias=None, out=None, SPLIT_K=8):
    """y[..., V] = x[..., H] . W[V, H]^T for a dense-layout weight stored [V, H]
    (comp_inference/transposed_linear_triton.py:813-883).  ``workspace`` and ``SPLIT_K`` are accepted for source
    compatibility; the split and its fp32 partials are internal."""
    V, H = int(weight_shape[0]), int(weight_shape[1])
    x2 = _check_x(x, H)
    M = x2.shape[0]
    w, keep = _lib.dense_weight(compressed_data, initial_states, stream_sizes, stream_offsets, tables, slot_map,
                                mantissas, V, H, int(tile_k), int(tile_n))
    lib = _lib.load()
    y = out.view(M, V) if out is not None else torch.empty((M, V), device=x2.device, dtype=torch.bfloat16)
    if y.dtype != torch.bfloat16 or y.stride(1) != 1:
        raise RuntimeError("out must be a bfloat16 tensor with unit inner stride")
    ws = _lib.workspace(x2.device, lib.ci_linear_workspace_bytes(M, V, 0, 0))
    b = _bias(bias, V)
    _lib.check(lib.ci_linear_transposed_dense(w, _lib.ptr(x2), x2.stride(0), M, _lib.ptr(b), _lib.ptr(y), y.stride(0),
                                              _lib.ptr(ws), ws.numel(), _lib.stream()))
    return out if out is not None else y.view(*x.shape[:-1], V)


def fused_rans_embedding_triton_uncoalesced(x, compressed_data, initial_states, tables, slot_map, weight_shape,
                                            stream_offsets, stream_sizes, tile_k, tile_n, mantissas, out=None):
    K, N = int(weight_shape[0]), int(weight_shape[1])
    ids = _lib.require_cuda(x, "x").reshape(-1).to(torch.int64).contiguous()
    n = ids.numel()
    w, keep = _lib.dense_weight(compressed_data, initial_states, stream_sizes, stream_offsets, tables, slot_map,
                                mantissas, K, N, int(tile_k), int(tile_n))
    o = out.view(n, N) if out is not None else torch.empty((n, N), device=x.device, dtype=torch.bfloat16)
    _lib.check(_lib.load().ci_embedding_dense(w, _lib.ptr(ids), n, _lib.ptr(o), o.stride(0) if n else N,
                                              _lib.stream()))
    return o.view(*x.shape, N)


def triton_matmul(a, b):
    """Dense bf16 matmul on an already decompressed [K,N] weight (comp_inference/triton_gemm.py:324-337).
    A plain library GEMM: nothing compressed is involved, so this is torch.matmul."""
    return torch.matmul(a, b)


# ---- the weightless steps between the linears of a decode step (csrc/glue.cu) -----------------------

def _rows(t):
    """A bf16 CUDA tensor as [rows, cols] with unit inner stride (a view where possible)."""
    if t.dtype != torch.bfloat16:
        raise RuntimeError(f"expected bfloat16, got {t.dtype}")
    t2 = _lib.require_cuda(t, "tensor").reshape(-1, t.shape[-1])
    return t2 if t2.stride(1) == 1 else t2.contiguous()


def add_rmsnorm(x, residual, weight, eps):
    """h = x (+ residual); returns (rmsnorm(h) * weight, h), both bf16 [..., H], in one kernel
    (h is x itself when there is no residual)."""
    x2 = _rows(x)
    rows, cols = x2.shape
    y = torch.empty((rows, cols), device=x.device, dtype=torch.bfloat16)
    r2 = _rows(residual) if residual is not None else None
    h = torch.empty((rows, cols), device=x.device, dtype=torch.bfloat16) if r2 is not None else None
    _lib.check(_lib.load().ci_add_rmsnorm(_lib.ptr(x2), x2.stride(0), _lib.ptr(r2), r2.stride(0) if r2 is not None else 0,
                                          _lib.ptr(weight), float(eps), rows, cols, _lib.ptr(y), cols, _lib.ptr(h), cols,
                                          _lib.stream()))
    shape = x.shape
    return y.view(shape), (h.view(shape) if h is not None else x)


def rope_kv(q, k, v, cos, sin, pos, k_cache, v_cache, head_dim):
    """Rotary embedding of position ``pos`` (a one-element int64 CUDA tensor) on q [B, n_q * d] and k [B, n_kv * d],
    and the write of k, v into the caches [B, n_kv, T, d] at that position; returns the rotated q [B, n_q, d]."""
    q2, k2, v2 = _rows(q), _rows(k), _rows(v)
    B = q2.shape[0]
    n_q, n_kv = q2.shape[1] // head_dim, k2.shape[1] // head_dim
    T = k_cache.shape[2]
    if not (k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.shape[0] >= B and k_cache.shape[1] == n_kv):
        raise RuntimeError("KV caches must be contiguous [B, n_kv, T, d] tensors")
    q_out = torch.empty((B, n_q, head_dim), device=q.device, dtype=torch.bfloat16)
    _lib.check(_lib.load().ci_rope_kv(_lib.ptr(q2), q2.stride(0), _lib.ptr(k2), k2.stride(0), _lib.ptr(v2), v2.stride(0),
                                      _lib.ptr(cos), _lib.ptr(sin), _lib.ptr(pos), B, n_q, n_kv, head_dim, T,
                                      _lib.ptr(q_out), _lib.ptr(k_cache), _lib.ptr(v_cache), _lib.stream()))
    return q_out


def decode_attention(q, k_cache, v_cache, pos, scale=None):
    """softmax(scale * q . K^T) . V for one query per (batch row, head) over cache positions 0 .. pos;
    q [B, n_q, d], caches [B, n_kv, T, d]; returns [B, n_q * d]."""
    B, n_q, d = q.shape
    n_kv, T = k_cache.shape[1], k_cache.shape[2]
    out = torch.empty((B, n_q * d), device=q.device, dtype=torch.bfloat16)
    lib = _lib.load()
    ws = _attention_workspace(q.device, lib.ci_decode_attention_workspace_bytes(B, n_q, d, T))
    _lib.check(lib.ci_decode_attention(_lib.ptr(q), _lib.ptr(k_cache), _lib.ptr(v_cache), _lib.ptr(pos), B, n_q,
                                       n_kv, d, T, float(scale if scale is not None else d ** -0.5),
                                       _lib.ptr(ws), ws.numel(), _lib.ptr(out), n_q * d, _lib.stream()))
    return out


_attn_ws = {}
_attn_retired = []


def _attention_workspace(device, nbytes):
    """Zeroed scratch of the attention kernel, one per (device, stream), never freed once handed out (a captured
    graph keeps the address)."""
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    ws = _attn_ws.get(key)
    if ws is None or ws.numel() < nbytes:
        if ws is not None:
            _attn_retired.append(ws)
        ws = torch.zeros(max(int(nbytes), 1 << 20), dtype=torch.uint8, device=device)
        _attn_ws[key] = ws
    return ws


def silu_mul(gate, up):
    """silu(gate) * up, element-wise, bf16 [..., F]; the inputs may be column slices of a wider tensor."""
    g2, u2 = _rows(gate), _rows(up)
    rows, cols = g2.shape
    out = torch.empty((rows, cols), device=gate.device, dtype=torch.bfloat16)
    _lib.check(_lib.load().ci_silu_mul(_lib.ptr(g2), g2.stride(0), _lib.ptr(u2), u2.stride(0), rows, cols, _lib.ptr(out),
                                       cols, _lib.stream()))
    return out.view(*gate.shape)
