"""GPU: the allocation-free fused linear (ci_linear_static) against ci_linear.

Some callers of this library are not allowed to allocate device memory while the model runs (a
server that partitioned its memory up front, a plug-in that only gets input and output buffers);
for them the scratch that ci_linear takes from the caller lives in a fixed array inside the library.
The results must be the same as with a caller-provided workspace, also when the entry point is
called again right away (the array keeps the previous call's contents).  Both entry points are
called straight through the C ABI.  The file name sorts last so that a run that stops at the first
failure has already run every other test.
"""
import ctypes as C

import pytest
import torch

from conftest import make_weight

pytestmark = pytest.mark.gpu


def _call(lib, fn, w, x, y, ws=None):
    from comp_inference_b200 import _lib
    M = x.shape[0]
    if ws is None:
        rc = fn(w, _lib.ptr(x), x.stride(0), M, None, _lib.ptr(y), y.stride(0), _lib.stream())
    else:
        rc = fn(w, _lib.ptr(x), x.stride(0), M, None, _lib.ptr(y), y.stride(0), _lib.ptr(ws), ws.numel(), 0,
                _lib.stream())
    _lib.check(rc)


@pytest.mark.parametrize("K,N,th,M", [(1024, 512, 128, 1), (4096, 4096, 128, 4), (300, 100, 256, 16), (4096, 11008, 128, 16)])
def test_static_scratch_matches_workspace_version(K, N, th, M):
    import comp_inference_b200 as ci
    from comp_inference_b200 import _lib
    lib = _lib.load()
    W = make_weight(K, N, seed=K + N + M).cuda()
    c = ci.compress_weight_cuda(W, th, 32)
    w, keep = _lib.tiled_weight(c["rans_exp_stream"], c["rans_exp_states"], c["rans_exp_tables"],
                                c["rans_exp_slot_map"], c["rans_exp_tile_offsets"], c["rans_exp_tile_max_lens"],
                                c["rans_man_raw"], K, N, c["tile_height"], c["tile_width"], want_max=True)
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(M)).to(torch.bfloat16).cuda()
    ws = torch.zeros(lib.ci_linear_workspace_bytes(M, N, K, th), dtype=torch.uint8, device="cuda")
    want = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    _call(lib, lib.ci_linear, w, x, want, ws)
    ref = x.float() @ W.float()
    assert float((want.float() - ref).abs().max() / ref.abs().max()) <= 1e-2
    got = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    _call(lib, lib.ci_linear_static, w, x, got)          # first call: kernel code is loaded, the array's address looked up
    torch.cuda.synchronize()
    assert torch.equal(got.view(torch.uint16), want.view(torch.uint16))
    for _ in range(2):                                   # twice in a row: the shared array is reused as it was left
        got.fill_(float("nan"))
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        _call(lib, lib.ci_linear_static, w, x, got)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        # the property the entry point exists for: the call itself takes no device memory
        assert free_after == free_before, (free_before, free_after)
        assert torch.equal(got.view(torch.uint16), want.view(torch.uint16))
    # nothing went wrong inside the built-in array either: its status word (which the per-call clearing leaves
    # alone) is zero
    code = C.c_uint32(99)
    assert lib.ci_linear_static_status(C.byref(code), 0, _lib.stream()) == 0 and code.value == 0


def test_static_scratch_rejects_what_does_not_fit():
    import comp_inference_b200 as ci
    from comp_inference_b200 import _lib
    lib = _lib.load()
    assert lib.ci_linear_static_max_bytes() == 16 << 20
    K, N = 256, 64
    W = make_weight(K, N, seed=1).cuda()
    c = ci.compress_weight_cuda(W, 64, 32)
    w, keep = _lib.tiled_weight(c["rans_exp_stream"], c["rans_exp_states"], c["rans_exp_tables"],
                                c["rans_exp_slot_map"], c["rans_exp_tile_offsets"], c["rans_exp_tile_max_lens"],
                                c["rans_man_raw"], K, N, 64, 32, want_max=True)
    x = torch.zeros(17, K, dtype=torch.bfloat16, device="cuda")
    y = torch.zeros(17, N, dtype=torch.bfloat16, device="cuda")
    rc = lib.ci_linear_static(w, _lib.ptr(x), K, 17, None, _lib.ptr(y), N, _lib.stream())
    assert rc == -4 and b"at most 16" in lib.ci_last_error()
    big = _lib.TiledWeight.from_buffer_copy(w)
    big.N = 40000                                         # 16 rows x 40000 outputs would need ~41 MB of partials
    rc = lib.ci_linear_static(big, _lib.ptr(x), K, 16, None, _lib.ptr(y), 40000, _lib.stream())
    assert rc == -4 and b"built-in array" in lib.ci_last_error()
