"""Tensor-parallel exchange: a one-shot all-reduce over peer memory for the small activation tensors
that row-parallel linears produce (ci_allreduce_oneshot), with NCCL as the route for anything that does
not fit it.  The reference has no multi-GPU code.

The buffers every peer writes into come from torch's symmetric memory (CUDA IPC / fabric handles mapped
into each process); only plain peer loads and stores are used on them.
"""
import ctypes as C

import torch
import torch.distributed as dist

from . import _lib


class OneShotAllReduce:
    """all_reduce(sum) for bf16 tensors of at most ``capacity`` elements on ``group``; in place.

    Falls back to ``dist.all_reduce`` for larger tensors, other dtypes, or when symmetric memory cannot be
    set up on this system (``self.native`` is then False and ``self.why`` says why)."""

    def __init__(self, group=None, capacity: int = 1 << 16, device=None):
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.capacity = (int(capacity) + 7) // 8 * 8
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.native, self.why = False, ""
        if self.world == 1:
            self.why = "single rank"
            return
        if self.world > 8:
            self.why = "more than 8 ranks"
            return
        try:
            import torch.distributed._symmetric_memory as symm
            lib = _lib.load()
            total = lib.ci_allreduce_buffer_bytes(self.world, self.capacity)
            self._buf = symm.empty(total, dtype=torch.uint8, device=self.device)
            self._buf.zero_()
            torch.cuda.synchronize(self.device)
            name = self.group.group_name if hasattr(self.group, "group_name") else self.group
            self._hdl = symm.rendezvous(self._buf, name)
            ptrs = [int(p) for p in self._hdl.buffer_ptrs]
            self._bufs = (C.c_void_p * self.world)(*ptrs)
            self._counters = torch.zeros(lib.ci_allreduce_counter_bytes(), dtype=torch.uint8, device=self.device)
            self._status = torch.zeros(1, dtype=torch.int32, device=self.device)
            # a second buffer with its own call sequence for the exchange fused into the row-parallel GEMV
            self._buf_f = symm.empty(total, dtype=torch.uint8, device=self.device)
            self._buf_f.zero_()
            torch.cuda.synchronize(self.device)
            self._hdl_f = symm.rendezvous(self._buf_f, name)
            self._bufs_f = (C.c_void_p * self.world)(*[int(p) for p in self._hdl_f.buffer_ptrs])
            self._counter_f = torch.zeros(lib.ci_linear_allreduce_counter_bytes(), dtype=torch.uint8,
                                          device=self.device)
            dist.barrier(self.group)                           # every rank's buffer is zeroed before anyone writes
            torch.cuda.synchronize(self.device)
            self.native = True
            self._self_test()
        except Exception as e:                                  # no peer access, no symmetric memory, ...
            self.native = False
            self.why = f"{type(e).__name__}: {e}"

    def _self_test(self):
        """Two small exchanges checked against NCCL before the first real use; every rank takes the same
        verdict, so either all of them use the peer-memory kernel or none does."""
        ok = True
        for n in (min(self.capacity, 4096), 3):
            x = (torch.arange(n, device=self.device, dtype=torch.float32) % 13 - 6 + self.rank).to(torch.bfloat16)
            want = x.clone()
            dist.all_reduce(want, group=self.group)
            got = self(x.clone())
            torch.cuda.synchronize(self.device)
            ok = ok and bool(torch.equal(got, want)) and self.status() == 0     # small integers: sums are exact
        verdict = torch.tensor([1 if ok else 0], device=self.device, dtype=torch.int32)
        dist.all_reduce(verdict, op=dist.ReduceOp.MIN, group=self.group)
        if int(verdict.item()) == 0:
            self.native = False
            self.why = "self-test against NCCL failed on some rank"

    def status(self) -> int:
        """0, or 9 if a wait for a peer ran out (reading it synchronises with the device)."""
        return int(self._status.item()) if self.native else 0

    def fused_linear(self, w, x2: torch.Tensor, n_out: int, bias=None):
        """y = all_reduce(x2 @ W_shard) (+ bias) in one kernel (ci_linear_allreduce) for one or two activation
        rows; returns None when this route does not apply (the caller then multiplies and reduces separately).
        ``w`` is the ci_tiled_weight descriptor of this rank's row shard."""
        M = x2.shape[0]
        if not self.native or M > 2 or n_out % 2 or M * n_out > self.capacity:
            return None
        from . import ops
        lib = _lib.load()
        y = torch.empty((M, n_out), device=x2.device, dtype=torch.bfloat16)
        ws = _lib.workspace(x2.device, lib.ci_linear_workspace_bytes(M, n_out, w.K, w.tile_h))
        b = ops._bias(bias, n_out)
        rc = lib.ci_linear_allreduce(w, _lib.ptr(x2), x2.stride(0), M, _lib.ptr(b), _lib.ptr(y), _lib.ptr(ws),
                                     ws.numel(), self._bufs_f, self.capacity, _lib.ptr(self._counter_f), self.rank,
                                     self.world, _lib.ptr(self._status), _lib.stream())
        if rc == -1:                                            # CI_E_INVALID: the weight does not qualify
            return None
        _lib.check(rc)
        return y

    def __call__(self, t: torch.Tensor) -> torch.Tensor:
        if (not self.native or t.dtype != torch.bfloat16 or not t.is_cuda or not t.is_contiguous()
                or t.numel() > self.capacity):
            if self.world > 1:
                dist.all_reduce(t, group=self.group)
            return t
        _lib.check(_lib.load().ci_allreduce_oneshot(_lib.ptr(t), _lib.ptr(t), t.numel(), self.capacity, self._bufs,
                                                    _lib.ptr(self._counters), self.rank, self.world,
                                                    _lib.ptr(self._status), _lib.stream()))
        return t
