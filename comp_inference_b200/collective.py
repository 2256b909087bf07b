"""Tensor-parallel exchanges over peer memory for the small activation tensors of decode steps: a one-shot
all-reduce for the outputs of row-parallel linears (ci_allreduce_oneshot, and the same protocol inside the
GEMV kernel: ci_linear_allreduce) and a one-shot all-gather for the logits of a vocabulary-parallel LM head
(ci_allgather_oneshot), with NCCL as the route for anything that does not fit them.  The reference has no
multi-GPU code.

The buffers every peer writes into come from torch's symmetric memory (CUDA IPC / fabric handles mapped
into each process); only plain peer loads and stores are used on them.  Symmetric memory would also bind
every buffer to an NVLink multicast object where the hardware has one; nothing here uses multicast, and a
rank that ends while its memory is bound to such an object can fault its peers' GPUs, so the binding is
switched off (TORCH_SYMM_MEM_DISABLE_MULTICAST=1) before the first buffer is made.
"""
import ctypes as C
import os

os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")

import torch
import torch.distributed as dist

from . import _lib


def _peer_buffer(nbytes, device, group):
    """(tensor, handle, array of every rank's pointer) of a zeroed symmetric-memory buffer."""
    os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"
    import torch.distributed._symmetric_memory as symm
    buf = symm.empty(nbytes, dtype=torch.uint8, device=device)
    buf.zero_()
    torch.cuda.synchronize(device)
    name = group.group_name if hasattr(group, "group_name") else group
    hdl = symm.rendezvous(buf, name)
    world = dist.get_world_size(group)
    ptrs = (C.c_void_p * world)(*[int(p) for p in hdl.buffer_ptrs])
    return buf, hdl, ptrs


class _PeerExchange:
    def _base_init(self, group, capacity, device):
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.capacity = (int(capacity) + 7) // 8 * 8
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.native, self.why = False, ""
        if self.world == 1:
            self.why = "single rank"
            return False
        if self.world > 8:
            self.why = "more than 8 ranks"
            return False
        return True

    def _agree(self, ok, why):
        """Every rank takes the same verdict: either all use the peer-memory kernel or none does."""
        verdict = torch.tensor([1 if ok else 0], device=self.device, dtype=torch.int32)
        dist.all_reduce(verdict, op=dist.ReduceOp.MIN, group=self.group)
        if int(verdict.item()) == 0:
            self.native = False
            self.why = why

    def status(self) -> int:
        """0, or 9 if a wait for a peer ran out (reading it synchronises with the device)."""
        return int(self._status.item()) if self.native else 0

    def check_status(self):
        """Raises if a wait for a peer ran out in any call so far (ci_status: CI_E_DEVICE)."""
        if self.native:
            _lib.check(_lib.load().ci_status(_lib.ptr(self._status), None, 0, _lib.stream()))

    def close(self):
        """Lines the ranks up and releases the peer-mapped buffers; call it before a rank leaves, with none of
        its kernels in flight, so that no peer is left writing into memory that is going away."""
        if self.native:
            torch.cuda.synchronize(self.device)
            dist.barrier(self.group)
            self.native = False
            self.why = "closed"
            for name in ("_bufs", "_hdl", "_buf", "_bufs_f", "_hdl_f", "_buf_f"):
                if hasattr(self, name):
                    delattr(self, name)
            torch.cuda.synchronize(self.device)


class OneShotAllReduce(_PeerExchange):
    """all_reduce(sum) for bf16 tensors of at most ``capacity`` elements on ``group``; in place.

    Falls back to ``dist.all_reduce`` for larger tensors, other dtypes, or when symmetric memory cannot be
    set up on this system (``self.native`` is then False and ``self.why`` says why)."""

    def __init__(self, group=None, capacity: int = 1 << 16, device=None):
        if not self._base_init(group, capacity, device):
            return
        try:
            lib = _lib.load()
            total = lib.ci_allreduce_buffer_bytes(self.world, self.capacity)
            self._buf, self._hdl, self._bufs = _peer_buffer(total, self.device, self.group)
            self._counters = torch.zeros(lib.ci_allreduce_counter_bytes(), dtype=torch.uint8, device=self.device)
            self._status = torch.zeros(1, dtype=torch.int32, device=self.device)
            # a second buffer with its own call sequence for the exchange fused into the row-parallel GEMV
            self._buf_f, self._hdl_f, self._bufs_f = _peer_buffer(total, self.device, self.group)
            self._counter_f = torch.zeros(lib.ci_linear_allreduce_counter_bytes(), dtype=torch.uint8,
                                          device=self.device)
            dist.barrier(self.group)                           # every rank's buffer is zeroed before anyone writes
            torch.cuda.synchronize(self.device)
            self.native = True
        except Exception as e:                                  # no peer access, no symmetric memory, ...
            self.native = False
            self.why = f"{type(e).__name__}: {e}"
        # a rank whose set-up failed must still take part in the group's verdict
        self._agree(self.native, "symmetric memory could not be set up on some rank")
        if self.native:
            self._self_test()

    def _self_test(self):
        """Two small exchanges checked against NCCL before the first real use."""
        ok = True
        for n in (min(self.capacity, 4096), 3):
            x = (torch.arange(n, device=self.device, dtype=torch.float32) % 13 - 6 + self.rank).to(torch.bfloat16)
            want = x.clone()
            dist.all_reduce(want, group=self.group)
            got = self(x.clone())
            torch.cuda.synchronize(self.device)
            ok = ok and bool(torch.equal(got, want)) and self.status() == 0     # small integers: sums are exact
        self._agree(ok, "self-test against NCCL failed on some rank")

    def fused_qualifies(self, w, M: int, n_out: int) -> bool:
        """Whether ALL ranks can run ci_linear_allreduce on their shard ``w`` for M rows (a collective call:
        every rank of the group must make it, for the same layer, in the same order).  Shards differ in their
        deepest tile, so a rank's own answer is not enough; the group takes the minimum."""
        mine = (self.native and 1 <= M <= 2 and n_out % 2 == 0 and M * n_out <= self.capacity
                and _lib.load().ci_linear_allreduce_qualifies(w, M) == 1)
        if self.world == 1:
            return bool(mine)
        verdict = torch.tensor([1 if mine else 0], device=self.device, dtype=torch.int32)
        dist.all_reduce(verdict, op=dist.ReduceOp.MIN, group=self.group)
        return bool(verdict.item())

    def fused_linear(self, w, x2: torch.Tensor, n_out: int, bias=None):
        """y = all_reduce(x2 @ W_shard) (+ bias) in one kernel (ci_linear_allreduce) for one or two activation
        rows.  Only for layers that passed ``fused_qualifies`` on every rank; a refusal here raises instead of
        quietly taking another route, because the peers would wait for this rank's stores."""
        M = x2.shape[0]
        from . import ops
        lib = _lib.load()
        if x2.data_ptr() % 8 or x2.stride(0) % 4:
            x2 = x2.contiguous().clone()                        # the kernel reads the rows as aligned 8-byte quads
        y = torch.empty((M, n_out), device=x2.device, dtype=torch.bfloat16)
        ws = _lib.workspace(x2.device, lib.ci_linear_workspace_bytes(M, n_out, w.K, w.tile_h))
        b = ops._bias(bias, n_out)
        _lib.check(lib.ci_linear_allreduce(w, _lib.ptr(x2), x2.stride(0), M, _lib.ptr(b), _lib.ptr(y), _lib.ptr(ws),
                                           ws.numel(), self._bufs_f, self.capacity, _lib.ptr(self._counter_f),
                                           self.rank, self.world, _lib.ptr(self._status), _lib.stream()))
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


class OneShotAllGather(_PeerExchange):
    """y[M, world * cols] = concatenation along the last dimension of every rank's bf16 x[M, cols] (the logits
    of a vocabulary-parallel LM head).  Peer-memory kernel for M * cols <= capacity, NCCL otherwise."""

    def __init__(self, group=None, capacity: int = 1 << 16, device=None):
        if not self._base_init(group, capacity, device):
            return
        try:
            lib = _lib.load()
            total = lib.ci_allreduce_buffer_bytes(self.world, self.capacity)
            self._buf, self._hdl, self._bufs = _peer_buffer(total, self.device, self.group)
            self._counters = torch.zeros(lib.ci_allreduce_counter_bytes(), dtype=torch.uint8, device=self.device)
            self._status = torch.zeros(1, dtype=torch.int32, device=self.device)
            dist.barrier(self.group)
            torch.cuda.synchronize(self.device)
            self.native = True
        except Exception as e:
            self.native = False
            self.why = f"{type(e).__name__}: {e}"
        self._agree(self.native, "symmetric memory could not be set up on some rank")
        if self.native:
            x = (torch.arange(2 * 6, device=self.device, dtype=torch.float32).view(2, 6) + 100 * self.rank).to(torch.bfloat16)
            want = self._nccl(x)
            got = self(x)
            torch.cuda.synchronize(self.device)
            self._agree(bool(torch.equal(got, want)) and self.status() == 0, "self-test against NCCL failed on some rank")

    def _nccl(self, x2):
        M, cols = x2.shape
        parts = torch.empty((self.world, M, cols), device=x2.device, dtype=x2.dtype)
        dist.all_gather_into_tensor(parts, x2.contiguous(), group=self.group)
        return parts.permute(1, 0, 2).reshape(M, self.world * cols)

    def __call__(self, x2: torch.Tensor) -> torch.Tensor:
        M, cols = x2.shape
        if self.world == 1:
            return x2
        if (not self.native or x2.dtype != torch.bfloat16 or cols % 2 or M * cols > self.capacity
                or not x2.is_contiguous()):
            return self._nccl(x2)
        y = torch.empty((M, self.world * cols), device=x2.device, dtype=torch.bfloat16)
        _lib.check(_lib.load().ci_allgather_oneshot(_lib.ptr(x2), _lib.ptr(y), M, cols, self.capacity, self._bufs,
                                                    _lib.ptr(self._counters), self.rank, self.world,
                                                    _lib.ptr(self._status), _lib.stream()))
        return y
