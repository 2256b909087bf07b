"""Module wrappers over the compressed buffers and the Hugging Face model patcher
(the reference's comp_inference/pytorch_runtime.py:386-642), with the same class
names, constructor arguments and buffer names, so a saved package loads unchanged.

Buffers are device-resident; the per-forward ``.to(device)`` calls of the
reference (its CPU "on-demand offloading", pytorch_runtime.py:440-459) are gone
because there is no CPU path here.
"""
import torch
import torch.nn as nn

from . import _lib
from . import ops

_BUFFERS = (("rans_exp_stream", torch.uint8), ("rans_exp_states", torch.uint32), ("rans_exp_tables", torch.uint32),
            ("rans_exp_slot_map", torch.uint8), ("rans_exp_tile_offsets", torch.uint32),
            ("rans_exp_tile_max_lens", torch.uint32), ("rans_man_raw", torch.uint8), ("rans_info", torch.int32))


class RansWorkspace:
    """Source compatibility only (pytorch_runtime.py:386-394): hands out a bf16 [split_k, M, N] buffer that
    NOTHING in this package reads or writes.  Callers that pass ``workspace=`` to the ops keep working;
    the kernels' own ticket counters and fp32 partial sums live in one zeroed buffer per (device, CUDA
    stream) that is never freed once handed out (``_lib.workspace``)."""
    _buffer = None

    @classmethod
    def get_workspace(cls, M, N, split_k, device):
        elements = max(M * N * split_k, 1)
        if cls._buffer is None or cls._buffer.numel() < elements or cls._buffer.device != torch.device(device):
            cls._buffer = torch.zeros(elements * 2, device=device, dtype=torch.bfloat16)
        return cls._buffer[:elements].view(split_k, M, N)


class _RansBase(nn.Module):
    def _register(self):
        for name, dt in _BUFFERS:
            self.register_buffer(name, torch.empty(0, dtype=dt))

    def _stored_shape(self):
        """(K, N) of the matrix as it is stored."""
        raise NotImplementedError

    def load_compressed(self, c, validate=False):
        """Adopts the tensors of a dict produced by comp_inference.compress_weight_cuda (or a saved package).
        ``validate``: run ci_validate_tiled_metadata on host copies first and raise on malformed metadata."""
        if validate:
            K, N = self._stored_shape()
            _lib.validate_compressed(c, K, N, int(self.tile_k), int(self.tile_n))
        for name, _ in _BUFFERS:
            if name in c:
                setattr(self, name, c[name])
        return self

    def prepare(self):
        """Everything a forward would otherwise do lazily on its first call (descriptor, prepared decode
        table, the deepest tile -- one device-to-host read): call it once the buffers are on the GPU and
        before a CUDA graph is captured.  Subclasses add their own one-time work."""
        if self.rans_exp_stream.is_cuda and self.rans_exp_states.numel():
            self._weight(*self._stored_shape())
        return self

    _handle = None

    def _weight(self, K, N):
        """The ci_tiled_weight descriptor of this module's buffers, built once (with the prepared decode
        table and the deepest tile) and rebuilt only if a buffer was replaced."""
        key = (self.rans_exp_stream.data_ptr(), self.rans_exp_states.data_ptr(), self.rans_man_raw.data_ptr(),
               self.rans_exp_tile_offsets.data_ptr(), self.tile_k, self.tile_n)
        if self._handle is None or self._handle[0] != key:
            w, keep = _lib.tiled_weight(self.rans_exp_stream, self.rans_exp_states, self.rans_exp_tables,
                                        self.rans_exp_slot_map, self.rans_exp_tile_offsets,
                                        self.rans_exp_tile_max_lens, self.rans_man_raw, K, N, int(self.tile_k),
                                        int(self.tile_n), want_max=True)
            self._handle = (key, w, keep)
        return self._handle[1]


_scratch = {}
_scratch_retired = []


def _decode_scratch(device, K, N):
    """The bf16 buffer the decode-then-GEMM route decodes into: one per (device, stream) -- two streams may run
    this route at the same time -- grown on demand.  A buffer that is outgrown is kept alive, not freed: a
    captured graph may still write to it."""
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < K * N:
        if buf is not None:
            _scratch_retired.append(buf)
        buf = torch.empty(K * N, dtype=torch.bfloat16, device=device)
        _scratch[key] = buf
    return buf[:K * N].view(K, N)


def _decode_then_gemm(w_desc, K, N, x2, bias=None, transposed=False):
    """x2 [M, K] times the compressed weight behind ``w_desc``: one stand-alone decode into the device's scratch
    buffer, then a library GEMM.  ``transposed``: the weight is stored [N, K] (the LM head's stored layout) and
    the GEMM reads it as its transpose."""
    rows, cols = (N, K) if transposed else (K, N)
    w = _decode_scratch(x2.device, rows, cols)
    _lib.check(_lib.load().ci_decode_bf16(w_desc, _lib.ptr(w), _lib.stream()))
    y = torch.matmul(x2, w.t() if transposed else w)
    if bias is not None:
        y += bias
    return y


class RansLinear(_RansBase):
    """nn.Linear replacement; weight stored compressed as [K=in, N=out] (pytorch_runtime.py:397-459).

    ``prefill_policy`` chooses what a call with more than 16 activation rows runs (up to 16 rows every policy
    runs the fused decode-GEMV kernels):
    "fused" the decode-GEMM kernel at every size (tcgen05, the decoded weight never leaves the chip);
    "decode_then_gemm" / "auto" (default) from ``prefill_rows`` rows up the stand-alone decoder into a reused
    per-device scratch buffer followed by a library GEMM -- the reference's decompress + triton_matmul pair
    (comp_inference/triton_gemm.py:324-337): the weight is decoded once however many rows there are, at the full
    rate of the stand-alone decoder.  Measured on a B200 over one Llama-2-7B block this route is the faster one
    at every row count above 16 (0.31 ms against 0.50 ms at 17 rows, 0.32 / 0.53 at 128, 0.38 / 0.70 at 512,
    0.50 / 1.24 at 1024), hence the default ``prefill_rows`` = 17.
    """

    def __init__(self, in_features: int, out_features: int, tile_k: int = 1024, tile_n: int = 32, split_k: int = 1,
                 has_bias: bool = False, prefill_policy: str = "auto", prefill_rows: int = 17):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.tile_k, self.tile_n, self.split_k = tile_k, tile_n, split_k
        if prefill_policy not in ("auto", "fused", "decode_then_gemm"):
            raise ValueError("prefill_policy must be 'auto', 'fused' or 'decode_then_gemm'")
        self.prefill_policy, self.prefill_rows = prefill_policy, int(prefill_rows)
        self._register()
        if has_bias:
            self.register_buffer("bias", torch.empty(out_features, dtype=torch.bfloat16))
        else:
            self.bias = None

    def _stored_shape(self):
        return self.in_features, self.out_features

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        K, N = self.in_features, self.out_features
        x2 = ops._check_x(x, K)
        if self.prefill_policy != "fused" and x2.shape[0] >= max(self.prefill_rows, 17):
            return _decode_then_gemm(self._weight(K, N), K, N, x2, self.bias).view(*x.shape[:-1], N)
        y = ops._linear_call(self._weight(K, N), x2, x2.shape[0], N, self.bias, None,
                             self.split_k if self.split_k > 1 else 0, False)
        return y.view(*x.shape[:-1], N)


class RansFusedLinear(RansLinear):
    """Several projections that read the same input, stored and run as ONE compressed matrix: q|k|v of an
    attention block, gate|up of a SwiGLU MLP (the tensors rans_compress_qkv_fused / rans_compress_gate_up_fused
    produce, comp_inference/comp_inference.py:242-341, saved under the first projection's name,
    comp_inference/rans_saving.py:52-60).  One launch instead of three (two): at batch 1 a launch has a fixed
    cost of several microseconds whatever its size.

    It takes the place of the first projection; ``forward`` runs the whole matrix, remembers the result and
    returns the first block.  The other projections become RansFusedSlice modules that hand out their block of
    the remembered result -- the model's own attention / MLP code stays as it is and must call the first
    projection first (Hugging Face's Llama-family code does)."""

    def __init__(self, in_features, parts, tile_k=1024, tile_n=32, **kw):
        parts = [int(p) for p in parts]
        super().__init__(in_features, sum(parts), tile_k, tile_n, **kw)
        self.parts = parts
        self._last = None

    def forward(self, x):
        self._last = super().forward(x)
        return self._last[..., :self.parts[0]]


class RansFusedSlice(nn.Module):
    """Block [start, end) of the output of the RansFusedLinear that replaced this module's first sibling."""

    def __init__(self, owner: RansFusedLinear, start: int, end: int):
        super().__init__()
        self.__dict__["_owner"] = owner                         # not a submodule: its buffers are saved once
        self.start, self.end = int(start), int(end)
        self.in_features, self.out_features = owner.in_features, self.end - self.start

    def forward(self, x):
        return self._owner._last[..., self.start:self.end]


class RansLMHead(_RansBase):
    """LM head whose weight is stored [V=out, H=in] (pytorch_runtime.py:462-505).

    The reference keeps the head in the embedding's layout so that a tied table is stored once, and
    contracts along the columns of that layout with a kernel of its own.  On a 180 GB part the cheaper
    trade is a second encoding: with ``fast_twin`` (default) the table is decoded once, its transpose
    [H, V] re-encoded on the GPU (bit-exact weights, +0.72 bytes per weight of device memory) and every
    call then runs the ordinary fused decode-linear, which is several times faster than the
    column-contracting kernel.  The twin is built by ``prepare()`` -- the loaders call it once the buffers
    are on the GPU -- or, failing that, by the first forward (which then cannot sit in a captured graph).
    ``fast_twin=False`` keeps the reference's single-copy behaviour.
    """

    def __init__(self, in_features: int, out_features: int, tile_k: int = 1024, tile_n: int = 32,
                 fast_twin: bool = True, twin_tile=(128, 32), prefill_policy: str = "auto", prefill_rows: int = 17):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.tile_k, self.tile_n = tile_k, tile_n
        self.fast_twin, self.twin_tile = bool(fast_twin), (int(twin_tile[0]), int(twin_tile[1]))
        self.prefill_policy, self.prefill_rows = prefill_policy, int(prefill_rows)   # as in RansLinear
        self._register()

    _twin = None

    def _stored_shape(self):
        return self.out_features, self.in_features

    def prepare(self):
        if self.rans_exp_stream.is_cuda and self.rans_exp_states.numel():
            if self.fast_twin:
                self._twin_weight()
            else:
                super().prepare()
        return self

    def _twin_weight(self):
        """Descriptor of the [H, V] re-encoding, built on first use and rebuilt if the buffers change."""
        V, H = self.out_features, self.in_features
        key = (self.rans_exp_stream.data_ptr(), self.rans_exp_states.data_ptr(), self.rans_man_raw.data_ptr())
        if self._twin is None or self._twin[0] != key:
            from . import comp_inference as ci_mod
            w_vh = ops.rans_decompress_bf16(self.rans_exp_stream, self.rans_exp_states, self.rans_exp_tables,
                                            self.rans_exp_slot_map, (V, H), self.rans_exp_tile_offsets,
                                            self.rans_exp_tile_max_lens, int(self.tile_k), int(self.tile_n),
                                            self.rans_man_raw)
            c = ci_mod.compress_weight_cuda(w_vh.t().contiguous(), *self.twin_tile)
            del w_vh
            w, keep = _lib.tiled_weight(c["rans_exp_stream"], c["rans_exp_states"], c["rans_exp_tables"],
                                        c["rans_exp_slot_map"], c["rans_exp_tile_offsets"],
                                        c["rans_exp_tile_max_lens"], c["rans_man_raw"], H, V, int(c["tile_height"]),
                                        int(c["tile_width"]), want_max=True)
            self._twin = (key, w, keep, c)
        return self._twin[1]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        V, H = self.out_features, self.in_features
        x2 = ops._check_x(x, H)
        if self.prefill_policy != "fused" and x2.shape[0] >= max(self.prefill_rows, 17):   # logits of a whole prompt
            if self.fast_twin:
                y = _decode_then_gemm(self._twin_weight(), H, V, x2)
            else:
                y = _decode_then_gemm(self._weight(V, H), H, V, x2, transposed=True)
        elif self.fast_twin:
            y = ops._linear_call(self._twin_weight(), x2, x2.shape[0], V, None, None, 0, False)
        else:
            y = ops._linear_call(self._weight(V, H), x2, x2.shape[0], V, None, None, 0, True)
        return y.view(*x.shape[:-1], V)


class RansEmbedding(_RansBase):
    """nn.Embedding replacement; table stored [V, H] (pytorch_runtime.py:508-549)."""

    def __init__(self, num_embeddings: int, embedding_dim: int, tile_k: int = 1024, tile_n: int = 32):
        super().__init__()
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.tile_k, self.tile_n = tile_k, tile_n
        self._register()

    def _stored_shape(self):
        return self.num_embeddings, self.embedding_dim

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        V, H = self.num_embeddings, self.embedding_dim
        ids = _lib.require_cuda(x, "x").reshape(-1).to(torch.int64).contiguous()
        out = torch.empty((ids.numel(), H), device=x.device, dtype=torch.bfloat16)
        _lib.check(_lib.load().ci_embedding(self._weight(V, H), _lib.ptr(ids), ids.numel(), _lib.ptr(out), H,
                                            _lib.stream()))
        return out.view(*x.shape, H)


def prepare_model(model):
    """Calls ``prepare()`` on every compressed module of a model that already sits on the GPU: descriptors,
    decode tables, the LM head's transposed twin and -- in a tensor-parallel group, where it is a collective
    step every rank must reach -- the agreement on which row-parallel layers exchange inside their kernel.
    After this no forward allocates persistent state or reads anything back from the device, so a decode
    step can be captured in a CUDA graph.  Ends with a status check (raises on a kernel-reported error)."""
    for m in model.modules():
        if isinstance(m, (_RansBase, RansVocabParallelLMHead)):
            m.prepare()
    if torch.cuda.is_available():
        _lib.check_status()
    return model


def _info_shape(info):
    info = [int(v) for v in info.tolist()]
    rank = info[6]
    return tuple(info[11:11 + rank]) if len(info) >= 11 + rank else None


_FUSED_FAMILIES = (("q_proj", ("k_proj", "v_proj")), ("gate_proj", ("up_proj",)))


def _fused_parts(model, name, module, state_dict):
    """[width of every block] if ``name`` holds a concatenated projection in state_dict (its stored width is
    the sum of this module's and its siblings' widths and the siblings have no tensors of their own), else None."""
    parent_name, _, leaf = name.rpartition(".")
    for first, others in _FUSED_FAMILIES:
        if leaf != first or f"{name}.rans_info" not in state_dict:
            continue
        shape = _info_shape(state_dict[f"{name}.rans_info"])
        if shape is None or len(shape) != 2 or shape[1] == module.out_features:
            return None
        parent = model.get_submodule(parent_name) if parent_name else model
        sibs = [getattr(parent, o, None) for o in others]
        if any(s is None or not hasattr(s, "out_features") for s in sibs):
            return None
        if any(f"{parent_name}.{o}.rans_exp_stream" in state_dict or f"{parent_name}.{o}.weight" in state_dict
               for o in others):
            return None
        parts = [module.out_features] + [s.out_features for s in sibs]
        return parts if sum(parts) == shape[1] else None
    return None


def _install_fused(model, name, fused, parts):
    """Puts ``fused`` in place of the first projection and slice modules in place of its siblings."""
    parent_name, _, leaf = name.rpartition(".")
    parent = model.get_submodule(parent_name) if parent_name else model
    others = dict(_FUSED_FAMILIES)[leaf]
    setattr(parent, leaf, fused)
    start = parts[0]
    for o, width in zip(others, parts[1:]):
        setattr(parent, o, RansFusedSlice(fused, start, start + width))
        start += width


def _tile_of(state_dict, layer_configs, name, default_th, default_tw):
    """Tile size of a module: the rans_info record stored next to the stream wins, then config.json's
    layer_configs (under the module's name or its fused alias), then the package default."""
    cfg = layer_configs.get(name) or layer_configs.get(name.replace("q_proj", "qkv_proj")) or \
        layer_configs.get(name.replace("gate_proj", "gate_up_proj")) or {}
    th, tw = cfg.get("tile_height", default_th), cfg.get("tile_width", default_tw)
    info = state_dict.get(f"{name}.rans_info")
    if info is not None and info.numel() >= 11 and int(info[9]) and int(info[10]):
        th, tw = int(info[9]), int(info[10])
    return int(th), int(tw)


def patch_model(model, state_dict, layer_configs=None, default_th=1024, default_tw=32, split_k=1, validate=True):
    """Swaps every module that has ``<name>.rans_exp_stream`` in state_dict for its Rans* counterpart and
    assigns all tensors by name (the body of load_compressed_model_with_auto_model, pytorch_runtime.py:572-637).
    A package saved with fused projections (q|k|v under q_proj, gate|up under gate_proj) gets a RansFusedLinear
    and slice modules.  ``validate``: check every compressed module's metadata on the host first
    (ci_validate_tiled_metadata) and raise on the first inconsistency instead of loading it."""
    layer_configs = layer_configs or {}
    replacements = []
    for name, module in model.named_modules():
        if "lm_head" in name or isinstance(module, (RansLinear, RansEmbedding, RansLMHead, RansFusedSlice)):
            continue
        if f"{name}.rans_exp_stream" not in state_dict:
            continue
        th, tw = _tile_of(state_dict, layer_configs, name, default_th, default_tw)
        if isinstance(module, nn.Linear):
            parts = _fused_parts(model, name, module, state_dict)
            if parts is not None:
                replacements.append((name, RansFusedLinear(module.in_features, parts, th, tw, split_k=split_k), parts))
            else:
                replacements.append((name, RansLinear(module.in_features, module.out_features, th, tw, split_k,
                                                      module.bias is not None), None))
        elif isinstance(module, nn.Embedding):
            replacements.append((name, RansEmbedding(module.num_embeddings, module.embedding_dim, th, tw), None))
    for name, new_layer, parts in replacements:
        if parts is not None:
            _install_fused(model, name, new_layer, parts)
            continue
        parent_name, _, child = name.rpartition(".")
        parent = model.get_submodule(parent_name) if parent_name else model
        setattr(parent, child, new_layer)
    if hasattr(model, "lm_head") and "lm_head.rans_exp_stream" in state_dict and not isinstance(
            model.lm_head, (RansLMHead, RansVocabParallelLMHead)):
        th, tw = _tile_of(state_dict, layer_configs, "lm_head", default_th, default_tw)
        model.lm_head = RansLMHead(model.lm_head.in_features, model.lm_head.out_features, tile_k=th, tile_n=tw)
    if validate:
        for name, module in model.named_modules():
            if isinstance(module, _RansBase) and f"{name}.rans_exp_stream" in state_dict:
                K, N = module._stored_shape()
                c = {k: state_dict[f"{name}.{k}"] for k, _ in _BUFFERS if f"{name}.{k}" in state_dict}
                try:
                    _lib.validate_compressed(c, K, N, int(module.tile_k), int(module.tile_n))
                except RuntimeError as e:
                    raise RuntimeError(f"{name}: {e}") from None
    targets = dict(model.named_buffers())
    targets.update(dict(model.named_parameters()))
    for name, target in targets.items():
        if name in state_dict:
            target.data = state_dict[name].contiguous()
    return model


def load_compressed_model_with_auto_model(model_id: str, safetensors_path: str, split_k: int = 1,
                                          compile_model: bool = False):
    """Loads the dense Hugging Face model, swaps in the compressed modules, moves everything to the GPU
    (pytorch_runtime.py:552-642).  ``compile_model`` is accepted and ignored: there is no tracing compiler here."""
    from safetensors.torch import load_file
    from transformers import AutoModelForCausalLM
    _lib.load()
    model = AutoModelForCausalLM.from_pretrained(model_id, torch_dtype=torch.bfloat16, trust_remote_code=True)
    quant = getattr(model.config, "quantization_config", {}) or {}
    if not isinstance(quant, dict):
        quant = quant.to_dict() if hasattr(quant, "to_dict") else dict(quant)
    state_dict = load_file(safetensors_path, device="cpu")
    patch_model(model, state_dict, quant.get("layer_configs", {}), quant.get("default_tile_height", 1024),
                quant.get("default_tile_width", 32), split_k)
    return prepare_model(model.cuda())


# ------------------------------------------------------------------------- tensor parallel

_COLUMN_PARALLEL = ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj")
_ROW_PARALLEL = ("o_proj", "down_proj")


class RansRowParallelLinear(RansLinear):
    """Row shard (a slice of the input features) of a compressed linear: every rank multiplies its
    slice and the partial outputs are summed over the group -- the only exchange of a tensor-parallel
    block, on activations; compressed weights never move.  The bias is added once, after the sum.

    ``reducer``: a collective.OneShotAllReduce (peer-memory kernel) or None (NCCL).  ``fuse_exchange``: for one
    or two activation rows run ci_linear_allreduce, i.e. let the GEMV's final-reduction warps push their sums to
    the peers themselves instead of writing a partial output for a second kernel.

    Whether a layer takes the fused route is decided ONCE, by ``prepare()``, as the minimum over the group of
    every rank's own answer (shards differ in their deepest tile, so ranks can disagree; a rank that went its own
    way would leave the others waiting for its stores).  ``prepare()`` is therefore a collective call; the model
    patcher makes it for every layer in the same order on every rank, and a forward that finds the layer
    unprepared makes it first (so do not let that first forward happen inside a graph capture)."""

    def __init__(self, *args, group=None, reducer=None, fuse_exchange=True, **kw):
        super().__init__(*args, **kw)
        self.group = group
        self.reducer = reducer          # e.g. collective.OneShotAllReduce; None = NCCL all-reduce
        self.fuse_exchange = bool(fuse_exchange)
        self._fuse_rows = None          # rows up to which the fused exchange is used; None = not decided yet

    @property
    def _fusable(self):
        return bool(self._fuse_rows)

    def prepare(self):
        super().prepare()
        K, N = self.in_features, self.out_features
        ask = getattr(self.reducer, "fused_qualifies", None)
        rows = 0
        if ask is not None and self.rans_exp_stream.is_cuda and self.fuse_exchange:
            ok1 = ask(self._weight(K, N), 1, N)                 # collective: the group's minimum
            ok2 = ask(self._weight(K, N), 2, N)
            rows = 2 if (ok1 and ok2) else (1 if ok1 else 0)
        self._fuse_rows = rows
        return self

    def forward(self, x):
        import torch.distributed as dist
        if self._fuse_rows is None:
            self.prepare()
        K, N = self.in_features, self.out_features
        if self._fuse_rows:
            x2 = ops._check_x(x, K)
            if x2.shape[0] <= self._fuse_rows:                  # decode steps: multiply and exchange in one kernel
                y = self.reducer.fused_linear(self._weight(K, N), x2, N, self.bias)
                return y.view(*x.shape[:-1], N)
        bias, self.bias = self.bias, None
        try:
            y = super().forward(x)
        finally:
            self.bias = bias
        if self.reducer is not None:
            self.reducer(y)
        else:
            dist.all_reduce(y, group=self.group)
        if bias is not None:
            y += bias
        return y


class RansVocabParallelLMHead(nn.Module):
    """One rank's slice of the vocabulary of an LM head stored [V, H]: logits for rows
    [rank * V / world, (rank + 1) * V / world) from this rank's own weights, then an all-gather of the
    [M, V / world] blocks -- the second exchange of a tensor-parallel model, again on activations only.

    The slice is cut out of the compressed arrays on tile rows (sharding.tile_rows), decoded once on the GPU,
    trimmed to the exact rows, transposed and re-encoded as [H, V / world] (the same twin RansLMHead builds for
    the whole table), so each rank holds and decodes 1 / world of the head.  ``gather``: a
    collective.OneShotAllGather (peer-memory kernel for decode-sized outputs) or None (NCCL)."""

    def __init__(self, c, rank, world, group=None, gather=None, device=None, twin_tile=(128, 32)):
        super().__init__()
        from . import sharding
        from . import comp_inference as ci_mod
        V, H = c["shape"]
        if V % world or (V // world) % 2:
            raise ValueError(f"a vocabulary of {V} cannot be cut into {world} even slices")
        self.in_features, self.out_features = H, V
        self.rank, self.world, self.group, self.gather = rank, world, group, gather
        th = c["tile_height"]
        per = V // world
        r0, r1 = rank * per, (rank + 1) * per
        k0, k1 = r0 // th, -(-r1 // th)
        device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        sub = {k: (v.to(device) if torch.is_tensor(v) else v) for k, v in sharding.tile_rows(c, k0, k1).items()}
        rows = sub["shape"][0]
        w = ops.rans_decompress_bf16(sub["rans_exp_stream"], sub["rans_exp_states"], sub["rans_exp_tables"],
                                     sub["rans_exp_slot_map"], (rows, H), sub["rans_exp_tile_offsets"],
                                     sub["rans_exp_tile_max_lens"], th, c["tile_width"], sub["rans_man_raw"])
        mine = w[r0 - k0 * th:r1 - k0 * th].t().contiguous()     # [H, V / world]
        del w, sub
        self._c = ci_mod.compress_weight_cuda(mine, *twin_tile)
        del mine
        self._w, self._keep = _lib.tiled_weight(
            self._c["rans_exp_stream"], self._c["rans_exp_states"], self._c["rans_exp_tables"],
            self._c["rans_exp_slot_map"], self._c["rans_exp_tile_offsets"], self._c["rans_exp_tile_max_lens"],
            self._c["rans_man_raw"], H, per, int(self._c["tile_height"]), int(self._c["tile_width"]), want_max=True)
        self.per_rank = per

    def prepare(self):
        return self

    def forward(self, x):
        import torch.distributed as dist
        H, V = self.in_features, self.out_features
        x2 = ops._check_x(x, H)
        M = x2.shape[0]
        if M >= 17:                                             # a whole prompt: decode once, library GEMM
            y = _decode_then_gemm(self._w, H, self.per_rank, x2)
        else:
            y = ops._linear_call(self._w, x2, M, self.per_rank, None, None, 0, False)
        if self.gather is not None:
            full = self.gather(y)
        else:
            parts = torch.empty((self.world, M, self.per_rank), device=y.device, dtype=y.dtype)
            dist.all_gather_into_tensor(parts, y, group=self.group)
            full = parts.permute(1, 0, 2).reshape(M, V)
        return full.view(*x.shape[:-1], V)


def _state_to_compressed(state_dict, name, th, tw):
    """The package tensors of one module as the dict sharding.shard_rows / shard_cols work on."""
    shape = _info_shape(state_dict[name + ".rans_info"])
    c = {k: state_dict[f"{name}.{k}"] for k in ("rans_exp_stream", "rans_exp_states", "rans_exp_tables",
                                                "rans_exp_slot_map", "rans_exp_tile_offsets",
                                                "rans_exp_tile_max_lens", "rans_man_raw")}
    c.update(shape=(int(shape[0]), int(shape[1])), tile_height=int(th), tile_width=int(tw))
    return c


def _retiled(c, device, tile_height):
    """The same weight re-encoded with another tile height (decoded and encoded on the GPU, bit-exact)."""
    from . import comp_inference as ci_mod
    K, N = c["shape"]
    g = {k: (v.to(device) if torch.is_tensor(v) else v) for k, v in c.items()}
    w = ops.rans_decompress_bf16(g["rans_exp_stream"], g["rans_exp_states"], g["rans_exp_tables"],
                                 g["rans_exp_slot_map"], (K, N), g["rans_exp_tile_offsets"],
                                 g["rans_exp_tile_max_lens"], c["tile_height"], c["tile_width"], g["rans_man_raw"])
    return ci_mod.compress_weight_cuda(w, int(tile_height), c["tile_width"])


def _shard(c, kind, rank, world, device, parts=None, retile=None):
    """This rank's shard of a compressed [K, N] weight.  Cut out of the compressed arrays when the cut falls
    on tile boundaries; otherwise (Llama-2's 11008 rows over 8 ranks = 10.75 tiles) the rank decodes the
    weight once on the GPU and re-encodes its slice.  ``parts``: block widths of a concatenated projection
    (the rank takes its slice of every block).  ``retile``: tile height the shard is to have (re-encoded on the
    GPU if the package has another)."""
    from . import sharding
    from . import comp_inference as ci_mod
    K, N = c["shape"]
    th, tw = c["tile_height"], c["tile_width"]
    want = int(retile) if retile else th
    if kind == "col" and sharding.can_shard_cols(N, tw, world, parts):
        sc = sharding.shard_cols(c, rank, world, parts)
        return sc if want == th else _retiled(sc, device, want)
    if kind == "row" and sharding.can_shard_rows(K, th, world):
        sc = sharding.shard_rows(c, rank, world)
        return sc if want == th else _retiled(sc, device, want)
    if (kind == "col" and any(p % world for p in (parts or [N]))) or (kind == "row" and K % world):
        raise ValueError(f"{K}x{N} cannot be split {kind}-wise over {world} ranks")
    g = {k: (v.to(device) if torch.is_tensor(v) else v) for k, v in c.items()}
    w = ops.rans_decompress_bf16(g["rans_exp_stream"], g["rans_exp_states"], g["rans_exp_tables"],
                                 g["rans_exp_slot_map"], (K, N), g["rans_exp_tile_offsets"],
                                 g["rans_exp_tile_max_lens"], th, tw, g["rans_man_raw"])
    if kind == "col":
        pieces, start = [], 0
        for p in (parts or [N]):
            n = p // world
            pieces.append(w[:, start + rank * n:start + (rank + 1) * n])
            start += p
        part = torch.cat(pieces, dim=1)
    else:
        k = K // world
        part = w[rank * k:(rank + 1) * k]
    return ci_mod.compress_weight_cuda(part.contiguous(), want, tw)


def patch_model_tensor_parallel(model, state_dict, rank, world, group=None, layer_configs=None, default_th=1024,
                                default_tw=32, device=None, oneshot_rows=16, vocab_parallel=True,
                                shard_tile_height=None):
    """patch_model for one rank of a tensor-parallel group.  q/k/v/gate/up projections (separate or
    concatenated) are cut column-wise (each rank owns a slice of the heads / of the FFN width), o/down
    projections row-wise with an all-reduce of their outputs; the LM head is cut by vocabulary with an
    all-gather of the logits (``vocab_parallel``; a vocabulary that does not divide stays replicated); the
    embedding table (one row gather per token, no arithmetic to share) and every uncompressed parameter are
    replicated.  The attention and MLP modules of the model are left as they are: they take the number of heads
    and the FFN width from the tensors they are handed.  ``shard_tile_height``: re-encode every linear shard with
    this tile height at load (on the GPU, bit-exact weights).  A shard's launch is bounded by the length of one
    stream rather than by throughput once the matrix is small, so shards of a package written with tall tiles run
    faster with 64-row tiles (measured on a B200, Llama-2-7B block: 2 GPUs 132 -> 121 us per step, 8 GPUs 53 -> 50);
    None keeps the package's tiles.  Returns the model, moved to ``device`` and prepared (prepare_model), i.e.
    ready for graph capture."""
    layer_configs = layer_configs or {}
    device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
    reducer = gather = None
    head = getattr(model, "lm_head", None)
    if world > 1 and oneshot_rows:
        # outputs of up to `oneshot_rows` activation rows go through the peer-memory exchanges, larger ones
        # (prefill) through NCCL; the exchanges themselves fall back to NCCL where peer memory is not available
        from .collective import OneShotAllGather, OneShotAllReduce
        width = max((m.out_features for m in model.modules() if isinstance(m, nn.Linear) and m is not head), default=0)
        reducer = OneShotAllReduce(group, capacity=oneshot_rows * width, device=device)
    sharded = {}
    for name, module in list(model.named_modules()):
        if not isinstance(module, nn.Linear) or f"{name}.rans_exp_stream" not in state_dict:
            continue
        leaf = name.rsplit(".", 1)[-1]
        kind = "col" if leaf in _COLUMN_PARALLEL else "row" if leaf in _ROW_PARALLEL else None
        if kind is None or world == 1:
            continue
        th, tw = _tile_of(state_dict, layer_configs, name, default_th, default_tw)
        parts = _fused_parts(model, name, module, state_dict) if kind == "col" else None
        c = _shard(_state_to_compressed(state_dict, name, th, tw), kind, rank, world, device, parts,
                   retile=shard_tile_height)
        k, n = c["shape"]
        has_bias = module.bias is not None and parts is None
        if parts is not None:
            new = RansFusedLinear(k, [p // world for p in parts], c["tile_height"], c["tile_width"])
        elif kind == "row":
            new = RansRowParallelLinear(k, n, c["tile_height"], c["tile_width"], 1, has_bias, group=group,
                                        reducer=reducer)
        else:
            new = RansLinear(k, n, c["tile_height"], c["tile_width"], 1, has_bias)
        new.load_compressed(c)
        if has_bias:
            b = state_dict[name + ".bias"].to(torch.bfloat16)
            new.bias = b[rank * n:(rank + 1) * n].contiguous() if kind == "col" else b.contiguous()
        if parts is not None:
            _install_fused(model, name, new, new.parts)
        else:
            parent_name, _, child = name.rpartition(".")
            setattr(model.get_submodule(parent_name) if parent_name else model, child, new)
        sharded[name] = new
    if (world > 1 and vocab_parallel and isinstance(head, nn.Linear) and "lm_head.rans_exp_stream" in state_dict
            and head.out_features % world == 0 and (head.out_features // world) % 2 == 0):
        if oneshot_rows:
            gather = OneShotAllGather(group, capacity=oneshot_rows * (head.out_features // world), device=device)
        th, tw = _tile_of(state_dict, layer_configs, "lm_head", default_th, default_tw)
        model.lm_head = RansVocabParallelLMHead(_state_to_compressed(state_dict, "lm_head", th, tw), rank, world,
                                                group=group, gather=gather, device=device)
        sharded["lm_head"] = model.lm_head
    rest = {k: v for k, v in state_dict.items() if not any(k.startswith(n + ".") for n in sharded)}
    patch_model(model, rest, layer_configs, default_th, default_tw)
    model._ci_exchanges = [e for e in (reducer, gather) if e is not None]
    return prepare_model(model.to(device))


def close_tensor_parallel(model):
    """Releases the peer-mapped exchange buffers of a model patched by patch_model_tensor_parallel (a collective
    step: every rank calls it, with no kernel of the model in flight, before any rank leaves)."""
    for e in getattr(model, "_ci_exchanges", []):
        e.close()
    model._ci_exchanges = []
