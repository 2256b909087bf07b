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
    """Kept for source compatibility (pytorch_runtime.py:386-394).  Split-K partials of this package
    live in an internal fp32 buffer per device; this returns a view of that buffer's storage size-wise
    compatible placeholder so callers that pass ``workspace=`` keep working."""
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

    def load_compressed(self, c):
        """Adopts the tensors of a dict produced by comp_inference.compress_weight_cuda (or a saved package)."""
        for name, _ in _BUFFERS:
            if name in c:
                setattr(self, name, c[name])
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


def _decode_scratch(device, K, N):
    """One bf16 buffer per device, grown on demand, that the decode-then-GEMM prefill path decodes into."""
    buf = _scratch.get(device)
    if buf is None or buf.numel() < K * N:
        buf = torch.empty(K * N, dtype=torch.bfloat16, device=device)
        _scratch[device] = buf
    return buf[:K * N].view(K, N)


class RansLinear(_RansBase):
    """nn.Linear replacement; weight stored compressed as [K=in, N=out] (pytorch_runtime.py:397-459).

    ``prefill_policy`` chooses what a call with many activation rows runs:
    "fused" (default) the decode-GEMM kernel (tcgen05, the decoded weight never leaves the chip);
    "decode_then_gemm" the stand-alone decoder into a reused per-device scratch buffer followed by a
    library GEMM -- the reference's decompress + triton_matmul pair (comp_inference/triton_gemm.py:324-337) --
    which at present is the faster of the two from ``prefill_rows`` rows up because the decoder runs at
    twice the rate of the GEMM's decode warps and the weight is decoded once however many rows there are.
    """

    def __init__(self, in_features: int, out_features: int, tile_k: int = 1024, tile_n: int = 32, split_k: int = 1,
                 has_bias: bool = False, prefill_policy: str = "fused", prefill_rows: int = 256):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.tile_k, self.tile_n, self.split_k = tile_k, tile_n, split_k
        if prefill_policy not in ("fused", "decode_then_gemm"):
            raise ValueError("prefill_policy must be 'fused' or 'decode_then_gemm'")
        self.prefill_policy, self.prefill_rows = prefill_policy, int(prefill_rows)
        self._register()
        if has_bias:
            self.register_buffer("bias", torch.empty(out_features, dtype=torch.bfloat16))
        else:
            self.bias = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        K, N = self.in_features, self.out_features
        x2 = ops._check_x(x, K)
        if self.prefill_policy == "decode_then_gemm" and x2.shape[0] >= self.prefill_rows:
            w = _decode_scratch(x2.device, K, N)
            _lib.check(_lib.load().ci_decode_bf16(self._weight(K, N), _lib.ptr(w), _lib.stream()))
            y = torch.matmul(x2, w)
            if self.bias is not None:
                y += self.bias
            return y.view(*x.shape[:-1], N)
        y = ops._linear_call(self._weight(K, N), x2, x2.shape[0], N, self.bias, None,
                             self.split_k if self.split_k > 1 else 0, False)
        return y.view(*x.shape[:-1], N)


class RansLMHead(_RansBase):
    """LM head whose weight is stored [V=out, H=in] (pytorch_runtime.py:462-505).

    The reference keeps the head in the embedding's layout so that a tied table is stored once, and
    contracts along the columns of that layout with a kernel of its own.  On a 180 GB part the cheaper
    trade is a second encoding: with ``fast_twin`` (default) the first forward decodes the table once,
    re-encodes its transpose [H, V] on the GPU (bit-exact weights, +0.72 bytes per weight of device
    memory) and every call then runs the ordinary fused decode-linear, which is several times faster
    than the column-contracting kernel.  ``fast_twin=False`` keeps the reference's single-copy behaviour.
    """

    def __init__(self, in_features: int, out_features: int, tile_k: int = 1024, tile_n: int = 32,
                 fast_twin: bool = True, twin_tile=(128, 32)):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.tile_k, self.tile_n = tile_k, tile_n
        self.fast_twin, self.twin_tile = bool(fast_twin), (int(twin_tile[0]), int(twin_tile[1]))
        self._register()

    _twin = None

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
        if self.fast_twin:
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

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        V, H = self.num_embeddings, self.embedding_dim
        ids = _lib.require_cuda(x, "x").reshape(-1).to(torch.int64).contiguous()
        out = torch.empty((ids.numel(), H), device=x.device, dtype=torch.bfloat16)
        _lib.check(_lib.load().ci_embedding(self._weight(V, H), _lib.ptr(ids), ids.numel(), _lib.ptr(out), H,
                                            _lib.stream()))
        return out.view(*x.shape, H)


def patch_model(model, state_dict, layer_configs=None, default_th=1024, default_tw=32, split_k=1):
    """Swaps every module that has ``<name>.rans_exp_stream`` in state_dict for its Rans* counterpart and
    assigns all tensors by name (the body of load_compressed_model_with_auto_model, pytorch_runtime.py:572-637)."""
    layer_configs = layer_configs or {}
    replacements = []
    for name, module in model.named_modules():
        if "lm_head" in name or isinstance(module, (RansLinear, RansEmbedding, RansLMHead)):
            continue
        if f"{name}.rans_exp_stream" not in state_dict:
            continue
        th = layer_configs.get(name, {}).get("tile_height", default_th)
        tw = layer_configs.get(name, {}).get("tile_width", default_tw)
        if isinstance(module, nn.Linear):
            replacements.append((name, RansLinear(module.in_features, module.out_features, th, tw, split_k,
                                                  module.bias is not None)))
        elif isinstance(module, nn.Embedding):
            replacements.append((name, RansEmbedding(module.num_embeddings, module.embedding_dim, th, tw)))
    for name, new_layer in replacements:
        parent_name, _, child = name.rpartition(".")
        parent = model.get_submodule(parent_name) if parent_name else model
        setattr(parent, child, new_layer)
    if hasattr(model, "lm_head") and "lm_head.rans_exp_stream" in state_dict:
        th = layer_configs.get("lm_head", {}).get("tile_height", default_th)
        tw = layer_configs.get("lm_head", {}).get("tile_width", default_tw)
        model.lm_head = RansLMHead(model.lm_head.in_features, model.lm_head.out_features, tile_k=th, tile_n=tw)
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
    return model.cuda()


# ------------------------------------------------------------------------- tensor parallel

_COLUMN_PARALLEL = ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj")
_ROW_PARALLEL = ("o_proj", "down_proj")


class RansRowParallelLinear(RansLinear):
    """Row shard (a slice of the input features) of a compressed linear: every rank multiplies its
    slice and the partial outputs are summed over the group -- the only exchange of a tensor-parallel
    block, on activations; compressed weights never move.  The bias is added once, after the sum.

    ``reducer``: a collective.OneShotAllReduce (peer-memory kernel) or None (NCCL).  ``fuse_exchange``: for one
    or two activation rows run ci_linear_allreduce, i.e. let the GEMV's final-reduction warps push their sums to
    the peers themselves instead of writing a partial output for a second kernel.  On 2 B200s the two routes are
    within 1 % of each other (the separate kernel overlaps with the next kernel's preamble and synchronises the
    ranks once instead of once per column group); more activation rows always take the separate route."""

    def __init__(self, *args, group=None, reducer=None, fuse_exchange=True, **kw):
        super().__init__(*args, **kw)
        self.group = group
        self.reducer = reducer          # e.g. collective.OneShotAllReduce; None = NCCL all-reduce
        self._fusable = bool(fuse_exchange)

    def forward(self, x):
        import torch.distributed as dist
        fused = getattr(self.reducer, "fused_linear", None)
        if fused is not None and self._fusable:
            K, N = self.in_features, self.out_features
            x2 = ops._check_x(x, K)
            if x2.shape[0] <= 2:                                # decode steps: multiply and exchange in one kernel
                y = fused(self._weight(K, N), x2, N, self.bias)
                if y is not None:
                    return y.view(*x.shape[:-1], N)
                self._fusable = False                           # this weight does not qualify: do not ask again
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


def _state_to_compressed(state_dict, name, th, tw):
    """The package tensors of one module as the dict sharding.shard_rows / shard_cols work on."""
    info = state_dict[name + ".rans_info"].tolist()
    rank = info[6]
    shape = tuple(info[11:11 + rank]) if len(info) >= 11 + rank else None
    c = {k: state_dict[f"{name}.{k}"] for k in ("rans_exp_stream", "rans_exp_states", "rans_exp_tables",
                                                "rans_exp_slot_map", "rans_exp_tile_offsets",
                                                "rans_exp_tile_max_lens", "rans_man_raw")}
    if len(info) >= 11 and info[9] and info[10]:
        th, tw = int(info[9]), int(info[10])
    c.update(shape=(int(shape[0]), int(shape[1])), tile_height=int(th), tile_width=int(tw))
    return c


def _shard(c, kind, rank, world, device):
    """This rank's shard of a compressed [K, N] weight.  Cut out of the compressed arrays when the cut falls
    on tile boundaries; otherwise (Llama-2's 11008 rows over 8 ranks = 10.75 tiles) the rank decodes the
    weight once on the GPU and re-encodes its slice."""
    from . import sharding
    from . import comp_inference as ci_mod
    K, N = c["shape"]
    th, tw = c["tile_height"], c["tile_width"]
    if kind == "col" and sharding.can_shard_cols(N, tw, world):
        return sharding.shard_cols(c, rank, world)
    if kind == "row" and sharding.can_shard_rows(K, th, world):
        return sharding.shard_rows(c, rank, world)
    if (kind == "col" and N % world) or (kind == "row" and K % world):
        raise ValueError(f"{K}x{N} cannot be split {kind}-wise over {world} ranks")
    g = {k: (v.to(device) if torch.is_tensor(v) else v) for k, v in c.items()}
    w = ops.rans_decompress_bf16(g["rans_exp_stream"], g["rans_exp_states"], g["rans_exp_tables"],
                                 g["rans_exp_slot_map"], (K, N), g["rans_exp_tile_offsets"],
                                 g["rans_exp_tile_max_lens"], th, tw, g["rans_man_raw"])
    if kind == "col":
        n = N // world
        part = w[:, rank * n:(rank + 1) * n]
    else:
        k = K // world
        part = w[rank * k:(rank + 1) * k]
    return ci_mod.compress_weight_cuda(part.contiguous(), th, tw)


def patch_model_tensor_parallel(model, state_dict, rank, world, group=None, layer_configs=None, default_th=1024,
                                default_tw=32, device=None, oneshot_rows=16):
    """patch_model for one rank of a tensor-parallel group.  q/k/v/gate/up projections are cut column-wise
    (each rank owns a slice of the heads / of the FFN width), o/down projections row-wise with an all-reduce
    of their outputs; embedding, LM head and every uncompressed parameter are replicated.  The attention
    and MLP modules of the model are left as they are: they take the number of heads and the FFN width
    from the tensors they are handed.  Returns the model, moved to ``device``."""
    layer_configs = layer_configs or {}
    device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
    reducer = None
    if world > 1 and oneshot_rows:
        # outputs of up to `oneshot_rows` activation rows go through the peer-memory all-reduce, larger ones
        # (prefill) through NCCL; the reducer itself falls back to NCCL where peer memory is not available
        from .collective import OneShotAllReduce
        width = max((m.out_features for m in model.modules() if isinstance(m, nn.Linear)), default=0)
        reducer = OneShotAllReduce(group, capacity=oneshot_rows * width, device=device)
    sharded = {}
    for name, module in list(model.named_modules()):
        if not isinstance(module, nn.Linear) or f"{name}.rans_exp_stream" not in state_dict:
            continue
        leaf = name.rsplit(".", 1)[-1]
        kind = "col" if leaf in _COLUMN_PARALLEL else "row" if leaf in _ROW_PARALLEL else None
        if kind is None or world == 1:
            continue
        th = layer_configs.get(name, {}).get("tile_height", default_th)
        tw = layer_configs.get(name, {}).get("tile_width", default_tw)
        c = _shard(_state_to_compressed(state_dict, name, th, tw), kind, rank, world, device)
        k, n = c["shape"]
        has_bias = module.bias is not None
        if kind == "row":
            new = RansRowParallelLinear(k, n, c["tile_height"], c["tile_width"], 1, has_bias, group=group,
                                        reducer=reducer)
        else:
            new = RansLinear(k, n, c["tile_height"], c["tile_width"], 1, has_bias)
        new.load_compressed(c)
        if has_bias:
            b = state_dict[name + ".bias"].to(torch.bfloat16)
            new.bias = b[rank * n:(rank + 1) * n].contiguous() if kind == "col" else b.contiguous()
        parent_name, _, child = name.rpartition(".")
        setattr(model.get_submodule(parent_name) if parent_name else model, child, new)
        sharded[name] = new
    rest = {k: v for k, v in state_dict.items() if not any(k.startswith(n + ".") for n in sharded)}
    patch_model(model, rest, layer_configs, default_th, default_tw)
    return model.to(device)
