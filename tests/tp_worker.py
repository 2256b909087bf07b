"""Child process of test_gpu_model.py::test_tensor_parallel_logits: one rank of a tensor-parallel group.
usage: python tp_worker.py <package_dir> <reference_logits.pt> <rank> <world> <port>"""
import datetime
import json
import os
import sys

os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"           # peer buffers are never bound to a multicast object
os.environ["NCCL_NVLS_ENABLE"] = "0"

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    pkg, ref_path, rank, world, port = sys.argv[1], sys.argv[2], int(sys.argv[3]), int(sys.argv[4]), sys.argv[5]
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"),
                            timeout=datetime.timedelta(seconds=120))
    import comp_inference_b200 as ci
    from safetensors.torch import load_file
    from transformers import AutoConfig, AutoModelForCausalLM
    with open(os.path.join(pkg, "config.json")) as f:
        raw = json.load(f)
    quant = raw.pop("quantization_config", {}) or {}
    config = AutoConfig.for_model(raw.pop("model_type"), **raw)
    model = AutoModelForCausalLM.from_config(config, torch_dtype=torch.bfloat16)
    state = load_file(os.path.join(pkg, "model.safetensors"), device="cpu")
    model = ci.patch_model_tensor_parallel(model, state, rank, world, None, quant.get("layer_configs", {}),
                                           quant.get("default_tile_height", 1024),
                                           quant.get("default_tile_width", 32)).eval()
    kinds = {type(m).__name__ for m in model.modules()}
    assert "RansRowParallelLinear" in kinds and "RansVocabParallelLMHead" in kinds, kinds
    q = model.model.layers[0].self_attn.q_proj
    fused = bool(quant.get("fused_projections"))
    assert ("RansFusedLinear" in kinds) == fused, (kinds, fused)
    assert q.out_features == (3 if fused else 1) * config.hidden_size // world, (q.out_features, world)
    ref = torch.load(ref_path)
    with torch.no_grad():
        logits = model(ref["ids"].cuda()).logits.float().cpu()
    err = float((logits - ref["logits"]).abs().max() / ref["logits"].abs().max())
    agree = float((logits.argmax(-1) == ref["logits"].argmax(-1)).float().mean())
    print(f"rank {rank}: rel err {err:.3e}, argmax agreement {agree:.3f}", flush=True)
    ok = err <= 3e-2 and agree > 0.9
    # one token per sequence = two activation rows: the row-parallel layers multiply and exchange in one kernel,
    # the logits come back through the one-shot all-gather
    with torch.no_grad():
        logits1 = model(ref["ids"][:, :1].cuda()).logits.float().cpu()
    err1 = float((logits1 - ref["logits1"]).abs().max() / ref["logits1"].abs().max())
    rows = [m for m in model.modules() if type(m).__name__ == "RansRowParallelLinear"]
    native = all(e.native for e in model._ci_exchanges)
    n_fused = sum(m._fusable for m in rows)
    print(f"rank {rank}: single-token rel err {err1:.3e}, fused layers {n_fused}/{len(rows)}, peer memory {native}",
          flush=True)
    ok = ok and err1 <= 3e-2 and (n_fused == len(rows) or not native)
    # every rank must hold the same logits (same summation order everywhere)
    mine = logits1.cuda()
    other = mine.clone()
    dist.broadcast(other, src=0)
    if not torch.equal(mine, other):
        ok = False
        print(f"rank {rank}: ranks disagree on the logits", flush=True)
    try:
        ci.check_status()
        for e in model._ci_exchanges:
            e.check_status()
    except RuntimeError as e:
        ok = False
        print(f"rank {rank}: {e}", flush=True)
    torch.cuda.synchronize()
    ci.close_tensor_parallel(model)           # barrier + release of the peer-mapped buffers, nothing in flight
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    os._exit(0 if ok else 1)                  # communicator clean-up is left to process exit


if __name__ == "__main__":
    main()
