"""Child process of test_gpu_model.py::test_tensor_parallel_logits: one rank of a tensor-parallel group.
usage: python tp_worker.py <package_dir> <reference_logits.pt> <rank> <world> <port>"""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    pkg, ref_path, rank, world, port = sys.argv[1], sys.argv[2], int(sys.argv[3]), int(sys.argv[4]), sys.argv[5]
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=port, NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
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
    assert "RansRowParallelLinear" in kinds, kinds
    q = model.model.layers[0].self_attn.q_proj
    assert q.out_features == config.hidden_size // world, (q.out_features, world)
    ref = torch.load(ref_path)
    with torch.no_grad():
        logits = model(ref["ids"].cuda()).logits.float().cpu()
    err = float((logits - ref["logits"]).abs().max() / ref["logits"].abs().max())
    agree = float((logits.argmax(-1) == ref["logits"].argmax(-1)).float().mean())
    print(f"rank {rank}: rel err {err:.3e}, argmax agreement {agree:.3f}", flush=True)
    ok = err <= 3e-2 and agree > 0.9
    # one token per sequence = two activation rows: the row-parallel layers multiply and exchange in one kernel
    with torch.no_grad():
        logits1 = model(ref["ids"][:, :1].cuda()).logits.float().cpu()
    err1 = float((logits1 - ref["logits1"]).abs().max() / ref["logits1"].abs().max())
    fused = [m._fusable for m in model.modules() if type(m).__name__ == "RansRowParallelLinear"]
    print(f"rank {rank}: single-token rel err {err1:.3e}, fused layers {sum(fused)}/{len(fused)}", flush=True)
    ok = ok and err1 <= 3e-2 and all(fused)
    dist.barrier()
    torch.cuda.synchronize()
    os._exit(0 if ok else 1)                  # communicator clean-up is left to process exit


if __name__ == "__main__":
    main()
