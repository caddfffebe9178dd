"""Training-throughput benchmark (secondary to bench.py): one optimizer step of a decoder on N GPUs.

    python bench_train.py --model llama7b --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \\
        bench_train.py --model opt13b --gpus N [--impl reference]

Models: ``llama7b`` (Llama-2-7B-shaped) and ``opt13b`` (OPT-13B-shaped: 40 layers, d 5120, 40 heads, FFN 20480,
vocab 50272), bf16, random init, micro-batch 4 x 2048 synthetic tokens, labels = inputs, ``sharded=True`` (ZeRO-3
for the parameters tensor parallelism leaves whole), AdamW.  A step = forward + backward + optimizer step; every
step copies its batch from pinned host memory and reads the loss back.  Prints one JSON line on rank 0; times
are CUDA-event times, max over ranks.  ``--layers`` shrinks the depth for quick probes (the line then says so).
"""
import argparse
import json
import os
import sys

import torch

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)
BATCH, SEQ = 4, 2048


def build_ours(name, layers, device):
    from tensor_parallel_b200.models.llama import LlamaConfig, LlamaForCausalLM
    from tensor_parallel_b200.models.opt import OPTConfig, OPTForCausalLM

    torch.set_default_dtype(torch.bfloat16)
    with torch.device(device):
        if name == "llama7b":
            cfg = LlamaConfig(num_hidden_layers=layers or 32, fused_lm_loss=True)
            model = LlamaForCausalLM(cfg)
        else:
            cfg = OPTConfig.opt_13b()
            cfg.num_hidden_layers = layers or 40
            model = OPTForCausalLM(cfg)
    torch.set_default_dtype(torch.float32)
    return model, cfg.vocab_size


def train_ours(model_name: str, steps: int, warmup: int, layers: int = 0, no_master: bool = False) -> dict:
    """Times ``steps`` optimizer steps of this framework on the process group that is already initialised (or on one
    GPU); returns the result record (meaningful on rank 0).  The caller owns process-group set-up and tear-down."""
    import gc

    import torch.distributed as dist

    import tensor_parallel_b200 as tp
    from tensor_parallel_b200.ops import native

    world = dist.get_world_size() if dist.is_initialized() else 1
    device = torch.device("cuda", torch.cuda.current_device())
    torch.manual_seed(0)
    model, vocab = build_ours(model_name, layers, device)
    tp_model = tp.tensor_parallel(model, [device], sharded=True) if world > 1 else model
    del model
    gc.collect()
    torch.cuda.empty_cache()
    opt = tp.optim.AdamW(tp_model.parameters(), lr=1e-5, weight_decay=0.1, master_weights=not no_master)
    gen = torch.Generator().manual_seed(1)
    batches = [torch.randint(0, vocab, (BATCH, SEQ), generator=gen).pin_memory() for _ in range(4)]

    def step(i):
        ids = batches[i % len(batches)].to(device, non_blocking=True)  # host -> device copy of this step's batch
        out = tp_model(input_ids=ids, labels=ids)
        out["loss"].backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return out["loss"].detach()

    def sync():
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(device)

    for i in range(warmup):
        loss = step(i)
    sync()
    before = native.launch_count
    torch.cuda.reset_peak_memory_stats(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        loss = step(warmup + i)
        loss_host = loss.float().cpu()  # device -> host read of the step's result
    e1.record()
    sync()
    ms = torch.tensor([e0.elapsed_time(e1)], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    if hasattr(tp_model, "check_status"):
        tp_model.check_status()
    ms = float(ms.item())
    record = {
        "metric": f"{model_name}_train_tokens_per_s", "value": BATCH * SEQ * steps / (ms / 1e3), "unit": "tokens/s",
        "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms / steps, "dtype": "bf16",
        "impl": "tensor_parallel_b200", "loss": float(loss_host), "layers": layers or "full",
        "gpu_launches": native.launch_count - before, "peak_mem_gb": torch.cuda.max_memory_allocated(device) / 2**30,
        "config": {"micro_batch": BATCH, "seq_len": SEQ, "optimizer": "AdamW (fused, fp32 master weights)" if not no_master else "AdamW (fused)",
                   "sharded": world > 1, "parallelism": f"tp{world}"},
        "h2d_bytes_per_step": BATCH * SEQ * 8, "d2h_bytes_per_step": 4,
    }
    del tp_model, opt
    gc.collect()
    torch.cuda.empty_cache()
    return record


def run_ours(args):
    import torch.distributed as dist

    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    record = train_ours(args.model, args.steps, args.warmup, args.layers, args.no_master)
    if rank == 0:
        print(json.dumps(record), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def train_reference(model_name: str, gpus: int, steps: int, warmup: int, layers: int = 0) -> dict:
    """The same step on the unmodified reference (``baseline/_ref``): its ``TensorParallel`` in threaded mode with
    ``sharded=True``, a plain-PyTorch Llama, ``torch.optim.AdamW(fused=True)``.  Called on rank 0 only."""
    import gc

    sys.path.insert(0, os.path.join(REPO, "baseline", "_ref"))
    sys.path.insert(0, os.path.join(REPO, "baseline"))
    import warnings

    warnings.filterwarnings("ignore")
    try:
        import tensor_parallel as ref_tp
        from ref_models import RefLlamaConfig, RefLlamaForCausalLM
        from tensor_parallel.slicing_configs import get_llama_config
    except Exception as exc:  # noqa: BLE001
        return {"impl": "reference", "unavailable": repr(exc)[:200]}
    if model_name != "llama7b":
        return {"impl": "reference", "unavailable": "reference arm implemented for llama7b only"}
    devices = [torch.device("cuda", i) for i in range(gpus)]
    torch.manual_seed(0)
    cfg = RefLlamaConfig(num_hidden_layers=layers or 32)
    torch.set_default_dtype(torch.bfloat16)
    with torch.device(devices[0]):
        model = RefLlamaForCausalLM(cfg)
        for p in model.parameters():
            if p.ndim >= 2:
                torch.nn.init.normal_(p, 0.0, 0.02)
    torch.set_default_dtype(torch.float32)
    tp_model = ref_tp.TensorParallel(model, device_ids=devices, tensor_parallel_config=get_llama_config(cfg, devices) if gpus > 1 else None,
                                     sharded=gpus > 1)
    if gpus > 1:
        del model
        gc.collect()
        torch.cuda.empty_cache()
    opt = torch.optim.AdamW(tp_model.parameters(), lr=1e-5, weight_decay=0.1, fused=True)
    gen = torch.Generator().manual_seed(1)
    batches = [torch.randint(0, cfg.vocab_size, (BATCH, SEQ), generator=gen).pin_memory() for _ in range(4)]

    def step(i):
        ids = batches[i % 4].to(devices[0], non_blocking=True)
        logits, _ = tp_model(ids, past_key_values=None, use_cache=False)
        loss = torch.nn.functional.cross_entropy(logits[:, :-1].float().reshape(-1, logits.shape[-1]), ids[:, 1:].reshape(-1))
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss.detach()

    for i in range(warmup):
        step(i)
    for d in devices:
        torch.cuda.synchronize(d)
    torch.cuda.set_device(devices[0])
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        loss_host = step(warmup + i).float().cpu()
    e1.record()
    for d in devices:
        torch.cuda.synchronize(d)
    ms = e0.elapsed_time(e1)
    record = {"metric": f"{model_name}_train_tokens_per_s", "value": BATCH * SEQ * steps / (ms / 1e3), "unit": "tokens/s",
              "n_gpus": gpus, "steps": steps, "warmup": warmup, "ms_per_step": ms / steps, "dtype": "bf16",
              "impl": "reference", "loss": float(loss_host), "layers": layers or "full",
              "peak_mem_gb": torch.cuda.max_memory_allocated(devices[0]) / 2**30,
              "config": {"micro_batch": BATCH, "seq_len": SEQ, "optimizer": "torch.optim.AdamW(fused=True)", "sharded": gpus > 1,
                         "parallelism": f"tp{gpus}"},
              "h2d_bytes_per_step": BATCH * SEQ * 8, "d2h_bytes_per_step": 4}
    del tp_model, opt
    gc.collect()
    torch.cuda.empty_cache()
    return record


def run_reference(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    print(json.dumps(train_reference(args.model, args.gpus, args.steps, args.warmup, args.layers)), flush=True)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama7b", choices=["llama7b", "opt13b"])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--no-master", action="store_true", help="no fp32 master copy of bf16 parameters (saves 4 bytes / parameter)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    a = ap.parse_args()
    run_reference(a) if a.impl == "reference" else run_ours(a)
