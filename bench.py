"""Headline benchmark: Llama-2-7B-shaped greedy decoding with a sharded KV cache.

    python bench.py --gpus 1 --steps 256 --warmup 8
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \\
        bench.py --gpus N --steps K --warmup W [--impl reference]

Config: 32 layers, d_model 4096, 32 heads (head_dim 128), SwiGLU FFN 11008, RMSNorm, vocab 32000, bf16,
random-init weights, synthetic uniform token ids; prefill batch 8 x 2048, then greedy decode.  One *step*
is one decode step for the whole batch (8 new tokens); the metric is decoded tokens per second of the
whole job.  Prints ONE JSON line on rank 0.

Timing: CUDA events on the launching stream, barrier + synchronize on both sides, max over ranks.  Each
step streams every weight shard and the KV cache (>= 1.7 GB per rank), far more than the 126 MB L2, so no
explicit L2 flush is needed between steps.  `e2e` times the same steps driven from the host through the
public API (`model.decode_step`): every step copies its input token ids from pinned host memory and reads
the new ids back.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

BATCH, PROMPT = 8, 2048
MODEL = dict(vocab_size=32000, hidden_size=4096, intermediate_size=11008, num_hidden_layers=32,
             num_attention_heads=32, num_key_value_heads=32, rms_norm_eps=1e-6, rope_theta=10000.0)


class ClockSampler:
    """Samples SM clocks / throttle reasons of the local GPUs with nvidia-smi while a region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.lines, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=lambda: [self.lines.append(l) for l in self.proc.stdout], daemon=True)
        self.thread.start()

    def stop(self, gpu_indices):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, sm_max, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9 or not f[0].isdigit() or int(f[0]) not in gpu_indices:
                continue
            try:
                sm.append(float(f[1])); sm_max.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(sm_max) if sm_max else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def emit(payload):
    print(json.dumps(payload), flush=True)


def visible_gpu_indices(n):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return [int(x) for x in vis.split(",")][:n]
        except ValueError:
            pass
    return list(range(n))


def base_record(args, impl):
    return {
        "metric": "llama2_7b_decode_tokens_per_s", "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic uniform token ids, random-init weights (seed 0, N(0,0.02))", "impl": impl,
        "config": {"model": "Llama-2-7B-shaped (32L, d4096, 32h x 128, ffn 11008, vocab 32000)", "global_batch": BATCH,
                   "seq_len": PROMPT, "prefill": f"{BATCH}x{PROMPT}", "decode": "greedy, sharded KV cache",
                   "parallelism": f"tp{args.gpus}", "l2": "per-step working set (weights + KV, >= 1.7 GB/rank) exceeds the 126 MB L2; no flush"},
    }


# ------------------------------------------------------------------------------------------------
# this framework
# ------------------------------------------------------------------------------------------------

def run_ours(args):
    import torch.distributed as dist

    import tensor_parallel_b200 as tp
    from tensor_parallel_b200.models.llama import LlamaConfig, LlamaForCausalLM
    from tensor_parallel_b200.ops import native

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    torch.manual_seed(0)
    torch.set_default_dtype(torch.bfloat16)
    with torch.device(device):
        model = LlamaForCausalLM(LlamaConfig(**MODEL))
    torch.set_default_dtype(torch.float32)
    model.eval()
    tp_model = tp.tensor_parallel(model, [device])  # distributed mode when a process group exists
    del model
    torch.cuda.empty_cache()

    gen = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, MODEL["vocab_size"], (BATCH, PROMPT), generator=gen)
    max_new = 2 * (args.steps + args.warmup) + 16

    def sync_all():
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(device)

    # build the engine and run one untimed prefill (library / plan / allocation warm-up), then time a second prefill
    tp_model.prefill(prompt, max_new_tokens=max_new)
    sync_all()
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    logits = tp_model.prefill(prompt, max_new_tokens=max_new)
    t1.record()
    sync_all()
    prefill_ms = t0.elapsed_time(t1)
    engine = tp_model._engine
    first = logits.argmax(-1)
    engine.ids[:BATCH].copy_(first)

    for _ in range(args.warmup):
        engine.decode_step(BATCH)
    engine.comm.check_status() if engine.comm is not None else native.device_state(device).check_status()

    sampler = ClockSampler()
    sampler.start()
    # ---- device-timed region: K graph replays ----
    sync_all()
    launches_before = native.launch_count
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        engine.decode_step(BATCH)
    e1.record()
    sync_all()
    ms = e0.elapsed_time(e1)
    # ---- end-to-end region: host-driven steps through the public API ----
    ids_host = torch.empty(BATCH, dtype=torch.int64).pin_memory()
    out_host = torch.empty(BATCH, dtype=torch.int64).pin_memory()
    ids_host.copy_(engine.next_ids[:BATCH])
    sync_all()
    h0 = torch.cuda.Event(enable_timing=True); h1 = torch.cuda.Event(enable_timing=True)
    h0.record()
    for _ in range(args.steps):
        tp_model.decode_step(ids_host, out_host)
        ids_host.copy_(out_host)
    h1.record()
    sync_all()
    e2e_ms = h0.elapsed_time(h1)
    clocks = sampler.stop(visible_gpu_indices(world) if world > 1 else [visible_gpu_indices(max(local_rank + 1, 1))[local_rank]])
    engine.comm.check_status() if engine.comm is not None else native.device_state(device).check_status()

    times = torch.tensor([ms, e2e_ms, prefill_ms], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms, prefill_ms = (float(t) for t in times.tolist())
    if rank == 0:
        rec = base_record(args, "tensor_parallel_b200")
        rec.update({
            "value": BATCH * args.steps / (ms / 1e3), "ms_per_step": ms / args.steps,
            "e2e": {"value": BATCH * args.steps / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": BATCH * 8, "d2h_bytes_per_step": BATCH * 8,
                    "api": "tensor_parallel(...).decode_step(pinned ids) -> pinned next ids"},
            "gpu_launches": engine.kernels_per_step * args.steps, "kernels_per_step": engine.kernels_per_step,
            "prefill_tokens_per_s": BATCH * PROMPT / (prefill_ms / 1e3), "prefill_ms": prefill_ms,
            "clocks": clocks,
        })
        emit(rec)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------
# the reference, unmodified, from baseline/_ref
# ------------------------------------------------------------------------------------------------

def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    ref_dir = os.path.join(REPO, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "tensor_parallel")):
        if rank == 0:
            emit({"impl": "reference", "unavailable": "baseline/_ref/tensor_parallel is not installed (pip --target baseline/_ref /root/reference)"})
        return
    if rank != 0:
        return  # the reference's multi-GPU mode is one process driving all GPUs from threads
    sys.path.insert(0, ref_dir)
    sys.path.insert(0, os.path.join(REPO, "baseline"))
    try:
        import warnings

        warnings.filterwarnings("ignore")
        import tensor_parallel as ref_tp  # the reference package
        from ref_models import RefLlamaConfig, RefLlamaForCausalLM
        from tensor_parallel.slicing_configs import get_llama_config
    except Exception as exc:  # noqa: BLE001
        emit({"impl": "reference", "unavailable": f"import failed: {exc!r}"[:300]})
        return
    if torch.cuda.device_count() < args.gpus:
        emit({"impl": "reference", "unavailable": f"needs {args.gpus} visible GPUs in one process, found {torch.cuda.device_count()}"})
        return
    devices = [torch.device("cuda", i) for i in range(args.gpus)]
    torch.manual_seed(0)
    cfg = RefLlamaConfig(**MODEL)
    torch.set_default_dtype(torch.bfloat16)
    with torch.device(devices[0]):
        model = RefLlamaForCausalLM(cfg)
        for p in model.parameters():
            if p.ndim >= 2:
                torch.nn.init.normal_(p, 0.0, 0.02)
    torch.set_default_dtype(torch.float32)
    model.eval()
    tp_config = get_llama_config(cfg, devices) if args.gpus > 1 else None
    tp_model = ref_tp.TensorParallel(model, device_ids=devices, tensor_parallel_config=tp_config, sharded=False)
    if args.gpus > 1:
        del model
        torch.cuda.empty_cache()

    gen = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, MODEL["vocab_size"], (BATCH, PROMPT), generator=gen).to(devices[0])

    def sync_all():
        for d in devices:
            torch.cuda.synchronize(d)

    with torch.no_grad():
        sync_all()
        t0 = time.perf_counter()
        logits, past = tp_model(prompt, past_key_values=None, use_cache=True, last_only=True)
        sync_all()
        prefill_ms = (time.perf_counter() - t0) * 1e3
        nxt = logits[:, -1].argmax(-1, keepdim=True)
        for _ in range(args.warmup):
            logits, past = tp_model(nxt, past_key_values=past, use_cache=True, last_only=True)
            nxt = logits[:, -1].argmax(-1, keepdim=True)
        sampler = ClockSampler()
        sampler.start()
        sync_all()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        torch.cuda.set_device(devices[0])
        e0.record()
        for _ in range(args.steps):
            logits, past = tp_model(nxt, past_key_values=past, use_cache=True, last_only=True)
            nxt = logits[:, -1].argmax(-1, keepdim=True)
        e1.record()
        sync_all()
        ms = e0.elapsed_time(e1)
        # end to end: ids come from pinned host memory every step and the result is read back
        ids_host = nxt.cpu().pin_memory()
        sync_all()
        h0 = torch.cuda.Event(enable_timing=True); h1 = torch.cuda.Event(enable_timing=True)
        h0.record()
        for _ in range(args.steps):
            ids_dev = ids_host.to(devices[0], non_blocking=True)
            logits, past = tp_model(ids_dev, past_key_values=past, use_cache=True, last_only=True)
            ids_host.copy_(logits[:, -1].argmax(-1, keepdim=True), non_blocking=True)
            torch.cuda.current_stream(devices[0]).synchronize()
        h1.record()
        sync_all()
        e2e_ms = h0.elapsed_time(h1)
        clocks = sampler.stop(visible_gpu_indices(args.gpus))
    rec = base_record(args, "reference")
    rec.update({
        "value": BATCH * args.steps / (ms / 1e3), "ms_per_step": ms / args.steps,
        "e2e": {"value": BATCH * args.steps / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                "h2d_bytes_per_step": BATCH * 8, "d2h_bytes_per_step": BATCH * 8},
        "gpu_launches": 0, "prefill_tokens_per_s": BATCH * PROMPT / (prefill_ms / 1e3), "prefill_ms": prefill_ms, "clocks": clocks,
        "reference_mode": "tensor_parallel.TensorParallel, threaded single process, torch.cuda.nccl collectives, cuBLAS GEMMs, SDPA attention",
    })
    emit(rec)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
