"""The other model configurations of the benchmark plan, through the public API (one process per GPU):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port P \\
        bench_configs.py --config falcon40b_infer|flan_t5_xl_train|opt13b_train [--layers L] [--impl reference]

``--impl reference`` (``falcon40b_infer`` only) runs the unmodified reference from ``baseline/_ref`` with its own
``get_refined_web_config`` rule table on a plain-PyTorch model of the same shape (``baseline/ref_models.py``): rank 0 drives all
GPUs from threads, which is the reference's multi-GPU mode.

* ``falcon40b_infer``  : Falcon-40B-shaped (60 layers, d 8192, 128 query / 8 KV heads of 64, parallel block, FFN 32768
  GeLU, vocab 65024), bf16; prefill batch 16 x 1024 then 128 greedy tokens with the head-sharded KV cache, served by the
  kernel-level engine (four kernels per layer and decode step, one fused GEMM + all-reduce per layer).
* ``flan_t5_xl_train`` : FLAN-T5-XL-shaped (24+24 layers, d 2048, 32 heads of 64, gated-GeLU FFN 5120, vocab 32128), bf16,
  seq2seq training step with ``sharded=True`` (ZeRO-3 inside the TP group); encoder batch 16 x 512, targets 16 x 128.
* ``opt13b_train``     : OPT-13B-shaped training step, micro-batch 4 x 2048, ``sharded=True``, AdamW.

Synthetic uniform token ids, random-init weights.  ``--layers`` shrinks the depth (the JSON line says so).  Times are
CUDA-event times, max over ranks.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)


def falcon_reference(args):
    """Falcon-40B-shaped inference on the reference (threaded mode, its RefinedWeb rule table, cuBLAS + SDPA + torch.cuda.nccl)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    ref_dir = os.path.join(REPO, "baseline", "_ref")
    sys.path.insert(0, ref_dir)
    sys.path.insert(0, os.path.join(REPO, "baseline"))
    import warnings

    warnings.filterwarnings("ignore")
    try:
        import tensor_parallel as ref_tp
        from ref_models import RefFalconConfig, RefFalconForCausalLM
        from tensor_parallel.slicing_configs import get_refined_web_config
    except Exception as exc:  # noqa: BLE001
        print(json.dumps({"config": args.config, "impl": "reference", "unavailable": repr(exc)[:200]}), flush=True)
        return
    gpus = args.gpus or torch.cuda.device_count()
    devices = [torch.device("cuda", i) for i in range(gpus)]
    torch.manual_seed(0)
    cfg = RefFalconConfig(n_layer=args.layers or 60)
    torch.set_default_dtype(torch.bfloat16)
    with torch.device(devices[0]):
        model = RefFalconForCausalLM(cfg).eval()
        for p in model.parameters():
            if p.ndim >= 2:
                torch.nn.init.normal_(p, 0.0, 0.02)
    torch.set_default_dtype(torch.float32)
    tp_model = ref_tp.TensorParallel(model, device_ids=devices, tensor_parallel_config=get_refined_web_config(cfg, devices) if gpus > 1 else None,
                                     sharded=False)
    if gpus > 1:
        del model
        torch.cuda.empty_cache()
    gen = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, cfg.vocab_size, (16, 1024), generator=gen).to(devices[0])
    new_tokens = args.decode_steps

    def sync():
        for d in devices:
            torch.cuda.synchronize(d)

    with torch.no_grad():
        tp_model(prompt[:, :64], past_key_values=None, use_cache=True, last_only=True)  # warm-up
        sync()
        torch.cuda.set_device(devices[0])
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
        logits, past = tp_model(prompt, past_key_values=None, use_cache=True, last_only=True)
        e1.record()
        nxt = logits[:, -1].argmax(-1, keepdim=True)
        for _ in range(new_tokens):
            logits, past = tp_model(nxt, past_key_values=past, use_cache=True, last_only=True)
            nxt = logits[:, -1].argmax(-1, keepdim=True)
        e2.record()
        sync()
    print(json.dumps({"config": args.config, "impl": "reference", "n_gpus": gpus, "layers": args.layers or "full", "dtype": "bf16",
                      "data": "synthetic", "prefill_ms": e0.elapsed_time(e1), "prefill_tokens_per_s": 16 * 1024 / (e0.elapsed_time(e1) / 1e3),
                      "decode_steps": new_tokens, "decode_ms_per_step": e1.elapsed_time(e2) / new_tokens,
                      "decode_tokens_per_s": 16 * new_tokens / (e1.elapsed_time(e2) / 1e3),
                      "reference_mode": "tensor_parallel.TensorParallel, threaded, get_refined_web_config"}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True, choices=["falcon40b_infer", "flan_t5_xl_train", "opt13b_train"])
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--gpus", type=int, default=0, help="reference arm: GPUs driven by rank 0 (default: all visible)")
    ap.add_argument("--decode-steps", type=int, default=127)
    args = ap.parse_args()
    if args.impl == "reference":
        if args.config != "falcon40b_infer":
            raise SystemExit("the reference arm of bench_configs.py covers falcon40b_infer (bench.py holds the Llama arms)")
        return falcon_reference(args)
    import tensor_parallel_b200 as tp
    from tensor_parallel_b200.ops import native

    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    torch.manual_seed(0)
    torch.set_default_dtype(torch.bfloat16)
    with torch.device(device):
        if args.config == "falcon40b_infer":
            from tensor_parallel_b200.models.falcon import FalconConfig, FalconForCausalLM

            cfg = FalconConfig.falcon_40b()
            if args.layers:
                cfg.n_layer = cfg.num_hidden_layers = args.layers
            model = FalconForCausalLM(cfg).eval()
        elif args.config == "flan_t5_xl_train":
            from tensor_parallel_b200.models.t5 import T5Config, T5ForConditionalGeneration

            cfg = T5Config.flan_t5_xl()
            if args.layers:
                cfg.num_layers = cfg.num_decoder_layers = args.layers
            model = T5ForConditionalGeneration(cfg)
        else:
            from tensor_parallel_b200.models.opt import OPTConfig, OPTForCausalLM

            cfg = OPTConfig.opt_13b()
            if args.layers:
                cfg.num_hidden_layers = args.layers
            model = OPTForCausalLM(cfg)
    torch.set_default_dtype(torch.float32)
    n_params = sum(p.numel() for p in model.parameters())
    training = args.config.endswith("_train")
    tp_model = tp.tensor_parallel(model, [device], sharded=training) if world > 1 else model
    del model
    torch.cuda.empty_cache()

    def sync():
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(device)

    gen = torch.Generator().manual_seed(1)
    rec = {"config": args.config, "n_gpus": world, "layers": args.layers or "full", "params": n_params, "dtype": "bf16",
           "impl": "tensor_parallel_b200", "data": "synthetic"}
    before = native.launch_count
    if args.config == "falcon40b_infer":
        if world == 1:
            tp_model = tp.TensorParallel(tp_model, [device])  # one device: the module itself, plus the serving API
        prompt = torch.randint(0, cfg.vocab_size, (16, 1024), generator=gen)
        new_tokens = args.decode_steps
        with torch.no_grad():
            tp_model.prefill(prompt, max_new_tokens=new_tokens + 8)  # builds the engine; library / allocation warm-up
            engine = tp_model._engine
            sync()
            e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            e0.record()
            logits = tp_model.prefill(prompt, max_new_tokens=new_tokens + 8)
            e1.record()
            engine.ids[:16].copy_(logits.argmax(-1))
            engine.decode_step(16)  # captures the graph (untimed)
            sync()
            e1b = torch.cuda.Event(enable_timing=True)
            e1b.record()
            for _ in range(new_tokens - 1):
                engine.decode_step(16)
            e2.record()
            sync()
            engine.check_status()
        t = torch.tensor([e0.elapsed_time(e1), e1b.elapsed_time(e2)], device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        rec.update(prefill_ms=float(t[0]), prefill_tokens_per_s=16 * 1024 / (float(t[0]) / 1e3), decode_ms_per_step=float(t[1]) / (new_tokens - 1),
                   decode_tokens_per_s=16 * (new_tokens - 1) / (float(t[1]) / 1e3), kernels_per_step=engine.kernels_per_step,
                   served_by="DecoderEngine (CUDA graph)")
    else:
        opt = tp.optim.AdamW(tp_model.parameters(), lr=1e-5, weight_decay=0.1)
        if args.config == "flan_t5_xl_train":
            batches = [dict(input_ids=torch.randint(0, cfg.vocab_size, (16, 512), generator=gen).pin_memory(),
                            labels=torch.randint(0, cfg.vocab_size, (16, 128), generator=gen).pin_memory()) for _ in range(2)]
            tokens = 16 * (512 + 128)
        else:
            ids = [torch.randint(0, cfg.vocab_size, (4, 2048), generator=gen).pin_memory() for _ in range(2)]
            batches = [dict(input_ids=x, labels=x) for x in ids]
            tokens = 4 * 2048

        def step(i):
            b = {k: v.to(device, non_blocking=True) for k, v in batches[i % 2].items()}
            loss = tp_model(**b)["loss"]
            loss.backward()
            opt.step()
            opt.zero_grad(set_to_none=True)
            return loss.detach()

        for i in range(args.warmup):
            step(i)
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.steps):
            loss_host = step(i).float().cpu()
        e1.record()
        sync()
        t = torch.tensor([e0.elapsed_time(e1)], device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0]) / args.steps
        rec.update(ms_per_step=ms, train_tokens_per_s=tokens / (ms / 1e3), loss=float(loss_host), sharded=world > 1)
    rec.update(native_kernel_launches=native.launch_count - before, peak_mem_gb=torch.cuda.max_memory_allocated(device) / 2**30)
    if rank == 0:
        print(json.dumps(rec), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
