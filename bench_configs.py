"""The other model configurations of the benchmark plan, through the public API (one process per GPU):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port P \\
        bench_configs.py --config falcon40b_infer|flan_t5_xl_train|opt13b_train [--layers L]

* ``falcon40b_infer``  : Falcon-40B-shaped (60 layers, d 8192, 128 query / 8 KV heads of 64, parallel block, FFN 32768
  GeLU, vocab 65024), bf16; prefill batch 16 x 1024 then 128 greedy tokens with the head-sharded KV cache.
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True, choices=["falcon40b_infer", "flan_t5_xl_train", "opt13b_train"])
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=2)
    args = ap.parse_args()
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
        from tensor_parallel_b200.models.generation import generate

        prompt = torch.randint(0, cfg.vocab_size, (16, 1024), generator=gen).to(device)
        with torch.no_grad():
            generate(tp_model, prompt[:, :64], max_new_tokens=2)  # warm-up
            sync()
            e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            e0.record()
            out = tp_model(input_ids=prompt, use_cache=True)
            e1.record()
            past, nxt = out["past_key_values"], out["logits"][:, -1].argmax(-1, keepdim=True)
            new_tokens = 127
            for _ in range(new_tokens):
                out = tp_model(input_ids=nxt, past_key_values=past, use_cache=True)
                past, nxt = out["past_key_values"], out["logits"][:, -1].argmax(-1, keepdim=True)
            e2.record()
            sync()
        t = torch.tensor([e0.elapsed_time(e1), e1.elapsed_time(e2)], device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        rec.update(prefill_ms=float(t[0]), prefill_tokens_per_s=16 * 1024 / (float(t[0]) / 1e3), decode_ms_per_step=float(t[1]) / new_tokens,
                   decode_tokens_per_s=16 * new_tokens / (float(t[1]) / 1e3))
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
