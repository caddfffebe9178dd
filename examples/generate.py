"""Text generation with a head-sharded KV cache.

    python examples/generate.py                                      # two CPU ranks, tiny model, generic path
    python examples/generate.py --devices cuda:0 --dtype bfloat16    # kernel-level serving engine, CUDA-graph decode
    torchrun --standalone --nproc-per-node 8 examples/generate.py --devices cuda --dtype bfloat16 --size 7b

On CUDA with bf16 Llama-shaped shards ``generate()`` runs the serving engine (prefill + one CUDA graph per decode step,
row-parallel GEMMs fused with their all-reduce); everything else goes through the generic loop.  Greedy, top-p and beam
search are available either way.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import tensor_parallel_b200 as tp  # noqa: E402
from tensor_parallel_b200.models.llama import LlamaConfig, LlamaForCausalLM  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--devices", nargs="+", default=["cpu", "cpu"])
    ap.add_argument("--dtype", default="float32")
    ap.add_argument("--size", default="tiny", choices=["tiny", "7b"])
    ap.add_argument("--new-tokens", type=int, default=8)
    args = ap.parse_args()
    devices = args.devices
    if "LOCAL_RANK" in os.environ:
        if not torch.distributed.is_initialized():
            torch.distributed.init_process_group("nccl" if devices[0].startswith("cuda") else "gloo")
        if devices == ["cuda"]:
            devices = [f"cuda:{os.environ['LOCAL_RANK']}"]
            torch.cuda.set_device(devices[0])

    torch.manual_seed(0)
    cfg = LlamaConfig.llama2_7b() if args.size == "7b" else LlamaConfig(vocab_size=1000, hidden_size=64, intermediate_size=176,
                                                                        num_hidden_layers=2, num_attention_heads=4)
    build_on = devices[0] if devices[0].startswith("cuda") else "cpu"
    with torch.device(build_on):
        model = LlamaForCausalLM(cfg).to(getattr(torch, args.dtype)).eval()
    model = tp.tensor_parallel(model, devices)
    prompt = torch.randint(0, cfg.vocab_size, (2, 12))
    greedy = model.generate(prompt, max_new_tokens=args.new_tokens)
    print("greedy :", greedy[0, 12:].tolist())
    if build_on == "cpu":  # (beam search and sampling use the generic path; fine on any device, shown here on CPU)
        beams = model.generate(prompt, max_new_tokens=args.new_tokens, num_beams=3)
        sample = model.generate(prompt, max_new_tokens=args.new_tokens, do_sample=True, top_p=0.9, generator=torch.Generator().manual_seed(0))
        print("beam   :", beams[0, 12:].tolist())
        print("top-p  :", sample[0, 12:].tolist())
    return greedy


if __name__ == "__main__":
    main()
