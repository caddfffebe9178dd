"""Fine-tune a tensor-parallel model and save it "as if it was never split".

    python examples/train_and_save.py                       # two CPU ranks in one process, tiny Llama
    python examples/train_and_save.py --devices cuda:0 cuda:1 --dtype bfloat16 --hidden 1024 --layers 8

The same script works under ``torchrun`` (one process per GPU): pass this process's device only, e.g.
``--devices cuda:$LOCAL_RANK``; ``tp.tensor_parallel`` sees the initialised process group and returns the
one-process-per-rank runtime.
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
    ap.add_argument("--hidden", type=int, default=64)
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    if "LOCAL_RANK" in os.environ and not torch.distributed.is_initialized():
        torch.distributed.init_process_group("nccl" if args.devices[0].startswith("cuda") else "gloo")

    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=1000, hidden_size=args.hidden, intermediate_size=args.hidden * 8 // 3 // 16 * 16,
                      num_hidden_layers=args.layers, num_attention_heads=max(4, args.hidden // 64))
    model = LlamaForCausalLM(cfg).to(getattr(torch, args.dtype))
    # sharded=True: every parameter that tensor parallelism leaves whole (norm weights ...) is ZeRO-3 sharded, so no
    # rank holds a duplicate and the gradients of those parameters are summed over the ranks
    model = tp.tensor_parallel(model, args.devices, sharded=True)
    optimizer = tp.optim.AdamW(model.parameters(), lr=1e-3, weight_decay=0.01)

    data = torch.randint(0, 1000, (4, 32))
    for step in range(args.steps):
        loss = model(input_ids=data, labels=data).loss
        loss.backward()
        optimizer.step()
        optimizer.zero_grad(set_to_none=True)
        print(f"step {step}: loss {loss.item():.4f}")

    with tp.save_tensor_parallel(model):  # the state dict of the original, unsplit module
        state = model.state_dict()
    print(f"{len(state)} tensors in the un-sharded state dict, e.g. {next(iter(state))}")
    if args.out:
        torch.save(state, args.out)
    restored = LlamaForCausalLM(cfg).to(getattr(torch, args.dtype))
    restored.load_state_dict(state)  # loads into the plain model, on any number of devices
    return loss.item()


if __name__ == "__main__":
    main()
