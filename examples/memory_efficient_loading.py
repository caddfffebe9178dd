"""Load a checkpoint into a tensor-parallel model chunk by chunk, never holding more than one chunk of the original
weights in memory: build the model on the ``meta`` device, wrap it, convert each chunk of the plain state dict to the
sharded key layout and place the pieces directly on their ranks.

    python examples/memory_efficient_loading.py
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import tensor_parallel_b200 as tp  # noqa: E402
from tensor_parallel_b200.models.gpt2 import GPT2Config, GPT2LMHeadModel  # noqa: E402


def main(devices=("cpu", "cpu")):
    torch.manual_seed(0)
    cfg = GPT2Config(vocab_size=500, n_positions=64, n_embd=64, n_layer=2, n_head=4)
    original = GPT2LMHeadModel(cfg)                      # stands for a checkpoint on disk ...
    full = original.state_dict()
    keys = list(full)
    chunks = [{k: full[k] for k in keys[i::3]} for i in range(3)]  # ... stored in three files

    with torch.device("meta"):
        skeleton = GPT2LMHeadModel(cfg)                  # no weight memory
    model = tp.tensor_parallel(skeleton, list(devices), sharded=False)
    for chunk in chunks:
        converted = tp.convert_state_dict(chunk, model.tensor_parallel_config, world_size=len(devices))
        tp.load_sharded_state_dict_(model, converted, strict=False)
    model.apply_sharding()                               # ZeRO-3 for what stayed replicated, now that the weights are real

    ids = torch.randint(0, 500, (2, 9))
    with torch.no_grad():
        diff = (model(input_ids=ids).logits - original(input_ids=ids).logits).abs().max().item()
    print(f"max |logits difference| to the original model: {diff:.2e}")
    print("device of every tensor:", sorted({str(d) for d in tp.infer_sharded_device_map(model).values()}))
    return diff


if __name__ == "__main__":
    main()
