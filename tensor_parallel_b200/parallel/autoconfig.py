"""Generic rule table for arbitrary modules: split every linear, embedding and convolution
layer on its own and gather (or sum) its output.  Less efficient than a hand-written table
(one collective per layer) but works for any ``nn.Module``.
Reference: ``src/tensor_parallel/autoconfig.py:12-75``.
"""
from __future__ import annotations

import re
from typing import Sequence

from torch import nn
from torch.nn.modules.conv import _ConvNd

from tensor_parallel_b200.parallel.actions import Scale, Split, SplitInGroupedChunks
from tensor_parallel_b200.parallel.rules import Config


def get_default_config(module: nn.Module, device_ids: Sequence) -> Config:
    world = len(device_ids)
    embedding_weights = {id(m.weight) for m in module.modules() if isinstance(m, (nn.Embedding, nn.EmbeddingBag))}
    state, inputs, outputs = {}, {}, {}

    for name, sub in module.named_modules():
        exact = f"^{re.escape(name)}$"
        tensor = lambda leaf: f"^{re.escape(name)}\\.{leaf}$"  # noqa: E731
        if isinstance(sub, (nn.Embedding, nn.EmbeddingBag)):
            if sub.max_norm is not None and sub.norm_type >= 2:
                raise ValueError(f"{name}: max_norm renormalisation needs whole embedding rows")
            # hidden-dim split: every rank looks up all ids and owns a column slice of the table
            state[tensor("weight")] = Split(world, dim=1)
            outputs[exact] = {0: "gather -1"}
        elif isinstance(sub, nn.Linear) and "lora_A" not in name and "lora_B" not in name:
            if id(sub.weight) in embedding_weights:
                # weight tied to an embedding table that is split along the hidden dim, i.e. along
                # this layer's input features: feed it the matching input slice and sum the outputs
                inputs[exact] = {0: Split(world, dim=-1)}
                outputs[exact] = {0: "sum"}
                if sub.bias is not None:
                    state[tensor("bias")] = Scale(world)
            else:
                state[f"^{re.escape(name)}\\.(weight|bias)$"] = Split(world, dim=0)
                outputs[exact] = {0: "gather -1"}
        elif isinstance(sub, _ConvNd):
            if sub.groups == 1:
                # output-channel split; transposed convs store weights as [in, out, ...]
                state[tensor("weight")] = Split(world, dim=1 if sub.transposed else 0)
                if sub.bias is not None:
                    state[tensor("bias")] = Split(world, dim=0)
                outputs[exact] = {0: "gather 1"}
            else:
                # grouped conv: keep ``groups`` intact and split the input channels inside each group
                if sub.transposed:
                    state[tensor("weight")] = SplitInGroupedChunks(world, dim=0, num_groups=sub.groups, chunk_size=1)
                else:
                    state[tensor("weight")] = Split(world, dim=1)
                if sub.bias is not None:
                    state[tensor("bias")] = Scale(world)
                inputs[exact] = {0: SplitInGroupedChunks(world, dim=1, num_groups=sub.groups, chunk_size=1)}
                outputs[exact] = {0: "sum"}
    return Config(state, inputs, outputs, {})
