"""Rule tables for T5 (encoder-decoder) and BERT (encoder-only).

T5: the reference leaves cross-attention (``EncDecAttention``) replicated because its patterns
only name ``SelfAttention`` (``src/tensor_parallel/slicing_configs.py:101-105``).  Here
cross-attention is head-parallel too by default; ``split_cross_attention=False`` restores the
reference's table bit for bit (its sharded checkpoints then load unchanged).
"""
from __future__ import annotations

from functools import partial
from typing import Sequence

import torch

from tensor_parallel_b200.parallel.actions import Scale, Split, SplitInChunks
from tensor_parallel_b200.parallel.aux import split_inner_dim, split_num_heads
from tensor_parallel_b200.parallel.kv import PerDeviceTensors
from tensor_parallel_b200.parallel.rules import Config


def get_t5_config(model_config, devices: Sequence[torch.device], split_cross_attention: bool = True) -> Config:
    world = len(devices)
    heads, head_dim = model_config.num_heads, model_config.d_kv
    attn = r"(SelfAttention|EncDecAttention)" if split_cross_attention else r"SelfAttention"

    def local_kv(kv, rank):
        """Cached ``(k, v)``: per-device carriers pick their element; plain full-head tensors
        (e.g. a cache produced by an unsplit model) are cut along the head dim."""
        if kv is None:
            return None
        k, v = kv[0], kv[1]
        if isinstance(k, PerDeviceTensors):
            return (k[rank], v[rank]) + tuple(kv[2:])
        cut = lambda t: torch.tensor_split(t, world, dim=1)[rank]  # noqa: E731
        return (cut(k), cut(v)) + tuple(kv[2:])

    return Config(
        state_rules={
            rf".*{attn}\.(q|k|v)\.(weight|bias)$": SplitInChunks(world, dim=0, chunk_size=head_dim),
            r".*relative_attention_bias\.weight$": Split(world, dim=1),
            rf".*{attn}\.o\.weight$": SplitInChunks(world, dim=1, chunk_size=head_dim),
            r".*DenseReluDense\.(wi|wi_0|wi_1)\.weight$": Split(world, dim=0),
            r".*DenseReluDense\.wo\.weight$": Split(world, dim=1),
            r".*embed_tokens\.weight$": Split(world, dim=1),
            r".*shared\.weight$": Split(world, dim=1),
            r".*lm_head\.weight$": Split(world, dim=1),  # tied to shared
        },
        input_rules={
            rf".*{attn}$": {"past_key_value": local_kv},
            r".*lm_head$": {0: "split -1"},
        },
        output_rules={
            rf".*{attn}$": {0: "sum", 1: "gather_kv"},
            r".*DenseReluDense$": {0: "sum"},
            r".*shared$": {0: "gather -1"},
            r".*embed_tokens$": {0: "gather -1"},
            r".*lm_head$": {0: "sum"},
        },
        attr_rules={
            rf".*{attn}$": {
                "n_heads": partial(split_num_heads, world_size=world),
                "inner_dim": partial(split_inner_dim, num_heads=heads, world_size=world),
            },
            r".*relative_attention_bias$": {"embedding_dim": partial(split_num_heads, world_size=world)},
        },
    )


def get_bert_config(model_config, devices: Sequence[torch.device]) -> Config:
    world = len(devices)
    heads = model_config.num_attention_heads
    head_dim = model_config.hidden_size // heads
    return Config(
        state_rules={
            r".*self\.(query|key|value)\.(weight|bias)$": SplitInChunks(world, dim=0, chunk_size=head_dim),
            r".*attention\.output\.dense\.weight$": SplitInChunks(world, dim=1, chunk_size=head_dim),
            r".*attention\.output\.dense\.bias$": Scale(world),
            r".*intermediate\.dense\.(weight|bias)$": Split(world, dim=0),
            r".*[0-9]\.output\.dense\.weight$": Split(world, dim=1),
            r".*[0-9]\.output\.dense\.bias$": Scale(world),
            r".*word_embeddings\.weight$": Split(world, dim=1),
            r".*position_embeddings\.weight$": Split(world, dim=1),
            r".*token_type_embeddings\.weight$": Split(world, dim=1),
        },
        input_rules={},
        output_rules={
            r".*attention\.output\.dense$": {0: "sum"},
            r".*[0-9]\.output\.dense$": {0: "sum"},
            r".*word_embeddings$": {0: "gather -1"},
            r".*position_embeddings$": {0: "gather -1"},
            r".*token_type_embeddings$": {0: "gather -1"},
        },
        attr_rules={
            r".*attention\.self$": {
                "num_attention_heads": partial(split_num_heads, world_size=world),
                "all_head_size": partial(split_inner_dim, num_heads=heads, world_size=world),
            }
        },
    )
