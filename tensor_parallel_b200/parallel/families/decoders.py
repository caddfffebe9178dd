"""Rule tables for decoder-only families.  Module / attribute names are the Hugging Face ones
of the era the reference targets (e.g. ``self_attn.num_heads``); attribute rules for names a
model does not have are skipped by the table builder, so the same table serves both the
self-contained models in ``tensor_parallel_b200.models`` and HF classes that kept the names.
"""
from __future__ import annotations

from functools import partial
from typing import Sequence

import torch

from tensor_parallel_b200.parallel.actions import Scale, Split, SplitInChunks, SplitInGroupedChunks, unit_bounds
from tensor_parallel_b200.parallel.aux import select_kv_for_rank, split_alibi, split_inner_dim, split_num_heads
from tensor_parallel_b200.parallel.rules import Config


def _cfg(model_config, *names, default=None):
    for name in names:
        if hasattr(model_config, name) and getattr(model_config, name) is not None:
            return getattr(model_config, name)
    if default is None:
        raise AttributeError(f"model config has none of {names}")
    return default


def _grouped_heads(q_per_kv: int, world: int):
    """num_heads -> local num_heads when heads are dealt out in whole KV groups."""
    return lambda n, rank: q_per_kv * split_num_heads(n // q_per_kv, rank=rank, world_size=world)


def get_llama_config(model_config, devices: Sequence[torch.device]) -> Config:
    world = len(devices)
    heads = model_config.num_attention_heads
    head_dim = getattr(model_config, "head_dim", None) or model_config.hidden_size // heads
    num_kv = getattr(model_config, "num_key_value_heads", None) or heads
    q_per_kv = heads // num_kv
    attrs = {
        "hidden_size": partial(split_inner_dim, num_heads=num_kv, world_size=world),
        "num_heads": _grouped_heads(q_per_kv, world),
        "num_key_value_heads": partial(split_num_heads, world_size=world),
    }
    # a head tied to the (hidden-split) embedding table keeps that split and becomes row-parallel: it reads its slice of
    # the hidden state and the partial logits are summed (small Llama-3.2 / Qwen2 checkpoints tie the two)
    tied = bool(getattr(model_config, "tie_word_embeddings", False))
    return Config(
        state_rules={
            r".*self_attn\.q_proj\.(weight|bias)$": SplitInChunks(world, dim=0, chunk_size=q_per_kv * head_dim),
            r".*self_attn\.k_proj\.(weight|bias)$": SplitInChunks(world, dim=0, chunk_size=head_dim),
            r".*self_attn\.v_proj\.(weight|bias)$": SplitInChunks(world, dim=0, chunk_size=head_dim),
            r".*self_attn\.o_proj\.weight$": SplitInChunks(world, dim=1, chunk_size=q_per_kv * head_dim),
            r".*self_attn\.o_proj\.bias$": Scale(world),
            r".*mlp\.gate_proj\.weight$": Split(world, dim=0),
            r".*mlp\.up_proj\.weight$": Split(world, dim=0),
            r".*mlp\.down_proj\.weight$": Split(world, dim=1),
            r".*embed_tokens\.weight$": Split(world, dim=1),
            r".*lm_head\.weight$": Split(world, dim=1 if tied else 0),
        },
        input_rules={r".*self_attn$": {"past_key_value": select_kv_for_rank}, **({r".*lm_head$": {0: "split -1"}} if tied else {})},
        output_rules={
            r".*self_attn$": {0: "sum", 2: "gather_kv"},
            r".*mlp$": {0: "sum"},
            r".*embed_tokens$": {0: "gather -1"},
            r".*lm_head$": {0: "sum" if tied else "gather -1"},
        },
        attr_rules={r".*self_attn$": attrs},
    )


def get_opt_config(model_config, devices: Sequence[torch.device]) -> Config:
    """OPT: separate q/k/v/out projections with biases, ReLU MLP ``fc1``/``fc2`` directly on the
    layer, learned positions, lm_head tied to ``embed_tokens``.  Two all-reduces per layer
    instead of the six all-gathers the automatic config needs."""
    world = len(devices)
    heads = model_config.num_attention_heads
    head_dim = model_config.hidden_size // heads
    return Config(
        state_rules={
            r".*self_attn\.(q_proj|k_proj|v_proj)\.(weight|bias)$": SplitInChunks(world, dim=0, chunk_size=head_dim),
            r".*self_attn\.out_proj\.weight$": SplitInChunks(world, dim=1, chunk_size=head_dim),
            r".*self_attn\.out_proj\.bias$": Scale(world),
            r".*\.fc1\.(weight|bias)$": Split(world, dim=0),
            r".*\.fc2\.weight$": Split(world, dim=1),
            r".*\.fc2\.bias$": Scale(world),
            r".*embed_tokens\.weight$": Split(world, dim=1),
            r".*embed_positions\.weight$": Split(world, dim=1),
            r".*lm_head\.weight$": Split(world, dim=1),  # tied to embed_tokens
        },
        input_rules={
            r".*self_attn$": {"past_key_value": select_kv_for_rank},
            r".*lm_head$": {0: "split -1"},
        },
        output_rules={
            r".*self_attn$": {0: "sum", 2: "gather_kv"},
            r".*\.fc2$": {0: "sum"},
            r".*embed_tokens$": {0: "gather -1"},
            r".*embed_positions$": {0: "gather -1"},
            r".*lm_head$": {0: "sum"},
        },
        attr_rules={
            r".*self_attn$": {
                "num_heads": partial(split_num_heads, world_size=world),
                "embed_dim": partial(split_inner_dim, num_heads=heads, world_size=world),
            }
        },
    )


def get_gpt2_config(model_config, devices: Sequence[torch.device]) -> Config:
    """GPT-2 stores linears as ``Conv1D`` (weight ``[in, out]``), so split dims are transposed."""
    world = len(devices)
    heads = _cfg(model_config, "num_attention_heads", "n_head")
    hidden = _cfg(model_config, "hidden_size", "n_embd")
    head_dim = hidden // heads
    inner = partial(split_inner_dim, num_heads=heads, world_size=world)

    def split_width(total: int, rank: int) -> int:
        lo, hi = unit_bounds(total, world, rank)
        return hi - lo

    def qkv_width(total: int, rank: int) -> int:  # nf of the fused c_attn = 3 * local hidden
        return 3 * inner(total // 3, rank=rank)

    return Config(
        state_rules={
            r".*c_attn\.weight$": SplitInGroupedChunks(world, dim=1, num_groups=3, chunk_size=head_dim),
            r".*c_attn\.bias$": SplitInGroupedChunks(world, dim=0, num_groups=3, chunk_size=head_dim),
            r".*q_attn\.weight$": SplitInChunks(world, dim=1, chunk_size=head_dim),
            r".*q_attn\.bias$": SplitInChunks(world, dim=0, chunk_size=head_dim),
            r".*attn\.c_proj\.weight$": SplitInChunks(world, dim=0, chunk_size=head_dim),
            r".*attn\.c_proj\.bias$": Scale(world),
            r".*c_fc\.weight$": Split(world, dim=1),
            r".*c_fc\.bias$": Split(world, dim=0),
            r".*mlp\.c_proj\.weight$": Split(world, dim=0),
            r".*mlp\.c_proj\.bias$": Scale(world),
            r".*wte\.weight$": Split(world, dim=1),
            r".*wpe\.weight$": Split(world, dim=1),
            r".*lm_head\.weight$": Split(world, dim=1),  # tied to wte
        },
        input_rules={
            r".*[0-9]\.attn$": {"layer_past": select_kv_for_rank},
            r".*lm_head$": {0: "split -1"},
        },
        output_rules={
            r".*[0-9]\.attn$": {0: "sum", 1: "gather_kv"},
            r".*mlp$": {0: "sum"},
            r".*wte$": {0: "gather -1"},
            r".*wpe$": {0: "gather -1"},
            r".*lm_head$": {0: "sum"},
        },
        attr_rules={
            r".*attn\.c_attn$": {"nf": qkv_width},
            r".*attn\.q_attn$": {"nf": lambda total, rank: inner(total, rank=rank)},
            r".*mlp\.c_fc$": {"nf": split_width},
            r".*[0-9]\.attn$": {
                "embed_dim": lambda total, rank: inner(total, rank=rank),
                "num_heads": partial(split_num_heads, world_size=world),
                "split_size": lambda total, rank: inner(total, rank=rank),
            },
        },
    )


def get_gptj_config(model_config, devices: Sequence[torch.device]) -> Config:
    """GPT-J: parallel attention + MLP block, untied lm_head with bias, rotary positions."""
    world = len(devices)
    heads = _cfg(model_config, "num_attention_heads", "n_head")
    hidden = _cfg(model_config, "hidden_size", "n_embd")
    head_dim = hidden // heads
    return Config(
        state_rules={
            r".*attn\.(q_proj|k_proj|v_proj)\.weight$": SplitInChunks(world, dim=0, chunk_size=head_dim),
            r".*attn\.out_proj\.weight$": SplitInChunks(world, dim=1, chunk_size=head_dim),
            r".*mlp\.fc_in\.(weight|bias)$": Split(world, dim=0),
            r".*mlp\.fc_out\.weight$": Split(world, dim=1),
            r".*mlp\.fc_out\.bias$": Scale(world),
            r".*wte\.weight$": Split(world, dim=1),
            r".*lm_head\.(weight|bias)$": Split(world, dim=0),
        },
        input_rules={r".*[0-9]\.attn$": {"layer_past": select_kv_for_rank}},
        output_rules={
            r".*[0-9]\.attn$": {0: "sum", 1: "gather_kv"},
            r".*mlp$": {0: "sum"},
            r".*wte$": {0: "gather -1"},
            r".*lm_head$": {0: "gather -1"},
        },
        attr_rules={
            r".*[0-9]\.attn$": {
                "embed_dim": partial(split_inner_dim, num_heads=heads, world_size=world),
                "num_attention_heads": partial(split_num_heads, world_size=world),
            }
        },
    )


def get_gpt_neox_config(model_config, devices: Sequence[torch.device]) -> Config:
    world = len(devices)
    heads = model_config.num_attention_heads
    head_dim = model_config.hidden_size // heads
    return Config(
        state_rules={
            # fused QKV is interleaved per head: [h0:q,k,v | h1:q,k,v | ...]
            r".*attention\.query_key_value\.(weight|bias)$": SplitInChunks(world, dim=0, chunk_size=3 * head_dim),
            r".*attention\.dense\.weight$": SplitInChunks(world, dim=1, chunk_size=head_dim),
            r".*attention\.dense\.bias$": Scale(world),
            r".*mlp\.dense_h_to_4h\.(weight|bias)$": Split(world, dim=0),
            r".*mlp\.dense_4h_to_h\.weight$": Split(world, dim=1),
            r".*mlp\.dense_4h_to_h\.bias$": Scale(world),
            r".*embed_in\.weight$": Split(world, dim=1),
            r".*embed_out\.(weight|bias)$": Split(world, dim=0),
        },
        input_rules={r".*attention$": {"layer_past": select_kv_for_rank}},
        output_rules={
            r".*attention$": {0: "sum", 1: "gather_kv"},
            r".*mlp$": {0: "sum"},
            r".*embed_in$": {0: "gather -1"},
            r".*embed_out$": {0: "gather -1"},
        },
        attr_rules={
            r".*attention$": {
                "num_attention_heads": partial(split_num_heads, world_size=world),
                "hidden_size": partial(split_inner_dim, num_heads=heads, world_size=world),
            }
        },
    )


def get_bloom_config(model_config, devices: Sequence[torch.device]) -> Config:
    world = len(devices)
    heads = _cfg(model_config, "n_head", "num_attention_heads")
    head_dim = model_config.hidden_size // heads
    return Config(
        state_rules={
            r".*self_attention\.query_key_value\.(weight|bias)$": SplitInChunks(world, dim=0, chunk_size=3 * head_dim),
            r".*self_attention\.dense\.weight$": SplitInChunks(world, dim=1, chunk_size=head_dim),
            r".*self_attention\.dense\.bias$": Scale(world),
            r".*mlp\.dense_h_to_4h\.(weight|bias)$": Split(world, dim=0),
            r".*mlp\.dense_4h_to_h\.weight$": Split(world, dim=1),
            r".*mlp\.dense_4h_to_h\.bias$": Scale(world),
            r".*word_embeddings\.weight$": Split(world, dim=1),
            r".*lm_head\.weight$": Split(world, dim=1),  # tied to word_embeddings
        },
        input_rules={
            r".*self_attention$": {
                "layer_past": select_kv_for_rank,
                "alibi": partial(split_alibi, num_heads=heads, world_size=world),
            },
            r".*lm_head$": {0: "split -1"},
        },
        output_rules={
            r".*self_attention$": {1: "gather_kv"},
            r".*self_attention\.dense$": {0: "sum"},
            r".*mlp\.dense_4h_to_h$": {0: "sum"},
            r".*word_embeddings$": {0: "gather -1"},
            r".*lm_head$": {0: "sum"},
        },
        attr_rules={r".*self_attention$": {"num_heads": partial(split_num_heads, world_size=world)}},
    )


class SplitCodegenQKV(SplitInChunks):
    """CodeGen's fused ``qkv_proj`` rows are laid out ``[mp=4][q|v|k][heads/4][head_dim]``; logical
    head ``i`` lives at ``(mp, h) = divmod(i, heads/4)``.  Ranks receive contiguous ranges of logical
    heads in units of 4 (matching the ``out_proj`` column split) and the local rows are written
    back in the same 4-block layout, so the unmodified attention code works on the slice."""

    MP = 4

    def __init__(self, world_size: int, head_dim: int):
        super().__init__(world_size, dim=0, chunk_size=head_dim)

    def _to_heads(self, tensor: torch.Tensor) -> torch.Tensor:
        hd, rest = self.chunk_size, tuple(tensor.shape[1:])
        per_mp = tensor.shape[0] // (self.MP * 3 * hd)
        blocks = tensor.reshape(self.MP, 3, per_mp, hd, *rest)
        return blocks.transpose(1, 2).reshape(self.MP * per_mp, 3, hd, *rest)

    def _from_heads(self, heads: torch.Tensor) -> torch.Tensor:
        hd, rest = self.chunk_size, tuple(heads.shape[3:])
        per_mp = heads.shape[0] // self.MP
        blocks = heads.reshape(self.MP, per_mp, 3, hd, *rest).transpose(1, 2)
        return blocks.reshape(self.MP * 3 * per_mp * hd, *rest)

    def __call__(self, tensor: torch.Tensor, rank: int) -> torch.Tensor:
        heads = self._to_heads(tensor)
        lo, hi = unit_bounds(heads.shape[0] // self.MP, self.world_size, rank)
        return self._from_heads(heads[self.MP * lo : self.MP * hi])

    def undo(self, tensors) -> torch.Tensor:
        return self._from_heads(torch.cat([self._to_heads(t.detach().cpu()) for t in tensors], dim=0))


def get_codegen_config(model_config, devices: Sequence[torch.device]) -> Config:
    world = len(devices)
    heads = _cfg(model_config, "num_attention_heads", "n_head")
    hidden = _cfg(model_config, "hidden_size", "n_embd")
    head_dim = hidden // heads

    def local_heads(n: int, rank: int) -> int:
        return 4 * split_num_heads(n // 4, rank=rank, world_size=world)

    return Config(
        state_rules={
            r".*attn\.qkv_proj\.weight$": SplitCodegenQKV(world, head_dim),
            r".*attn\.out_proj\.weight$": SplitInChunks(world, dim=1, chunk_size=4 * head_dim),
            r".*mlp\.fc_in\.(weight|bias)$": Split(world, dim=0),
            r".*mlp\.fc_out\.weight$": Split(world, dim=1),
            r".*mlp\.fc_out\.bias$": Scale(world),
            r".*wte\.weight$": Split(world, dim=1),
            r".*lm_head\.(weight|bias)$": Split(world, dim=0),
        },
        input_rules={r".*[0-9]\.attn$": {"layer_past": select_kv_for_rank}},
        output_rules={
            r".*[0-9]\.attn$": {0: "sum", 1: "gather_kv"},
            r".*mlp$": {0: "sum"},
            r".*wte$": {0: "gather -1"},
            r".*lm_head$": {0: "gather -1"},
        },
        attr_rules={
            r".*[0-9]\.attn$": {
                "embed_dim": lambda total, rank: local_heads(heads, rank) * head_dim,
                "num_attention_heads": local_heads,
            }
        },
    )


class SplitMultiQueryQKV(Split):
    """Fused ``query_key_value`` of a multi-query Falcon (falcon-7b layout): ``heads`` query heads followed by ONE shared
    key head and ONE shared value head.  The query heads are dealt out in whole heads; the shared key / value rows are
    kept on every rank.  (For training note that those shared rows then behave like any replicated parameter: each rank
    sees the gradient that flows through its own query heads only.)  The reference has no table for this layout."""

    def __init__(self, world_size: int, head_dim: int):
        super().__init__(world_size, dim=0)
        self.head_dim = head_dim

    def __call__(self, tensor, rank: int):
        q_rows = tensor.shape[0] - 2 * self.head_dim
        start, stop = unit_bounds(q_rows // self.head_dim, self.world_size, rank)
        return torch.cat([tensor[start * self.head_dim : stop * self.head_dim], tensor[q_rows:]], dim=0)

    def undo(self, tensors):
        shared = 2 * self.head_dim
        pieces = [t.detach().cpu() for t in tensors]
        return torch.cat([t[: t.shape[0] - shared] for t in pieces] + [pieces[0][-shared:]], dim=0)

    def __repr__(self):
        return f"SplitMultiQueryQKV(world_size={self.world_size}, head_dim={self.head_dim})"


def get_falcon_config(model_config, devices: Sequence[torch.device]) -> Config:
    """Falcon / RefinedWeb (new-decoder layout): fused QKV rows are ``[kv group][q_per_kv q heads | k | v]``.
    The block computes attention and MLP in parallel from the same input, so both partial
    outputs could share one all-reduce; the table keeps the reference's two ``"sum"`` sites
    (``src/tensor_parallel/slicing_configs.py:450-451``) and the fusion planner merges them."""
    world = len(devices)
    if getattr(model_config, "bias", False) or getattr(model_config, "alibi", False):
        raise ValueError("Falcon with biases or ALiBi is not supported by the predefined config")
    heads = _cfg(model_config, "n_head", "num_attention_heads")
    num_kv = _cfg(model_config, "n_head_kv", "num_kv_heads", default=heads if not getattr(model_config, "multi_query", False) else 1)
    head_dim = model_config.hidden_size // heads
    q_per_kv = heads // num_kv
    # multi-query models of the older layout (falcon-7b): all query heads, then one shared key and one shared value head
    new_layout = getattr(model_config, "new_decoder_architecture", hasattr(model_config, "n_head_kv"))
    shared_kv = bool(getattr(model_config, "multi_query", False)) and not new_layout and heads > 1
    if shared_kv:
        num_kv, q_per_kv = 1, heads
    elif num_kv < world:
        raise ValueError(f"Falcon with {num_kv} key/value groups cannot be split over {world} ranks by groups "
                         "(every rank needs at least one group)")
    qkv_action = SplitMultiQueryQKV(world, head_dim) if shared_kv else SplitInChunks(world, dim=0, chunk_size=(q_per_kv + 2) * head_dim)
    dense_chunk = head_dim if shared_kv else q_per_kv * head_dim
    local_heads = partial(split_num_heads, world_size=world) if shared_kv else _grouped_heads(q_per_kv, world)
    return Config(
        state_rules={
            r".*self_attention\.query_key_value\.weight$": qkv_action,
            r".*self_attention\.dense\.weight$": SplitInChunks(world, dim=1, chunk_size=dense_chunk),
            r".*mlp\.dense_h_to_4h\.weight$": Split(world, dim=0),
            r".*mlp\.dense_4h_to_h\.weight$": Split(world, dim=1),
            r".*word_embeddings\.weight$": Split(world, dim=1),
            r".*lm_head\.weight$": Split(world, dim=1),  # tied to word_embeddings
        },
        input_rules={
            r".*self_attention$": {"layer_past": select_kv_for_rank},
            r".*lm_head$": {0: "split -1"},
        },
        output_rules={
            r".*self_attention$": {0: "sum", 1: "gather_kv"},
            r".*\.mlp$": {0: "sum"},
            r".*word_embeddings$": {0: "gather -1"},
            r".*lm_head$": {0: "sum"},
        },
        attr_rules={
            r".*self_attention$": {
                "num_kv": partial(split_num_heads, world_size=world),        # remote-code RWForCausalLM
                "num_kv_heads": partial(split_num_heads, world_size=world),  # transformers' FalconAttention
                "num_heads": local_heads,
            }
        },
    )
