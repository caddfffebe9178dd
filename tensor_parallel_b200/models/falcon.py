"""Falcon-shaped decoder ("RefinedWeb", new decoder architecture): parallel attention + MLP
block reading the same input through two LayerNorms, fused ``query_key_value`` laid out per KV
group as ``[q_per_kv query heads | k | v]``, rotary positions, GeLU MLP, no biases, lm_head tied
to ``word_embeddings``.  Names / attributes (``num_kv``, ``num_heads``) follow the remote-code
``RWForCausalLM`` targeted by ``src/tensor_parallel/slicing_configs.py:409-462``.
"""
from __future__ import annotations

import torch
from torch import nn

from tensor_parallel_b200.models.common import CausalLMBase, LayerNorm, Linear, ModelOutput, ShapedConfig, init_weights_, past_length, update_kv
from tensor_parallel_b200.ops import functional as OF


class FalconConfig(ShapedConfig):
    model_type = "RefinedWeb"

    def __init__(self, vocab_size=65024, hidden_size=8192, n_layer=60, n_head=128, n_head_kv=8, layer_norm_epsilon=1e-5,
                 rope_theta=10000.0, ffn_mult=4, bias=False, alibi=False, **kw):
        super().__init__(vocab_size=vocab_size, hidden_size=hidden_size, n_layer=n_layer, n_head=n_head, n_head_kv=n_head_kv,
                         layer_norm_epsilon=layer_norm_epsilon, rope_theta=rope_theta, ffn_mult=ffn_mult, bias=bias, alibi=alibi,
                         num_attention_heads=n_head, num_hidden_layers=n_layer, **kw)

    @classmethod
    def falcon_40b(cls):
        return cls()


class FalconAttention(nn.Module):
    def __init__(self, config: FalconConfig):
        super().__init__()
        self.hidden_size = config.hidden_size
        self.num_heads = config.n_head
        self.num_kv = config.n_head_kv
        self.head_dim = config.hidden_size // config.n_head
        self.rope_theta = config.rope_theta
        self.query_key_value = Linear(config.hidden_size, (self.num_heads + 2 * self.num_kv) * self.head_dim, bias=False)
        self.dense = Linear(config.hidden_size, config.hidden_size, bias=False)

    def forward(self, hidden_states, layer_past=None, attention_mask=None, position_ids=None, use_cache=False):
        b, s, _ = hidden_states.shape
        q_per_kv = self.num_heads // self.num_kv
        fused = self.query_key_value(hidden_states).view(b, s, self.num_kv, q_per_kv + 2, self.head_dim)
        q = fused[:, :, :, :q_per_kv].reshape(b, s, self.num_heads, self.head_dim)
        k, v = fused[:, :, :, q_per_kv], fused[:, :, :, q_per_kv + 1]
        q = OF.apply_rope(q, position_ids, self.rope_theta)
        k = OF.apply_rope(k, position_ids, self.rope_theta)
        k_all, v_all, present = update_kv(layer_past, k, v)
        out = OF.attention(q, k_all, v_all, causal=True, bias=attention_mask)
        return self.dense(out.reshape(b, s, -1)), (present if use_cache else None)


class FalconMLP(nn.Module):
    def __init__(self, config: FalconConfig):
        super().__init__()
        self.dense_h_to_4h = Linear(config.hidden_size, config.ffn_mult * config.hidden_size, bias=False)
        self.dense_4h_to_h = Linear(config.ffn_mult * config.hidden_size, config.hidden_size, bias=False)

    def forward(self, x):
        return self.dense_4h_to_h(OF.gelu(self.dense_h_to_4h(x)))


class FalconDecoderLayer(nn.Module):
    parallel_block = True  # attention and MLP read the same input; their partial outputs may share one all-reduce

    def __init__(self, config: FalconConfig):
        super().__init__()
        self.ln_attn = LayerNorm(config.hidden_size, eps=config.layer_norm_epsilon)
        self.ln_mlp = LayerNorm(config.hidden_size, eps=config.layer_norm_epsilon)
        self.self_attention = FalconAttention(config)
        self.mlp = FalconMLP(config)

    def forward(self, hidden, layer_past=None, attention_mask=None, position_ids=None, use_cache=False):
        attn_out, present = self.self_attention(self.ln_attn(hidden), layer_past=layer_past, attention_mask=attention_mask,
                                                position_ids=position_ids, use_cache=use_cache)
        partial = attn_out + self.mlp(self.ln_mlp(hidden))
        reduce = self.__dict__.get("_tp_block_reduce")
        return hidden + (partial if reduce is None else reduce(partial)), present


class FalconModel(nn.Module):
    def __init__(self, config: FalconConfig):
        super().__init__()
        self.config = config  # lets the predefined rule table be found when the bare model (no head) is wrapped
        self.word_embeddings = nn.Embedding(config.vocab_size, config.hidden_size)
        self.h = nn.ModuleList([FalconDecoderLayer(config) for _ in range(config.n_layer)])
        self.ln_f = LayerNorm(config.hidden_size, eps=config.layer_norm_epsilon)

    def forward(self, input_ids=None, past_key_values=None, attention_mask=None, position_ids=None, inputs_embeds=None, use_cache=False):
        hidden = self.word_embeddings(input_ids) if inputs_embeds is None else inputs_embeds
        b, s = hidden.shape[:2]
        offset = past_length(past_key_values)
        if position_ids is None:
            position_ids = torch.arange(offset, offset + s, device=hidden.device)[None].expand(b, s)
        presents = []
        for i, layer in enumerate(self.h):
            hidden, present = layer(hidden, None if past_key_values is None else past_key_values[i], attention_mask, position_ids, use_cache)
            presents.append(present)
        return self.ln_f(hidden), (tuple(presents) if use_cache else None)


class FalconForCausalLM(CausalLMBase):
    def __init__(self, config: FalconConfig):
        super().__init__()
        self.config = config
        self.transformer = FalconModel(config)
        self.lm_head = Linear(config.hidden_size, config.vocab_size, bias=False)
        init_weights_(self)
        self.lm_head.weight = self.transformer.word_embeddings.weight  # tied

    def forward(self, input_ids=None, past_key_values=None, attention_mask=None, position_ids=None, inputs_embeds=None,
                labels=None, use_cache=False, **unused):
        hidden, presents = self.transformer(input_ids, past_key_values, attention_mask, position_ids, inputs_embeds, use_cache)
        logits = self.lm_head(hidden)
        return ModelOutput(loss=self.lm_loss(logits, labels), logits=logits, past_key_values=presents)
