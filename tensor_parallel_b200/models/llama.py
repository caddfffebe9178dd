"""Llama-shaped decoder (RMSNorm, rotary positions, SwiGLU MLP, optional GQA).

Module tree and attribute names follow ``transformers`` ``LlamaForCausalLM`` as targeted by the
reference's Llama table (``src/tensor_parallel/slicing_configs.py:345-406``): ``self_attn`` exposes
``hidden_size`` / ``num_heads`` / ``num_key_value_heads`` and returns ``(out, weights, present_kv)``.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from tensor_parallel_b200.models.common import CausalLMBase, Linear, ModelOutput, RMSNorm, ShapedConfig, init_weights_, past_length, update_kv
from tensor_parallel_b200.ops import functional as OF


class LlamaConfig(ShapedConfig):
    model_type = "llama"

    def __init__(self, vocab_size=32000, hidden_size=4096, intermediate_size=11008, num_hidden_layers=32,
                 num_attention_heads=32, num_key_value_heads=None, rms_norm_eps=1e-6, rope_theta=10000.0,
                 max_position_embeddings=4096, **kw):
        super().__init__(vocab_size=vocab_size, hidden_size=hidden_size, intermediate_size=intermediate_size,
                         num_hidden_layers=num_hidden_layers, num_attention_heads=num_attention_heads,
                         num_key_value_heads=num_key_value_heads or num_attention_heads, rms_norm_eps=rms_norm_eps,
                         rope_theta=rope_theta, max_position_embeddings=max_position_embeddings, **kw)

    @classmethod
    def llama2_7b(cls):
        return cls()


class LlamaAttention(nn.Module):
    def __init__(self, config: LlamaConfig):
        super().__init__()
        self.hidden_size = config.hidden_size
        self.num_heads = config.num_attention_heads
        self.num_key_value_heads = config.num_key_value_heads
        self.head_dim = config.hidden_size // config.num_attention_heads
        self.rope_theta = config.rope_theta
        self.q_proj = Linear(config.hidden_size, self.num_heads * self.head_dim, bias=False)
        self.k_proj = Linear(config.hidden_size, self.num_key_value_heads * self.head_dim, bias=False)
        self.v_proj = Linear(config.hidden_size, self.num_key_value_heads * self.head_dim, bias=False)
        self.o_proj = Linear(self.num_heads * self.head_dim, config.hidden_size, bias=False)

    def forward(self, hidden_states, attention_mask=None, position_ids=None, past_key_value=None,
                output_attentions=False, use_cache=False):
        b, s, _ = hidden_states.shape
        q = self.q_proj(hidden_states).view(b, s, -1, self.head_dim)
        k = self.k_proj(hidden_states).view(b, s, -1, self.head_dim)
        v = self.v_proj(hidden_states).view(b, s, -1, self.head_dim)
        q = OF.apply_rope(q, position_ids, self.rope_theta)
        k = OF.apply_rope(k, position_ids, self.rope_theta)
        k_all, v_all, present = update_kv(past_key_value, k, v)
        out = OF.attention(q, k_all, v_all, causal=True, bias=attention_mask)
        out = self.o_proj(out.reshape(b, s, -1))
        return out, None, (present if use_cache else None)


class LlamaMLP(nn.Module):
    def __init__(self, config: LlamaConfig):
        super().__init__()
        self.gate_proj = Linear(config.hidden_size, config.intermediate_size, bias=False)
        self.up_proj = Linear(config.hidden_size, config.intermediate_size, bias=False)
        self.down_proj = Linear(config.intermediate_size, config.hidden_size, bias=False)

    def forward(self, x):
        return self.down_proj(OF.swiglu(self.gate_proj(x), self.up_proj(x)))


class LlamaDecoderLayer(nn.Module):
    def __init__(self, config: LlamaConfig):
        super().__init__()
        self.self_attn = LlamaAttention(config)
        self.mlp = LlamaMLP(config)
        self.input_layernorm = RMSNorm(config.hidden_size, config.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, config.rms_norm_eps)

    def forward(self, hidden_states, attention_mask=None, position_ids=None, past_key_value=None, use_cache=False):
        attn_out, _, present = self.self_attn(
            self.input_layernorm(hidden_states), attention_mask=attention_mask, position_ids=position_ids,
            past_key_value=past_key_value, use_cache=use_cache,
        )
        hidden_states = hidden_states + attn_out
        hidden_states = hidden_states + self.mlp(self.post_attention_layernorm(hidden_states))
        return hidden_states, present


class LlamaModel(nn.Module):
    def __init__(self, config: LlamaConfig):
        super().__init__()
        self.config = config  # lets the predefined rule table be found when the bare model (no head) is wrapped
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList([LlamaDecoderLayer(config) for _ in range(config.num_hidden_layers)])
        self.norm = RMSNorm(config.hidden_size, config.rms_norm_eps)

    def forward(self, input_ids=None, attention_mask=None, position_ids=None, past_key_values=None,
                inputs_embeds=None, use_cache=False):
        hidden = self.embed_tokens(input_ids) if inputs_embeds is None else inputs_embeds
        b, s = hidden.shape[:2]
        offset = past_length(past_key_values)
        if position_ids is None:
            position_ids = torch.arange(offset, offset + s, device=hidden.device)[None].expand(b, s)
        presents = []
        for i, layer in enumerate(self.layers):
            hidden, present = layer(hidden, attention_mask, position_ids,
                                    None if past_key_values is None else past_key_values[i], use_cache)
            presents.append(present)
        return self.norm(hidden), (tuple(presents) if use_cache else None)


class LlamaForCausalLM(CausalLMBase):
    def __init__(self, config: LlamaConfig):
        super().__init__()
        self.config = config
        self.model = LlamaModel(config)
        self.lm_head = Linear(config.hidden_size, config.vocab_size, bias=False)
        init_weights_(self)

    def forward(self, input_ids=None, attention_mask=None, position_ids=None, past_key_values=None,
                inputs_embeds=None, labels=None, use_cache=False, **unused):
        hidden, presents = self.model(input_ids, attention_mask, position_ids, past_key_values, inputs_embeds, use_cache)
        logits, loss = self.head_and_loss(self.lm_head, hidden, labels)
        return ModelOutput(loss=loss, logits=logits, past_key_values=presents)
