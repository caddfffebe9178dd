"""OPT-shaped decoder: learned positions (offset 2), pre-LayerNorm, ReLU MLP (``fc1`` / ``fc2`` sit
directly on the layer), biases everywhere, lm_head tied to ``embed_tokens``.  Names follow
``transformers`` ``OPTForCausalLM``.  The reference has no OPT table (it falls back to the
automatic config); ``get_opt_config`` is new.
"""
from __future__ import annotations

import torch
from torch import nn

from tensor_parallel_b200.models.common import CausalLMBase, LayerNorm, Linear, ModelOutput, ShapedConfig, init_weights_, past_length, update_kv
from tensor_parallel_b200.ops import functional as OF


class OPTConfig(ShapedConfig):
    model_type = "opt"

    def __init__(self, vocab_size=50272, hidden_size=768, num_hidden_layers=12, ffn_dim=3072, num_attention_heads=12,
                 max_position_embeddings=2048, **kw):
        super().__init__(vocab_size=vocab_size, hidden_size=hidden_size, num_hidden_layers=num_hidden_layers, ffn_dim=ffn_dim,
                         num_attention_heads=num_attention_heads, max_position_embeddings=max_position_embeddings, **kw)

    @classmethod
    def opt_13b(cls):
        return cls(hidden_size=5120, num_hidden_layers=40, ffn_dim=20480, num_attention_heads=40)


class OPTAttention(nn.Module):
    def __init__(self, config: OPTConfig):
        super().__init__()
        self.embed_dim = config.hidden_size
        self.num_heads = config.num_attention_heads
        self.head_dim = self.embed_dim // self.num_heads
        self.q_proj = Linear(self.embed_dim, self.embed_dim)
        self.k_proj = Linear(self.embed_dim, self.embed_dim)
        self.v_proj = Linear(self.embed_dim, self.embed_dim)
        self.out_proj = Linear(self.embed_dim, self.embed_dim)

    def forward(self, hidden_states, past_key_value=None, attention_mask=None, use_cache=False):
        b, s, _ = hidden_states.shape
        q, k, v = (proj(hidden_states).view(b, s, -1, self.head_dim) for proj in (self.q_proj, self.k_proj, self.v_proj))
        k_all, v_all, present = update_kv(past_key_value, k, v)
        out = OF.attention(q, k_all, v_all, causal=True, bias=attention_mask)
        return self.out_proj(out.reshape(b, s, -1)), None, (present if use_cache else None)


class OPTDecoderLayer(nn.Module):
    def __init__(self, config: OPTConfig):
        super().__init__()
        self.self_attn = OPTAttention(config)
        self.self_attn_layer_norm = LayerNorm(config.hidden_size)
        self.fc1 = Linear(config.hidden_size, config.ffn_dim)
        self.fc2 = Linear(config.ffn_dim, config.hidden_size)
        self.final_layer_norm = LayerNorm(config.hidden_size)

    def forward(self, hidden, past_key_value=None, attention_mask=None, use_cache=False):
        attn_out, _, present = self.self_attn(self.self_attn_layer_norm(hidden), past_key_value=past_key_value,
                                              attention_mask=attention_mask, use_cache=use_cache)
        hidden = hidden + attn_out
        hidden = hidden + self.fc2(OF.relu(self.fc1(self.final_layer_norm(hidden))))
        return hidden, present


class OPTDecoder(nn.Module):
    POSITION_OFFSET = 2

    def __init__(self, config: OPTConfig):
        super().__init__()
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size)
        self.embed_positions = nn.Embedding(config.max_position_embeddings + self.POSITION_OFFSET, config.hidden_size)
        self.layers = nn.ModuleList([OPTDecoderLayer(config) for _ in range(config.num_hidden_layers)])
        self.final_layer_norm = LayerNorm(config.hidden_size)

    def forward(self, input_ids=None, past_key_values=None, attention_mask=None, inputs_embeds=None, use_cache=False):
        hidden = self.embed_tokens(input_ids) if inputs_embeds is None else inputs_embeds
        b, s = hidden.shape[:2]
        offset = past_length(past_key_values)
        positions = torch.arange(offset, offset + s, device=hidden.device)[None].expand(b, s) + self.POSITION_OFFSET
        hidden = hidden + self.embed_positions(positions)
        presents = []
        for i, layer in enumerate(self.layers):
            hidden, present = layer(hidden, None if past_key_values is None else past_key_values[i], attention_mask, use_cache)
            presents.append(present)
        return self.final_layer_norm(hidden), (tuple(presents) if use_cache else None)


class OPTModel(nn.Module):
    def __init__(self, config: OPTConfig):
        super().__init__()
        self.config = config  # lets the predefined rule table be found when the bare model (no head) is wrapped
        self.decoder = OPTDecoder(config)

    def forward(self, *args, **kwargs):
        return self.decoder(*args, **kwargs)


class OPTForCausalLM(CausalLMBase):
    def __init__(self, config: OPTConfig):
        super().__init__()
        self.config = config
        self.model = OPTModel(config)
        self.lm_head = Linear(config.hidden_size, config.vocab_size, bias=False)
        init_weights_(self)
        self.lm_head.weight = self.model.decoder.embed_tokens.weight  # tied

    def forward(self, input_ids=None, past_key_values=None, attention_mask=None, inputs_embeds=None, labels=None,
                use_cache=False, **unused):
        hidden, presents = self.model(input_ids, past_key_values, attention_mask, inputs_embeds, use_cache)
        logits = self.lm_head(hidden)
        return ModelOutput(loss=self.lm_loss(logits, labels), logits=logits, past_key_values=presents)
