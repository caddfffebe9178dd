"""GPT-NeoX-shaped decoder: per-head interleaved fused QKV, partial rotary (``rotary_pct``),
parallel residual, untied ``embed_out``.  Names / attributes (``num_attention_heads``,
``hidden_size`` on the attention module) follow ``transformers`` ``GPTNeoXForCausalLM`` as
targeted by ``src/tensor_parallel/slicing_configs.py:241-282``.
"""
from __future__ import annotations

import torch
from torch import nn

from tensor_parallel_b200.models.common import CausalLMBase, LayerNorm, Linear, ModelOutput, ShapedConfig, init_weights_, past_length, update_kv
from tensor_parallel_b200.ops import functional as OF


class GPTNeoXConfig(ShapedConfig):
    model_type = "gpt_neox"

    def __init__(self, vocab_size=50432, hidden_size=6144, num_hidden_layers=44, num_attention_heads=64, intermediate_size=None,
                 rotary_pct=0.25, rotary_emb_base=10000.0, layer_norm_eps=1e-5, use_parallel_residual=True, **kw):
        super().__init__(vocab_size=vocab_size, hidden_size=hidden_size, num_hidden_layers=num_hidden_layers,
                         num_attention_heads=num_attention_heads, intermediate_size=intermediate_size or 4 * hidden_size,
                         rotary_pct=rotary_pct, rotary_emb_base=rotary_emb_base, layer_norm_eps=layer_norm_eps,
                         use_parallel_residual=use_parallel_residual, **kw)


class GPTNeoXAttention(nn.Module):
    def __init__(self, config: GPTNeoXConfig):
        super().__init__()
        self.num_attention_heads = config.num_attention_heads
        self.hidden_size = config.hidden_size
        self.head_size = config.hidden_size // config.num_attention_heads
        self.rotary_ndims = int(self.head_size * config.rotary_pct)
        self.rope_theta = config.rotary_emb_base
        self.query_key_value = Linear(config.hidden_size, 3 * config.hidden_size)
        self.dense = Linear(config.hidden_size, config.hidden_size)

    def forward(self, hidden_states, attention_mask=None, position_ids=None, layer_past=None, use_cache=False):
        b, s, _ = hidden_states.shape
        fused = self.query_key_value(hidden_states).view(b, s, self.num_attention_heads, 3, self.head_size)
        q, k, v = fused[..., 0, :], fused[..., 1, :], fused[..., 2, :]
        q = OF.apply_rope(q, position_ids, self.rope_theta, self.rotary_ndims)
        k = OF.apply_rope(k, position_ids, self.rope_theta, self.rotary_ndims)
        k_all, v_all, present = update_kv(layer_past, k, v)
        out = OF.attention(q, k_all, v_all, causal=True, bias=attention_mask)
        return self.dense(out.reshape(b, s, -1)), (present if use_cache else None)


class GPTNeoXMLP(nn.Module):
    def __init__(self, config: GPTNeoXConfig):
        super().__init__()
        self.dense_h_to_4h = Linear(config.hidden_size, config.intermediate_size)
        self.dense_4h_to_h = Linear(config.intermediate_size, config.hidden_size)

    def forward(self, x):
        return self.dense_4h_to_h(OF.gelu(self.dense_h_to_4h(x)))


class GPTNeoXLayer(nn.Module):
    def __init__(self, config: GPTNeoXConfig):
        super().__init__()
        self.use_parallel_residual = config.use_parallel_residual
        self.parallel_block = bool(config.use_parallel_residual)
        self.input_layernorm = LayerNorm(config.hidden_size, eps=config.layer_norm_eps)
        self.post_attention_layernorm = LayerNorm(config.hidden_size, eps=config.layer_norm_eps)
        self.attention = GPTNeoXAttention(config)
        self.mlp = GPTNeoXMLP(config)

    def forward(self, hidden, attention_mask=None, position_ids=None, layer_past=None, use_cache=False):
        attn_out, present = self.attention(self.input_layernorm(hidden), attention_mask=attention_mask, position_ids=position_ids,
                                           layer_past=layer_past, use_cache=use_cache)
        if self.use_parallel_residual:
            partial = attn_out + self.mlp(self.post_attention_layernorm(hidden))
            reduce = self.__dict__.get("_tp_block_reduce")
            return hidden + (partial if reduce is None else reduce(partial)), present
        hidden = hidden + attn_out
        return hidden + self.mlp(self.post_attention_layernorm(hidden)), present


class GPTNeoXModel(nn.Module):
    def __init__(self, config: GPTNeoXConfig):
        super().__init__()
        self.config = config  # lets the predefined rule table be found when the bare model (no head) is wrapped
        self.embed_in = nn.Embedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList([GPTNeoXLayer(config) for _ in range(config.num_hidden_layers)])
        self.final_layer_norm = LayerNorm(config.hidden_size, eps=config.layer_norm_eps)

    def forward(self, input_ids=None, past_key_values=None, attention_mask=None, position_ids=None, inputs_embeds=None, use_cache=False):
        hidden = self.embed_in(input_ids) if inputs_embeds is None else inputs_embeds
        b, s = hidden.shape[:2]
        offset = past_length(past_key_values)
        if position_ids is None:
            position_ids = torch.arange(offset, offset + s, device=hidden.device)[None].expand(b, s)
        presents = []
        for i, layer in enumerate(self.layers):
            hidden, present = layer(hidden, attention_mask, position_ids, None if past_key_values is None else past_key_values[i], use_cache)
            presents.append(present)
        return self.final_layer_norm(hidden), (tuple(presents) if use_cache else None)


class GPTNeoXForCausalLM(CausalLMBase):
    def __init__(self, config: GPTNeoXConfig):
        super().__init__()
        self.config = config
        self.gpt_neox = GPTNeoXModel(config)
        self.embed_out = Linear(config.hidden_size, config.vocab_size, bias=False)
        init_weights_(self)

    def forward(self, input_ids=None, past_key_values=None, attention_mask=None, position_ids=None, inputs_embeds=None,
                labels=None, use_cache=False, **unused):
        hidden, presents = self.gpt_neox(input_ids, past_key_values, attention_mask, position_ids, inputs_embeds, use_cache)
        logits, loss = self.head_and_loss(self.embed_out, hidden, labels)
        return ModelOutput(loss=loss, logits=logits, past_key_values=presents)
