"""GPT-2-shaped decoder: learned positions, fused ``c_attn`` QKV stored as ``Conv1D``
(``weight[in, out]``), GeLU MLP, lm_head tied to ``wte``.  Names and attributes follow
``transformers`` ``GPT2LMHeadModel`` as targeted by ``src/tensor_parallel/slicing_configs.py:180-238``.
"""
from __future__ import annotations

import torch
from torch import nn

from tensor_parallel_b200.models.common import CausalLMBase, Conv1D, LayerNorm, Linear, ModelOutput, ShapedConfig, init_weights_, past_length, update_kv
from tensor_parallel_b200.ops import functional as OF


class GPT2Config(ShapedConfig):
    model_type = "gpt2"

    def __init__(self, vocab_size=50257, n_positions=1024, n_embd=768, n_layer=12, n_head=12, n_inner=None,
                 layer_norm_epsilon=1e-5, **kw):
        super().__init__(vocab_size=vocab_size, n_positions=n_positions, n_embd=n_embd, n_layer=n_layer, n_head=n_head,
                         n_inner=n_inner or 4 * n_embd, layer_norm_epsilon=layer_norm_epsilon,
                         hidden_size=n_embd, num_attention_heads=n_head, num_hidden_layers=n_layer, **kw)


class GPT2Attention(nn.Module):
    def __init__(self, config: GPT2Config):
        super().__init__()
        self.embed_dim = config.n_embd
        self.num_heads = config.n_head
        self.head_dim = self.embed_dim // self.num_heads
        self.split_size = self.embed_dim
        self.c_attn = Conv1D(3 * self.embed_dim, self.embed_dim)
        self.c_proj = Conv1D(self.embed_dim, self.embed_dim)

    def forward(self, hidden_states, layer_past=None, attention_mask=None, use_cache=False):
        b, s, _ = hidden_states.shape
        q, k, v = self.c_attn(hidden_states).split(self.split_size, dim=2)
        q, k, v = (t.reshape(b, s, -1, self.head_dim) for t in (q, k, v))
        k_all, v_all, present = update_kv(layer_past, k, v)
        out = OF.attention(q, k_all, v_all, causal=True, bias=attention_mask)
        return self.c_proj(out.reshape(b, s, -1)), (present if use_cache else None)


class GPT2MLP(nn.Module):
    def __init__(self, config: GPT2Config):
        super().__init__()
        self.c_fc = Conv1D(config.n_inner, config.n_embd)
        self.c_proj = Conv1D(config.n_embd, config.n_inner)

    def forward(self, x):
        return self.c_proj(OF.gelu(self.c_fc(x), approximate="tanh"))


class GPT2Block(nn.Module):
    def __init__(self, config: GPT2Config):
        super().__init__()
        self.ln_1 = LayerNorm(config.n_embd, eps=config.layer_norm_epsilon)
        self.attn = GPT2Attention(config)
        self.ln_2 = LayerNorm(config.n_embd, eps=config.layer_norm_epsilon)
        self.mlp = GPT2MLP(config)

    def forward(self, hidden, layer_past=None, attention_mask=None, use_cache=False):
        attn_out, present = self.attn(self.ln_1(hidden), layer_past=layer_past, attention_mask=attention_mask, use_cache=use_cache)
        hidden = hidden + attn_out
        return hidden + self.mlp(self.ln_2(hidden)), present


class GPT2Model(nn.Module):
    def __init__(self, config: GPT2Config):
        super().__init__()
        self.config = config  # lets the predefined rule table be found when the bare model (no head) is wrapped
        self.wte = nn.Embedding(config.vocab_size, config.n_embd)
        self.wpe = nn.Embedding(config.n_positions, config.n_embd)
        self.h = nn.ModuleList([GPT2Block(config) for _ in range(config.n_layer)])
        self.ln_f = LayerNorm(config.n_embd, eps=config.layer_norm_epsilon)

    def forward(self, input_ids=None, past_key_values=None, attention_mask=None, position_ids=None, inputs_embeds=None, use_cache=False):
        hidden = self.wte(input_ids) if inputs_embeds is None else inputs_embeds
        b, s = hidden.shape[:2]
        offset = past_length(past_key_values)
        if position_ids is None:
            position_ids = torch.arange(offset, offset + s, device=hidden.device)[None].expand(b, s)
        hidden = hidden + self.wpe(position_ids)
        presents = []
        for i, block in enumerate(self.h):
            hidden, present = block(hidden, None if past_key_values is None else past_key_values[i], attention_mask, use_cache)
            presents.append(present)
        return self.ln_f(hidden), (tuple(presents) if use_cache else None)


class GPT2LMHeadModel(CausalLMBase):
    def __init__(self, config: GPT2Config):
        super().__init__()
        self.config = config
        self.transformer = GPT2Model(config)
        self.lm_head = Linear(config.n_embd, config.vocab_size, bias=False)
        init_weights_(self)
        self.lm_head.weight = self.transformer.wte.weight  # tied

    def forward(self, input_ids=None, past_key_values=None, attention_mask=None, position_ids=None, inputs_embeds=None,
                labels=None, use_cache=False, **unused):
        hidden, presents = self.transformer(input_ids, past_key_values, attention_mask, position_ids, inputs_embeds, use_cache)
        logits = self.lm_head(hidden)
        return ModelOutput(loss=self.lm_loss(logits, labels), logits=logits, past_key_values=presents)
