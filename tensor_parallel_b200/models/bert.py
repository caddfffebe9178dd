"""BERT-shaped bidirectional encoder.  Names / attributes (``attention.self.num_attention_heads``,
``all_head_size``) follow ``transformers`` ``BertModel`` as targeted by
``src/tensor_parallel/slicing_configs.py:140-177``.
"""
from __future__ import annotations

import torch
from torch import nn

from tensor_parallel_b200.models.common import LayerNorm, Linear, ModelOutput, ShapedConfig, init_weights_
from tensor_parallel_b200.ops import functional as OF


class BertConfig(ShapedConfig):
    model_type = "bert"

    def __init__(self, vocab_size=30522, hidden_size=768, num_hidden_layers=12, num_attention_heads=12, intermediate_size=3072,
                 max_position_embeddings=512, type_vocab_size=2, layer_norm_eps=1e-12, **kw):
        super().__init__(vocab_size=vocab_size, hidden_size=hidden_size, num_hidden_layers=num_hidden_layers,
                         num_attention_heads=num_attention_heads, intermediate_size=intermediate_size,
                         max_position_embeddings=max_position_embeddings, type_vocab_size=type_vocab_size, layer_norm_eps=layer_norm_eps, **kw)


class BertEmbeddings(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.word_embeddings = nn.Embedding(config.vocab_size, config.hidden_size)
        self.position_embeddings = nn.Embedding(config.max_position_embeddings, config.hidden_size)
        self.token_type_embeddings = nn.Embedding(config.type_vocab_size, config.hidden_size)
        self.LayerNorm = LayerNorm(config.hidden_size, eps=config.layer_norm_eps)

    def forward(self, input_ids, token_type_ids=None):
        b, s = input_ids.shape
        positions = torch.arange(s, device=input_ids.device)[None].expand(b, s)
        token_type_ids = torch.zeros_like(input_ids) if token_type_ids is None else token_type_ids
        return self.LayerNorm(self.word_embeddings(input_ids) + self.position_embeddings(positions) + self.token_type_embeddings(token_type_ids))


class BertSelfAttention(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.num_attention_heads = config.num_attention_heads
        self.attention_head_size = config.hidden_size // config.num_attention_heads
        self.all_head_size = config.hidden_size
        self.query = Linear(config.hidden_size, self.all_head_size)
        self.key = Linear(config.hidden_size, self.all_head_size)
        self.value = Linear(config.hidden_size, self.all_head_size)

    def forward(self, hidden_states, attention_mask=None):
        b, s, _ = hidden_states.shape
        q, k, v = (p(hidden_states).view(b, s, -1, self.attention_head_size) for p in (self.query, self.key, self.value))
        return OF.attention(q, k, v, causal=False, bias=attention_mask).reshape(b, s, -1)


class BertSelfOutput(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.dense = Linear(config.hidden_size, config.hidden_size)
        self.LayerNorm = LayerNorm(config.hidden_size, eps=config.layer_norm_eps)

    def forward(self, hidden_states, input_tensor):
        return self.LayerNorm(self.dense(hidden_states) + input_tensor)


class BertAttention(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.self = BertSelfAttention(config)
        self.output = BertSelfOutput(config)

    def forward(self, hidden_states, attention_mask=None):
        return self.output(self.self(hidden_states, attention_mask), hidden_states)


class BertIntermediate(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.dense = Linear(config.hidden_size, config.intermediate_size)

    def forward(self, x):
        return OF.gelu(self.dense(x))


class BertOutput(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.dense = Linear(config.intermediate_size, config.hidden_size)
        self.LayerNorm = LayerNorm(config.hidden_size, eps=config.layer_norm_eps)

    def forward(self, hidden_states, input_tensor):
        return self.LayerNorm(self.dense(hidden_states) + input_tensor)


class BertLayer(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.attention = BertAttention(config)
        self.intermediate = BertIntermediate(config)
        self.output = BertOutput(config)

    def forward(self, hidden_states, attention_mask=None):
        attended = self.attention(hidden_states, attention_mask)
        return self.output(self.intermediate(attended), attended)


class BertEncoder(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.layer = nn.ModuleList([BertLayer(config) for _ in range(config.num_hidden_layers)])

    def forward(self, hidden_states, attention_mask=None):
        for layer in self.layer:
            hidden_states = layer(hidden_states, attention_mask)
        return hidden_states


class BertModel(nn.Module):
    def __init__(self, config: BertConfig):
        super().__init__()
        self.config = config
        self.embeddings = BertEmbeddings(config)
        self.encoder = BertEncoder(config)
        self.pooler_dense = None
        init_weights_(self)

    def forward(self, input_ids=None, attention_mask=None, token_type_ids=None, **unused):
        hidden = self.embeddings(input_ids, token_type_ids)
        bias = None
        if attention_mask is not None:
            bias = (1.0 - attention_mask[:, None, None, :].to(hidden.dtype)) * torch.finfo(hidden.dtype).min
        return ModelOutput(last_hidden_state=self.encoder(hidden, bias))
