"""BLOOM-shaped decoder: ALiBi position bias, per-head interleaved fused QKV, embedding LayerNorm,
GeLU MLP, lm_head tied to ``word_embeddings``.  The block builds ALiBi once for all heads and
hands it to ``self_attention(..., alibi=...)`` in the ``[batch * heads, 1, kv_len]`` layout, which
the BLOOM table slices per rank (``src/tensor_parallel/slicing_configs.py:32-72``).
"""
from __future__ import annotations

import math

import torch
from torch import nn

from tensor_parallel_b200.models.common import CausalLMBase, LayerNorm, Linear, ModelOutput, ShapedConfig, init_weights_, past_length, update_kv
from tensor_parallel_b200.ops import functional as OF


class BloomConfig(ShapedConfig):
    model_type = "bloom"

    def __init__(self, vocab_size=250880, hidden_size=1024, n_layer=24, n_head=16, layer_norm_epsilon=1e-5, **kw):
        super().__init__(vocab_size=vocab_size, hidden_size=hidden_size, n_layer=n_layer, n_head=n_head,
                         layer_norm_epsilon=layer_norm_epsilon, num_attention_heads=n_head, num_hidden_layers=n_layer, **kw)


def build_alibi_tensor(batch: int, kv_len: int, num_heads: int, dtype, device) -> torch.Tensor:
    """``[batch * num_heads, 1, kv_len]`` slopes * key position."""
    closest = 2 ** math.floor(math.log2(num_heads))
    base = 2.0 ** (-(2.0 ** -(math.log2(closest) - 3)))
    slopes = torch.pow(torch.tensor(base), torch.arange(1, closest + 1, dtype=torch.float32))
    if closest != num_heads:
        extra_base = 2.0 ** (-(2.0 ** -(math.log2(2 * closest) - 3)))
        extra = torch.pow(torch.tensor(extra_base), torch.arange(1, 2 * (num_heads - closest) + 1, 2, dtype=torch.float32))
        slopes = torch.cat([slopes, extra])
    positions = torch.arange(kv_len, dtype=torch.float32)[None, None, :]
    alibi = slopes[None, :, None] * positions  # [1, heads, kv]
    return alibi.expand(batch, -1, -1).reshape(batch * num_heads, 1, kv_len).to(device=device, dtype=dtype)


class BloomAttention(nn.Module):
    def __init__(self, config: BloomConfig):
        super().__init__()
        self.hidden_size = config.hidden_size
        self.num_heads = config.n_head
        self.head_dim = config.hidden_size // config.n_head
        self.query_key_value = Linear(config.hidden_size, 3 * config.hidden_size)
        self.dense = Linear(config.hidden_size, config.hidden_size)

    def forward(self, hidden_states, alibi=None, attention_mask=None, layer_past=None, use_cache=False):
        b, s, _ = hidden_states.shape
        fused = self.query_key_value(hidden_states).view(b, s, self.num_heads, 3, self.head_dim)
        q, k, v = fused[..., 0, :], fused[..., 1, :], fused[..., 2, :]
        k_all, v_all, present = update_kv(layer_past, k, v)
        bias = alibi.view(b, self.num_heads, 1, -1) if alibi is not None else None
        if attention_mask is not None:
            bias = attention_mask if bias is None else bias + attention_mask
        out = OF.attention(q, k_all, v_all, causal=True, bias=bias)
        return self.dense(out.reshape(b, s, -1)), (present if use_cache else None)


class BloomMLP(nn.Module):
    def __init__(self, config: BloomConfig):
        super().__init__()
        self.dense_h_to_4h = Linear(config.hidden_size, 4 * config.hidden_size)
        self.dense_4h_to_h = Linear(4 * config.hidden_size, config.hidden_size)

    def forward(self, x):
        return self.dense_4h_to_h(OF.gelu(self.dense_h_to_4h(x), approximate="tanh"))


class BloomBlock(nn.Module):
    def __init__(self, config: BloomConfig):
        super().__init__()
        self.input_layernorm = LayerNorm(config.hidden_size, eps=config.layer_norm_epsilon)
        self.self_attention = BloomAttention(config)
        self.post_attention_layernorm = LayerNorm(config.hidden_size, eps=config.layer_norm_epsilon)
        self.mlp = BloomMLP(config)

    def forward(self, hidden, alibi=None, attention_mask=None, layer_past=None, use_cache=False):
        attn_out, present = self.self_attention(self.input_layernorm(hidden), alibi=alibi, attention_mask=attention_mask,
                                                layer_past=layer_past, use_cache=use_cache)
        hidden = hidden + attn_out
        return hidden + self.mlp(self.post_attention_layernorm(hidden)), present


class BloomModel(nn.Module):
    def __init__(self, config: BloomConfig):
        super().__init__()
        self.config = config  # lets the predefined rule table be found when the bare model (no head) is wrapped
        self.num_heads = config.n_head
        self.word_embeddings = nn.Embedding(config.vocab_size, config.hidden_size)
        self.word_embeddings_layernorm = LayerNorm(config.hidden_size, eps=config.layer_norm_epsilon)
        self.h = nn.ModuleList([BloomBlock(config) for _ in range(config.n_layer)])
        self.ln_f = LayerNorm(config.hidden_size, eps=config.layer_norm_epsilon)

    def forward(self, input_ids=None, past_key_values=None, attention_mask=None, inputs_embeds=None, use_cache=False):
        hidden = self.word_embeddings(input_ids) if inputs_embeds is None else inputs_embeds
        hidden = self.word_embeddings_layernorm(hidden)
        b, s = hidden.shape[:2]
        kv_len = past_length(past_key_values) + s
        alibi = build_alibi_tensor(b, kv_len, self.num_heads, hidden.dtype, hidden.device)
        presents = []
        for i, block in enumerate(self.h):
            hidden, present = block(hidden, alibi=alibi, attention_mask=attention_mask,
                                    layer_past=None if past_key_values is None else past_key_values[i], use_cache=use_cache)
            presents.append(present)
        return self.ln_f(hidden), (tuple(presents) if use_cache else None)


class BloomForCausalLM(CausalLMBase):
    def __init__(self, config: BloomConfig):
        super().__init__()
        self.config = config
        self.transformer = BloomModel(config)
        self.lm_head = Linear(config.hidden_size, config.vocab_size, bias=False)
        init_weights_(self)
        self.lm_head.weight = self.transformer.word_embeddings.weight  # tied

    def forward(self, input_ids=None, past_key_values=None, attention_mask=None, inputs_embeds=None, labels=None, use_cache=False, **unused):
        hidden, presents = self.transformer(input_ids, past_key_values, attention_mask, inputs_embeds, use_cache)
        logits = self.lm_head(hidden)
        return ModelOutput(loss=self.lm_loss(logits, labels), logits=logits, past_key_values=presents)
