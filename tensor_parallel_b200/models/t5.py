"""T5-shaped encoder-decoder: bucketed relative position bias (first block of each stack owns
the table), un-scaled dot-product attention, RMS-style ``T5LayerNorm``, ReLU or gated-GeLU MLP
(``DenseReluDense``).  Names / attributes (``n_heads``, ``inner_dim``, ``SelfAttention``,
``EncDecAttention``) follow ``transformers`` ``T5ForConditionalGeneration`` as targeted by
``src/tensor_parallel/slicing_configs.py:75-137``.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
from torch import nn

from tensor_parallel_b200.models.common import Linear, ModelOutput, RMSNorm, ShapedConfig, init_weights_
from tensor_parallel_b200.ops import functional as OF


class T5Config(ShapedConfig):
    model_type = "t5"

    def __init__(self, vocab_size=32128, d_model=512, d_kv=64, d_ff=2048, num_layers=6, num_decoder_layers=None, num_heads=8,
                 relative_attention_num_buckets=32, relative_attention_max_distance=128, layer_norm_epsilon=1e-6,
                 feed_forward_proj="relu", tie_word_embeddings=True, decoder_start_token_id=0, pad_token_id=0, **kw):
        super().__init__(vocab_size=vocab_size, d_model=d_model, d_kv=d_kv, d_ff=d_ff, num_layers=num_layers,
                         num_decoder_layers=num_decoder_layers or num_layers, num_heads=num_heads,
                         relative_attention_num_buckets=relative_attention_num_buckets,
                         relative_attention_max_distance=relative_attention_max_distance, layer_norm_epsilon=layer_norm_epsilon,
                         feed_forward_proj=feed_forward_proj, tie_word_embeddings=tie_word_embeddings,
                         decoder_start_token_id=decoder_start_token_id, pad_token_id=pad_token_id,
                         is_gated_act=feed_forward_proj.startswith("gated"), **kw)

    @classmethod
    def flan_t5_xl(cls):
        return cls(d_model=2048, d_kv=64, d_ff=5120, num_layers=24, num_heads=32, feed_forward_proj="gated-gelu",
                   tie_word_embeddings=False)


def relative_position_bucket(relative_position, bidirectional: bool, num_buckets: int, max_distance: int):
    buckets = torch.zeros_like(relative_position)
    if bidirectional:
        num_buckets //= 2
        buckets = buckets + (relative_position > 0).long() * num_buckets
        relative_position = relative_position.abs()
    else:
        relative_position = -torch.min(relative_position, torch.zeros_like(relative_position))
    max_exact = num_buckets // 2
    is_small = relative_position < max_exact
    large = max_exact + (
        torch.log(relative_position.float().clamp(min=1) / max_exact) / math.log(max_distance / max_exact) * (num_buckets - max_exact)
    ).long()
    large = torch.min(large, torch.full_like(large, num_buckets - 1))
    return buckets + torch.where(is_small, relative_position, large)


class T5Attention(nn.Module):
    def __init__(self, config: T5Config, has_relative_attention_bias: bool, is_decoder: bool):
        super().__init__()
        self.is_decoder = is_decoder
        self.has_relative_attention_bias = has_relative_attention_bias
        self.relative_attention_num_buckets = config.relative_attention_num_buckets
        self.relative_attention_max_distance = config.relative_attention_max_distance
        self.d_model = config.d_model
        self.key_value_proj_dim = config.d_kv
        self.n_heads = config.num_heads
        self.inner_dim = self.n_heads * self.key_value_proj_dim
        self.q = Linear(self.d_model, self.inner_dim, bias=False)
        self.k = Linear(self.d_model, self.inner_dim, bias=False)
        self.v = Linear(self.d_model, self.inner_dim, bias=False)
        self.o = Linear(self.inner_dim, self.d_model, bias=False)
        if has_relative_attention_bias:
            self.relative_attention_bias = nn.Embedding(self.relative_attention_num_buckets, self.n_heads)

    def compute_bias(self, query_length: int, key_length: int, device):
        ctx = torch.arange(key_length - query_length, key_length, device=device)[:, None]
        mem = torch.arange(key_length, device=device)[None, :]
        buckets = relative_position_bucket(mem - ctx, not self.is_decoder, self.relative_attention_num_buckets,
                                           self.relative_attention_max_distance)
        return self.relative_attention_bias(buckets).permute(2, 0, 1)[None]  # [1, heads, q, k]

    def forward(self, hidden_states, mask=None, key_value_states=None, position_bias=None, past_key_value=None, use_cache=False):
        b, s, _ = hidden_states.shape
        d = self.key_value_proj_dim
        q = self.q(hidden_states).view(b, s, -1, d)
        is_cross = key_value_states is not None
        if is_cross and past_key_value is not None:
            k_cache, v_cache = past_key_value[0], past_key_value[1]
        else:
            source = key_value_states if is_cross else hidden_states
            k_cache = self.k(source).view(b, source.shape[1], -1, d).transpose(1, 2)
            v_cache = self.v(source).view(b, source.shape[1], -1, d).transpose(1, 2)
            if not is_cross and past_key_value is not None:
                k_cache = torch.cat((past_key_value[0], k_cache), dim=2)
                v_cache = torch.cat((past_key_value[1], v_cache), dim=2)
        key_length = k_cache.shape[2]
        if position_bias is None:
            if self.has_relative_attention_bias:
                position_bias = self.compute_bias(s, key_length, hidden_states.device)
            else:
                position_bias = torch.zeros(1, q.shape[2], s, key_length, device=hidden_states.device, dtype=hidden_states.dtype)
            if mask is not None:
                position_bias = position_bias + mask
        causal = self.is_decoder and not is_cross
        out = OF.attention(q, k_cache.transpose(1, 2), v_cache.transpose(1, 2), causal=causal, bias=position_bias, scale=1.0)
        out = self.o(out.reshape(b, s, -1))
        present = (k_cache, v_cache) if (self.is_decoder and use_cache) else None
        return out, present, position_bias


class T5LayerSelfAttention(nn.Module):
    def __init__(self, config, has_relative_attention_bias, is_decoder):
        super().__init__()
        self.SelfAttention = T5Attention(config, has_relative_attention_bias, is_decoder)
        self.layer_norm = RMSNorm(config.d_model, config.layer_norm_epsilon)

    def forward(self, hidden, attention_mask=None, position_bias=None, past_key_value=None, use_cache=False):
        out = self.SelfAttention(self.layer_norm(hidden), mask=attention_mask, position_bias=position_bias,
                                 past_key_value=past_key_value, use_cache=use_cache)
        return (hidden + out[0],) + tuple(out[1:])


class T5LayerCrossAttention(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.EncDecAttention = T5Attention(config, False, True)
        self.layer_norm = RMSNorm(config.d_model, config.layer_norm_epsilon)

    def forward(self, hidden, key_value_states, attention_mask=None, position_bias=None, past_key_value=None, use_cache=False):
        out = self.EncDecAttention(self.layer_norm(hidden), mask=attention_mask, key_value_states=key_value_states,
                                   position_bias=position_bias, past_key_value=past_key_value, use_cache=use_cache)
        return (hidden + out[0],) + tuple(out[1:])


class T5DenseActDense(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.wi = Linear(config.d_model, config.d_ff, bias=False)
        self.wo = Linear(config.d_ff, config.d_model, bias=False)

    def forward(self, x):
        return self.wo(OF.relu(self.wi(x)))


class T5DenseGatedActDense(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.wi_0 = Linear(config.d_model, config.d_ff, bias=False)
        self.wi_1 = Linear(config.d_model, config.d_ff, bias=False)
        self.wo = Linear(config.d_ff, config.d_model, bias=False)

    def forward(self, x):
        return self.wo(OF.geglu(self.wi_0(x), self.wi_1(x), approximate="tanh"))


class T5LayerFF(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.DenseReluDense = T5DenseGatedActDense(config) if config.is_gated_act else T5DenseActDense(config)
        self.layer_norm = RMSNorm(config.d_model, config.layer_norm_epsilon)

    def forward(self, hidden):
        return hidden + self.DenseReluDense(self.layer_norm(hidden))


class T5Block(nn.Module):
    def __init__(self, config, has_relative_attention_bias, is_decoder):
        super().__init__()
        self.is_decoder = is_decoder
        self.layer = nn.ModuleList([T5LayerSelfAttention(config, has_relative_attention_bias, is_decoder)])
        if is_decoder:
            self.layer.append(T5LayerCrossAttention(config))
        self.layer.append(T5LayerFF(config))

    def forward(self, hidden, attention_mask=None, position_bias=None, encoder_hidden_states=None, encoder_attention_mask=None,
                encoder_decoder_position_bias=None, past_key_value=None, use_cache=False):
        self_past = cross_past = None
        if past_key_value is not None:
            self_past, cross_past = tuple(past_key_value[:2]), (tuple(past_key_value[2:]) if len(past_key_value) > 2 else None)
        hidden, present, position_bias = self.layer[0](hidden, attention_mask, position_bias, self_past, use_cache)
        if self.is_decoder and encoder_hidden_states is not None:
            hidden, cross_present, encoder_decoder_position_bias = self.layer[1](
                hidden, encoder_hidden_states, encoder_attention_mask, encoder_decoder_position_bias, cross_past, use_cache)
            if present is not None:
                present = tuple(present) + tuple(cross_present)
        hidden = self.layer[-1](hidden)
        return hidden, present, position_bias, encoder_decoder_position_bias


class T5Stack(nn.Module):
    def __init__(self, config, embed_tokens, is_decoder):
        super().__init__()
        self.is_decoder = is_decoder
        self.embed_tokens = embed_tokens
        n = config.num_decoder_layers if is_decoder else config.num_layers
        self.block = nn.ModuleList([T5Block(config, i == 0, is_decoder) for i in range(n)])
        self.final_layer_norm = RMSNorm(config.d_model, config.layer_norm_epsilon)

    def forward(self, input_ids=None, attention_mask=None, encoder_hidden_states=None, encoder_attention_mask=None,
                inputs_embeds=None, past_key_values=None, use_cache=False):
        hidden = self.embed_tokens(input_ids) if inputs_embeds is None else inputs_embeds

        def additive(mask, like):
            if mask is None:
                return None
            return (1.0 - mask[:, None, None, :].to(like.dtype)) * torch.finfo(like.dtype).min

        mask = additive(attention_mask, hidden)
        enc_mask = additive(encoder_attention_mask, hidden)
        position_bias = enc_dec_bias = None
        presents = []
        for i, block in enumerate(self.block):
            hidden, present, position_bias, enc_dec_bias = block(
                hidden, mask, position_bias, encoder_hidden_states, enc_mask, enc_dec_bias,
                None if past_key_values is None else past_key_values[i], use_cache)
            presents.append(present)
        hidden = self.final_layer_norm(hidden)
        return ModelOutput(last_hidden_state=hidden, past_key_values=tuple(presents) if (use_cache and self.is_decoder) else None)


class T5ForConditionalGeneration(nn.Module):
    def __init__(self, config: T5Config):
        super().__init__()
        self.config = config
        self.model_dim = config.d_model
        self.shared = nn.Embedding(config.vocab_size, config.d_model)
        self.encoder = T5Stack(config, self.shared, is_decoder=False)
        self.decoder = T5Stack(config, self.shared, is_decoder=True)
        self.lm_head = Linear(config.d_model, config.vocab_size, bias=False)
        init_weights_(self, std=0.05)
        if config.tie_word_embeddings:
            self.lm_head.weight = self.shared.weight

    def get_encoder(self):
        return self.encoder

    def _shift_right(self, labels):
        shifted = labels.new_zeros(labels.shape)
        shifted[:, 1:] = labels[:, :-1]
        shifted[:, 0] = self.config.decoder_start_token_id
        return shifted.masked_fill(shifted == -100, self.config.pad_token_id)

    def forward(self, input_ids=None, attention_mask=None, decoder_input_ids=None, decoder_attention_mask=None,
                encoder_outputs=None, past_key_values=None, inputs_embeds=None, labels=None, use_cache=False, **unused):
        if encoder_outputs is None:
            encoder_outputs = self.encoder(input_ids=input_ids, attention_mask=attention_mask, inputs_embeds=inputs_embeds)
        enc_hidden = encoder_outputs["last_hidden_state"] if isinstance(encoder_outputs, dict) else encoder_outputs[0]
        if labels is not None and decoder_input_ids is None:
            decoder_input_ids = self._shift_right(labels)
        dec = self.decoder(input_ids=decoder_input_ids, attention_mask=decoder_attention_mask, encoder_hidden_states=enc_hidden,
                           encoder_attention_mask=attention_mask, past_key_values=past_key_values, use_cache=use_cache)
        hidden = dec.last_hidden_state
        if self.config.tie_word_embeddings:
            hidden = hidden * (self.model_dim ** -0.5)
        logits = self.lm_head(hidden)
        loss = None
        if labels is not None:
            loss = OF.cross_entropy(logits, labels.to(logits.device))
        return ModelOutput(loss=loss, logits=logits, past_key_values=dec.past_key_values, encoder_last_hidden_state=enc_hidden)

    @staticmethod
    def _reorder_cache(past, beam_idx):
        return tuple(tuple(t.index_select(0, beam_idx.to(t.device)) for t in layer) for layer in past)
