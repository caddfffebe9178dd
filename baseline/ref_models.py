"""Plain-PyTorch Llama-shaped decoder for the reference arm of ``bench.py``.

Only stock ``torch`` operators are used (``nn.Linear`` -> cuBLAS, ``F.scaled_dot_product_attention``,
``torch.cat`` KV cache), i.e. what Hugging Face modelling code executed inside the reference's shards.
Module / attribute names are the ones the reference's Llama rule table patches
(``self_attn.hidden_size`` / ``num_heads`` / ``num_key_value_heads``; ``self_attn`` returns
``(out, None, present_kv)`` and takes ``past_key_value=``), so the unmodified reference applies to it.
Nothing from ``tensor_parallel_b200`` is imported here.
"""
import math

import torch
import torch.nn.functional as F
from torch import nn


class RefLlamaConfig:
    model_type = "llama"

    def __init__(self, vocab_size=32000, hidden_size=4096, intermediate_size=11008, num_hidden_layers=32,
                 num_attention_heads=32, num_key_value_heads=32, rms_norm_eps=1e-6, rope_theta=10000.0):
        self.vocab_size, self.hidden_size, self.intermediate_size = vocab_size, hidden_size, intermediate_size
        self.num_hidden_layers, self.num_attention_heads, self.num_key_value_heads = num_hidden_layers, num_attention_heads, num_key_value_heads
        self.rms_norm_eps, self.rope_theta = rms_norm_eps, rope_theta


class RefRMSNorm(nn.Module):
    def __init__(self, hidden, eps):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden))
        self.variance_epsilon = eps

    def forward(self, x):
        dtype = x.dtype
        x = x.float()
        x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.variance_epsilon)
        return self.weight * x.to(dtype)


def rotary_tables(position_ids, head_dim, theta, dtype):
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=position_ids.device, dtype=torch.float32) / head_dim))
    ang = position_ids[:, None, :, None].float() * inv_freq
    emb = torch.cat((ang, ang), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def _rotate_half(x):
    a, b = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2 :]
    return torch.cat((-b, a), dim=-1)


class RefAttention(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.hidden_size = cfg.hidden_size
        self.num_heads = cfg.num_attention_heads
        self.num_key_value_heads = cfg.num_key_value_heads
        self.head_dim = cfg.hidden_size // cfg.num_attention_heads
        self.rope_theta = cfg.rope_theta
        self.q_proj = nn.Linear(cfg.hidden_size, self.num_heads * self.head_dim, bias=False)
        self.k_proj = nn.Linear(cfg.hidden_size, self.num_key_value_heads * self.head_dim, bias=False)
        self.v_proj = nn.Linear(cfg.hidden_size, self.num_key_value_heads * self.head_dim, bias=False)
        self.o_proj = nn.Linear(self.num_heads * self.head_dim, cfg.hidden_size, bias=False)

    def forward(self, hidden_states, attention_mask=None, position_ids=None, past_key_value=None, output_attentions=False, use_cache=False,
                position_embeddings=None):
        b, s, _ = hidden_states.shape
        q = self.q_proj(hidden_states).view(b, s, self.num_heads, self.head_dim).transpose(1, 2)
        k = self.k_proj(hidden_states).view(b, s, self.num_key_value_heads, self.head_dim).transpose(1, 2)
        v = self.v_proj(hidden_states).view(b, s, self.num_key_value_heads, self.head_dim).transpose(1, 2)
        if position_embeddings is None:
            position_embeddings = rotary_tables(position_ids, self.head_dim, self.rope_theta, q.dtype)
        cos, sin = position_embeddings  # computed once per forward by the model, as Hugging Face's modelling code does
        q = q * cos + _rotate_half(q) * sin
        k = k * cos + _rotate_half(k) * sin
        if past_key_value is not None:
            k = torch.cat([past_key_value[0], k], dim=2)
            v = torch.cat([past_key_value[1], v], dim=2)
        present = (k, v) if use_cache else None
        if self.num_key_value_heads != self.num_heads:
            rep = self.num_heads // self.num_key_value_heads
            k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
        out = F.scaled_dot_product_attention(q, k, v, is_causal=(s > 1))
        out = out.transpose(1, 2).reshape(b, s, self.num_heads * self.head_dim)
        return self.o_proj(out), None, present


class RefMLP(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.gate_proj = nn.Linear(cfg.hidden_size, cfg.intermediate_size, bias=False)
        self.up_proj = nn.Linear(cfg.hidden_size, cfg.intermediate_size, bias=False)
        self.down_proj = nn.Linear(cfg.intermediate_size, cfg.hidden_size, bias=False)

    def forward(self, x):
        return self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))


class RefDecoderLayer(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.self_attn = RefAttention(cfg)
        self.mlp = RefMLP(cfg)
        self.input_layernorm = RefRMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.post_attention_layernorm = RefRMSNorm(cfg.hidden_size, cfg.rms_norm_eps)

    def forward(self, h, position_ids, past_key_value=None, use_cache=False, position_embeddings=None):
        a, _, present = self.self_attn(self.input_layernorm(h), position_ids=position_ids, past_key_value=past_key_value, use_cache=use_cache,
                                       position_embeddings=position_embeddings)
        h = h + a
        return h + self.mlp(self.post_attention_layernorm(h)), present


class RefLlamaModel(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.layers = nn.ModuleList([RefDecoderLayer(cfg) for _ in range(cfg.num_hidden_layers)])
        self.norm = RefRMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.rotary_dim, self.rope_theta = cfg.hidden_size // cfg.num_attention_heads, cfg.rope_theta

    def forward(self, input_ids, past_key_values=None, use_cache=False):
        h = self.embed_tokens(input_ids)
        b, s = input_ids.shape
        offset = 0 if past_key_values is None else past_key_values[0][0].shape[2]
        position_ids = torch.arange(offset, offset + s, device=h.device)[None].expand(b, s)
        presents = []
        rotary = rotary_tables(position_ids, self.rotary_dim, self.rope_theta, h.dtype)
        for i, layer in enumerate(self.layers):
            h, present = layer(h, position_ids, None if past_key_values is None else past_key_values[i], use_cache, rotary)
            presents.append(present)
        return self.norm(h), tuple(presents)


class RefLlamaForCausalLM(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.config = cfg
        self.model = RefLlamaModel(cfg)
        self.lm_head = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False)

    def forward(self, input_ids, past_key_values=None, use_cache=True, last_only=False):
        h, presents = self.model(input_ids, past_key_values, use_cache)
        if last_only:
            h = h[:, -1:]
        return self.lm_head(h), presents


# ------------------------------------------------------------------------------------------------
# Falcon / RefinedWeb ("new decoder architecture"): parallel attention + MLP block, grouped fused QKV
# ------------------------------------------------------------------------------------------------


class RefFalconConfig:
    model_type = "RefinedWeb"

    def __init__(self, vocab_size=65024, hidden_size=8192, n_layer=60, n_head=128, n_head_kv=8, layer_norm_epsilon=1e-5,
                 rope_theta=10000.0, ffn_mult=4):
        self.vocab_size, self.hidden_size, self.n_layer, self.n_head, self.n_head_kv = vocab_size, hidden_size, n_layer, n_head, n_head_kv
        self.layer_norm_epsilon, self.rope_theta, self.ffn_mult = layer_norm_epsilon, rope_theta, ffn_mult
        self.bias = self.alibi = False
        self.num_attention_heads, self.num_hidden_layers = n_head, n_layer


class RefFalconAttention(nn.Module):
    """Attribute names (``num_kv``, ``num_heads``) and the ``layer_past`` keyword are the ones the reference's
    ``get_refined_web_config`` patches (``src/tensor_parallel/slicing_configs.py:409-462``)."""

    def __init__(self, cfg):
        super().__init__()
        self.hidden_size, self.num_heads, self.num_kv = cfg.hidden_size, cfg.n_head, cfg.n_head_kv
        self.head_dim = cfg.hidden_size // cfg.n_head
        self.rope_theta = cfg.rope_theta
        self.query_key_value = nn.Linear(cfg.hidden_size, (self.num_heads + 2 * self.num_kv) * self.head_dim, bias=False)
        self.dense = nn.Linear(cfg.hidden_size, cfg.hidden_size, bias=False)

    def forward(self, hidden_states, layer_past=None, position_embeddings=None, use_cache=False):
        b, s, _ = hidden_states.shape
        q_per_kv = self.num_heads // self.num_kv
        fused = self.query_key_value(hidden_states).view(b, s, self.num_kv, q_per_kv + 2, self.head_dim)
        q = fused[:, :, :, :q_per_kv].reshape(b, s, self.num_heads, self.head_dim).transpose(1, 2)
        k, v = fused[:, :, :, q_per_kv].transpose(1, 2), fused[:, :, :, q_per_kv + 1].transpose(1, 2)
        cos, sin = position_embeddings
        q = q * cos + _rotate_half(q) * sin
        k = k * cos + _rotate_half(k) * sin
        if layer_past is not None:
            k = torch.cat([layer_past[0], k], dim=2)
            v = torch.cat([layer_past[1], v], dim=2)
        present = (k, v) if use_cache else None
        if q_per_kv > 1:
            k, v = k.repeat_interleave(q_per_kv, dim=1), v.repeat_interleave(q_per_kv, dim=1)
        out = F.scaled_dot_product_attention(q, k, v, is_causal=(s > 1))
        return self.dense(out.transpose(1, 2).reshape(b, s, self.num_heads * self.head_dim)), present


class RefFalconMLP(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.dense_h_to_4h = nn.Linear(cfg.hidden_size, cfg.ffn_mult * cfg.hidden_size, bias=False)
        self.dense_4h_to_h = nn.Linear(cfg.ffn_mult * cfg.hidden_size, cfg.hidden_size, bias=False)

    def forward(self, x):
        return self.dense_4h_to_h(F.gelu(self.dense_h_to_4h(x)))


class RefFalconLayer(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.ln_attn = nn.LayerNorm(cfg.hidden_size, eps=cfg.layer_norm_epsilon)
        self.ln_mlp = nn.LayerNorm(cfg.hidden_size, eps=cfg.layer_norm_epsilon)
        self.self_attention = RefFalconAttention(cfg)
        self.mlp = RefFalconMLP(cfg)

    def forward(self, h, layer_past, rotary, use_cache):
        a, present = self.self_attention(self.ln_attn(h), layer_past=layer_past, position_embeddings=rotary, use_cache=use_cache)
        return h + a + self.mlp(self.ln_mlp(h)), present


class RefFalconModel(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.word_embeddings = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.h = nn.ModuleList([RefFalconLayer(cfg) for _ in range(cfg.n_layer)])
        self.ln_f = nn.LayerNorm(cfg.hidden_size, eps=cfg.layer_norm_epsilon)
        self.rotary_dim, self.rope_theta = cfg.hidden_size // cfg.n_head, cfg.rope_theta

    def forward(self, input_ids, past_key_values=None, use_cache=False):
        h = self.word_embeddings(input_ids)
        b, s = input_ids.shape
        offset = 0 if past_key_values is None else past_key_values[0][0].shape[2]
        position_ids = torch.arange(offset, offset + s, device=h.device)[None].expand(b, s)
        rotary = rotary_tables(position_ids, self.rotary_dim, self.rope_theta, h.dtype)
        presents = []
        for i, layer in enumerate(self.h):
            h, present = layer(h, None if past_key_values is None else past_key_values[i], rotary, use_cache)
            presents.append(present)
        return self.ln_f(h), tuple(presents)


class RefFalconForCausalLM(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.config = cfg
        self.transformer = RefFalconModel(cfg)
        self.lm_head = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False)
        self.lm_head.weight = self.transformer.word_embeddings.weight  # tied

    def forward(self, input_ids, past_key_values=None, use_cache=True, last_only=False):
        h, presents = self.transformer(input_ids, past_key_values, use_cache)
        if last_only:
            h = h[:, -1:]
        return self.lm_head(h), presents
