"""GPT-J- and CodeGen-shaped decoders: one LayerNorm feeding attention and MLP in parallel,
interleaved rotary embedding on the first ``rotary_dim`` features, untied lm_head with bias.
GPT-J keeps separate ``q_proj/k_proj/v_proj``; CodeGen fuses them as ``qkv_proj`` in the
``[mp=4][q|v|k][heads/4][head_dim]`` row layout (``src/tensor_parallel/slicing_configs.py:285-342``).
"""
from __future__ import annotations

import torch
from torch import nn

from tensor_parallel_b200.models.common import CausalLMBase, LayerNorm, Linear, ModelOutput, ShapedConfig, init_weights_, past_length, update_kv
from tensor_parallel_b200.ops import functional as OF


class GPTJConfig(ShapedConfig):
    model_type = "gptj"

    def __init__(self, vocab_size=50400, n_embd=4096, n_layer=28, n_head=16, rotary_dim=64, n_inner=None,
                 layer_norm_epsilon=1e-5, rope_theta=10000.0, **kw):
        super().__init__(vocab_size=vocab_size, n_embd=n_embd, n_layer=n_layer, n_head=n_head, rotary_dim=rotary_dim,
                         n_inner=n_inner or 4 * n_embd, layer_norm_epsilon=layer_norm_epsilon, rope_theta=rope_theta,
                         hidden_size=n_embd, num_attention_heads=n_head, num_hidden_layers=n_layer, **kw)


class CodeGenConfig(GPTJConfig):
    model_type = "codegen"


class GPTJAttention(nn.Module):
    def __init__(self, config: GPTJConfig):
        super().__init__()
        self.embed_dim = config.n_embd
        self.num_attention_heads = config.n_head
        self.head_dim = self.embed_dim // self.num_attention_heads
        self.rotary_dim, self.rope_theta = config.rotary_dim, config.rope_theta
        self.q_proj = Linear(self.embed_dim, self.embed_dim, bias=False)
        self.k_proj = Linear(self.embed_dim, self.embed_dim, bias=False)
        self.v_proj = Linear(self.embed_dim, self.embed_dim, bias=False)
        self.out_proj = Linear(self.embed_dim, self.embed_dim, bias=False)

    def _qkv(self, hidden_states):
        b, s, _ = hidden_states.shape
        return tuple(p(hidden_states).view(b, s, -1, self.head_dim) for p in (self.q_proj, self.k_proj, self.v_proj))

    def forward(self, hidden_states, layer_past=None, attention_mask=None, position_ids=None, use_cache=False):
        b, s, _ = hidden_states.shape
        q, k, v = self._qkv(hidden_states)
        q = OF.apply_rope(q, position_ids, self.rope_theta, self.rotary_dim, interleaved=True)
        k = OF.apply_rope(k, position_ids, self.rope_theta, self.rotary_dim, interleaved=True)
        k_all, v_all, present = update_kv(layer_past, k, v)
        out = OF.attention(q, k_all, v_all, causal=True, bias=attention_mask)
        return self.out_proj(out.reshape(b, s, -1)), (present if use_cache else None)


class CodeGenAttention(GPTJAttention):
    MP = 4

    def __init__(self, config: GPTJConfig):
        nn.Module.__init__(self)
        self.embed_dim = config.n_embd
        self.num_attention_heads = config.n_head
        self.head_dim = self.embed_dim // self.num_attention_heads
        self.rotary_dim, self.rope_theta = config.rotary_dim, config.rope_theta
        self.qkv_proj = Linear(self.embed_dim, 3 * self.embed_dim, bias=False)
        self.out_proj = Linear(self.embed_dim, self.embed_dim, bias=False)

    def _qkv(self, hidden_states):
        b, s, _ = hidden_states.shape
        fused = self.qkv_proj(hidden_states).view(b, s, self.MP, 3, -1, self.head_dim)
        q, v, k = fused[:, :, :, 0], fused[:, :, :, 1], fused[:, :, :, 2]
        return tuple(t.reshape(b, s, -1, self.head_dim) for t in (q, k, v))


class GPTJMLP(nn.Module):
    def __init__(self, config: GPTJConfig):
        super().__init__()
        self.fc_in = Linear(config.n_embd, config.n_inner)
        self.fc_out = Linear(config.n_inner, config.n_embd)

    def forward(self, x):
        return self.fc_out(OF.gelu(self.fc_in(x), approximate="tanh"))


class GPTJBlock(nn.Module):
    attention_class = GPTJAttention
    parallel_block = True  # attention and MLP read the same input; their partial outputs may share one all-reduce

    def __init__(self, config: GPTJConfig):
        super().__init__()
        self.ln_1 = LayerNorm(config.n_embd, eps=config.layer_norm_epsilon)
        self.attn = self.attention_class(config)
        self.mlp = GPTJMLP(config)

    def forward(self, hidden, layer_past=None, attention_mask=None, position_ids=None, use_cache=False):
        normed = self.ln_1(hidden)
        attn_out, present = self.attn(normed, layer_past=layer_past, attention_mask=attention_mask, position_ids=position_ids, use_cache=use_cache)
        partial = attn_out + self.mlp(normed)
        reduce = self.__dict__.get("_tp_block_reduce")
        return hidden + (partial if reduce is None else reduce(partial)), present


class CodeGenBlock(GPTJBlock):
    attention_class = CodeGenAttention


class GPTJModel(nn.Module):
    block_class = GPTJBlock

    def __init__(self, config: GPTJConfig):
        super().__init__()
        self.config = config  # lets the predefined rule table be found when the bare model (no head) is wrapped
        self.wte = nn.Embedding(config.vocab_size, config.n_embd)
        self.h = nn.ModuleList([self.block_class(config) for _ in range(config.n_layer)])
        self.ln_f = LayerNorm(config.n_embd, eps=config.layer_norm_epsilon)

    def forward(self, input_ids=None, past_key_values=None, attention_mask=None, position_ids=None, inputs_embeds=None, use_cache=False):
        hidden = self.wte(input_ids) if inputs_embeds is None else inputs_embeds
        b, s = hidden.shape[:2]
        offset = past_length(past_key_values)
        if position_ids is None:
            position_ids = torch.arange(offset, offset + s, device=hidden.device)[None].expand(b, s)
        presents = []
        for i, block in enumerate(self.h):
            hidden, present = block(hidden, None if past_key_values is None else past_key_values[i], attention_mask, position_ids, use_cache)
            presents.append(present)
        return self.ln_f(hidden), (tuple(presents) if use_cache else None)


class CodeGenModel(GPTJModel):
    block_class = CodeGenBlock


class GPTJForCausalLM(CausalLMBase):
    model_class = GPTJModel

    def __init__(self, config: GPTJConfig):
        super().__init__()
        self.config = config
        self.transformer = self.model_class(config)
        self.lm_head = Linear(config.n_embd, config.vocab_size, bias=True)
        init_weights_(self)

    def forward(self, input_ids=None, past_key_values=None, attention_mask=None, position_ids=None, inputs_embeds=None,
                labels=None, use_cache=False, **unused):
        hidden, presents = self.transformer(input_ids, past_key_values, attention_mask, position_ids, inputs_embeds, use_cache)
        logits, loss = self.head_and_loss(self.lm_head, hidden, labels)
        return ModelOutput(loss=loss, logits=logits, past_key_values=presents)


class CodeGenForCausalLM(GPTJForCausalLM):
    model_class = CodeGenModel
