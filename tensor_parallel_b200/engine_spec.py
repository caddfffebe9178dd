"""Family-independent description of a decoder shard, read by the serving engine.

The engine does not care which class a shard is an instance of: an adapter below walks the module tree by
the parameter names that the rule tables of ``parallel/families`` key on (``self_attn.q_proj``,
``self_attention.query_key_value``, ``fc1`` ...), so the self-contained model zoo and the Hugging Face classes of
the same family are served alike.  What comes out is a :class:`DecoderSpec`: per layer the local (already
sharded) tensors in one canonical form - separate q / k / v row blocks, row-parallel output projections, an
MLP that is either gated or plain - plus the handful of scalars that select kernels (norm kind, rotary
layout, activation, sequential or parallel residual).

Adapters return ``None`` for a model they cannot describe exactly (an extra per-head norm, a scaled
embedding, ALiBi, a sliding window shorter than the cache ...); such models keep the generic module path.
Reference counterpart: none - the reference always runs the wrapped Hugging Face modules
(``src/tensor_parallel/pretrained_model.py:75-111``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

import torch


def unwrap(module):
    return module.__dict__.get("tp_wrapped_module", module) if hasattr(module, "__dict__") else module


def _get(module, *path):
    for name in path:
        module = unwrap(getattr(unwrap(module), name))
    return module


def _w(linear):
    return unwrap(linear).weight.detach()


def _b(linear):
    bias = getattr(unwrap(linear), "bias", None)
    return None if bias is None else bias.detach()


@dataclass
class LayerSpec:
    ln1_w: torch.Tensor                       # norm in front of the attention (weight; bias for LayerNorm)
    ln1_b: Optional[torch.Tensor]
    wq: torch.Tensor                          # [local q heads * head_dim, hidden]
    wk: torch.Tensor
    wv: torch.Tensor
    bq: Optional[torch.Tensor]
    bk: Optional[torch.Tensor]
    bv: Optional[torch.Tensor]
    wo: torch.Tensor                          # [hidden, local q heads * head_dim]  (row-parallel)
    bo: Optional[torch.Tensor]                # the shard's copy: bias / world
    ln2_w: Optional[torch.Tensor]             # norm in front of the MLP; None: a parallel block that shares ln1
    ln2_b: Optional[torch.Tensor]
    w_up: torch.Tensor                        # [local ffn, hidden]  (fc1 / dense_h_to_4h / up_proj)
    b_up: Optional[torch.Tensor]
    w_gate: Optional[torch.Tensor]            # gated MLPs only
    b_gate: Optional[torch.Tensor]
    w_down: torch.Tensor                      # [hidden, local ffn]  (row-parallel)
    b_down: Optional[torch.Tensor]            # bias / world


@dataclass
class DecoderSpec:
    family: str
    hidden: int
    head_dim: int
    norm: str                                 # "rms" | "layernorm"
    eps: float
    rotary_dim: int                           # 0: no rotary embedding
    rope_theta: float
    rope_interleaved: bool
    parallel_block: bool                      # attention and MLP both read the block input; one residual add
    act: str                                  # "silu" | "gelu" | "gelu_tanh" | "relu"
    vocab_size: int
    embed: torch.Tensor                       # local table: [vocab, hidden] or, hidden-split, [vocab, hidden / world]
    pos_embed: Optional[torch.Tensor]         # learned positions (local slice like ``embed``)
    pos_offset: int
    final_ln_w: torch.Tensor
    final_ln_b: Optional[torch.Tensor]
    head_w: torch.Tensor                      # vocab-split: [vocab / world, hidden]; hidden-split (tied): [vocab, hidden / world]
    head_split: str                           # "vocab" | "hidden"
    layers: List[LayerSpec] = field(default_factory=list)

    def parameters(self):
        """Every tensor the engine derives its own buffers from (used to notice that weights have changed)."""
        seen = [self.embed, self.pos_embed, self.final_ln_w, self.final_ln_b, self.head_w]
        for layer in self.layers:
            seen.extend(vars(layer).values())
        return [t for t in seen if isinstance(t, torch.Tensor)]


def _rope_theta(cfg) -> float:
    """Base of the rotary frequencies; raises for scaled / extrapolated variants (linear, NTK, YaRN, llama3 ...).
    Newer ``transformers`` keep everything in ``rope_parameters`` (``rope_scaling`` is then an alias of it)."""
    params = getattr(cfg, "rope_parameters", None) or getattr(cfg, "rope_scaling", None) or {}
    if isinstance(params, dict):
        kind = params.get("rope_type", params.get("type", "default"))
        if kind not in ("default", None):
            raise ValueError(f"scaled rotary embeddings ({kind})")
    theta = getattr(cfg, "rope_theta", None)
    if theta is None and isinstance(params, dict):
        theta = params.get("rope_theta")
    return float(10000.0 if theta is None else theta)


def _llama_like(lm, cfg, max_seq: int) -> Optional[DecoderSpec]:
    """Llama, Mistral, Qwen2 (self-contained or Hugging Face): RMSNorm, rotary, SwiGLU, sequential residual."""
    model_type = getattr(cfg, "model_type", "")
    if model_type not in ("llama", "mistral", "qwen2"):
        return None  # qwen3 normalises q / k per head, gemma scales the embedding and offsets the norm weight
    window = getattr(cfg, "sliding_window", None)
    if window is not None and window < max_seq and (model_type == "mistral" or getattr(cfg, "use_sliding_window", False)):
        return None
    if getattr(cfg, "hidden_act", "silu") != "silu":
        return None
    heads = cfg.num_attention_heads
    head_dim = getattr(cfg, "head_dim", None) or cfg.hidden_size // heads
    model = _get(lm, "model")
    embed = _get(model, "embed_tokens").weight.detach()
    head = _get(lm, "lm_head")
    head_w = _w(head)
    spec = DecoderSpec(
        family=model_type, hidden=cfg.hidden_size, head_dim=head_dim, norm="rms", eps=float(cfg.rms_norm_eps),
        rotary_dim=head_dim, rope_theta=_rope_theta(cfg), rope_interleaved=False, parallel_block=False, act="silu",
        vocab_size=cfg.vocab_size, embed=embed, pos_embed=None, pos_offset=0,
        final_ln_w=_get(model, "norm").weight.detach(), final_ln_b=None, head_w=head_w,
        head_split="vocab" if head_w.shape[1] == cfg.hidden_size else "hidden",
    )
    if _b(head) is not None:
        return None
    for layer in unwrap(model).layers:
        layer = unwrap(layer)
        attn, mlp = _get(layer, "self_attn"), _get(layer, "mlp")
        if hasattr(attn, "q_norm") or hasattr(attn, "k_norm"):
            return None
        spec.layers.append(LayerSpec(
            ln1_w=_get(layer, "input_layernorm").weight.detach(), ln1_b=None,
            wq=_w(attn.q_proj), wk=_w(attn.k_proj), wv=_w(attn.v_proj), bq=_b(attn.q_proj), bk=_b(attn.k_proj), bv=_b(attn.v_proj),
            wo=_w(attn.o_proj), bo=_b(attn.o_proj),
            ln2_w=_get(layer, "post_attention_layernorm").weight.detach(), ln2_b=None,
            w_up=_w(mlp.up_proj), b_up=_b(mlp.up_proj), w_gate=_w(mlp.gate_proj), b_gate=_b(mlp.gate_proj),
            w_down=_w(mlp.down_proj), b_down=_b(mlp.down_proj),
        ))
    return spec


def _opt(lm, cfg, max_seq: int) -> Optional[DecoderSpec]:
    """OPT: learned positions (offset 2), pre-LayerNorm, ReLU MLP on the layer itself, biases, tied head."""
    if not getattr(cfg, "do_layer_norm_before", True) or getattr(cfg, "word_embed_proj_dim", cfg.hidden_size) != cfg.hidden_size:
        return None  # opt-350m: post-norm and projected embeddings
    if getattr(cfg, "activation_function", "relu") != "relu":
        return None
    decoder = _get(lm, "model", "decoder")
    if getattr(decoder, "final_layer_norm", None) is None:
        return None
    if max_seq > cfg.max_position_embeddings:
        return None
    head_w = _w(_get(lm, "lm_head"))
    final_ln = unwrap(decoder.final_layer_norm)
    spec = DecoderSpec(
        family="opt", hidden=cfg.hidden_size, head_dim=cfg.hidden_size // cfg.num_attention_heads, norm="layernorm", eps=1e-5,
        rotary_dim=0, rope_theta=10000.0, rope_interleaved=False, parallel_block=False, act="relu", vocab_size=cfg.vocab_size,
        embed=_get(decoder, "embed_tokens").weight.detach(), pos_embed=_get(decoder, "embed_positions").weight.detach(), pos_offset=2,
        final_ln_w=final_ln.weight.detach(), final_ln_b=final_ln.bias.detach(), head_w=head_w,
        head_split="vocab" if head_w.shape[1] == cfg.hidden_size else "hidden",
    )
    for layer in unwrap(decoder).layers:
        layer = unwrap(layer)
        attn = _get(layer, "self_attn")
        ln1, ln2 = unwrap(layer.self_attn_layer_norm), unwrap(layer.final_layer_norm)
        spec.layers.append(LayerSpec(
            ln1_w=ln1.weight.detach(), ln1_b=ln1.bias.detach(),
            wq=_w(attn.q_proj), wk=_w(attn.k_proj), wv=_w(attn.v_proj), bq=_b(attn.q_proj), bk=_b(attn.k_proj), bv=_b(attn.v_proj),
            wo=_w(attn.out_proj), bo=_b(attn.out_proj),
            ln2_w=ln2.weight.detach(), ln2_b=ln2.bias.detach(),
            w_up=_w(layer.fc1), b_up=_b(layer.fc1), w_gate=None, b_gate=None, w_down=_w(layer.fc2), b_down=_b(layer.fc2),
        ))
    return spec


def _falcon(lm, cfg, max_seq: int) -> Optional[DecoderSpec]:
    """Falcon / RefinedWeb: parallel attention + MLP block, fused query_key_value, rotary, GeLU, tied head.  Covers the
    grouped layout ``[group][q heads | k | v]`` (40B, "new decoder architecture") and the multi-query layout of the
    7B model (all query heads, then one shared key and value head)."""
    if getattr(cfg, "alibi", False) or getattr(cfg, "bias", False):
        return None
    heads = getattr(cfg, "n_head", None) or cfg.num_attention_heads
    head_dim = cfg.hidden_size // heads
    new_arch = getattr(cfg, "new_decoder_architecture", hasattr(cfg, "n_head_kv"))
    multi_query = bool(getattr(cfg, "multi_query", False)) and not new_arch
    if not new_arch and not getattr(cfg, "parallel_attn", True):
        return None  # sequential falcon-rw variants
    if not new_arch and not multi_query:
        return None  # per-head [q | k | v] triples of the oldest layout
    num_kv = 1 if multi_query else (getattr(cfg, "n_head_kv", None) or getattr(cfg, "num_kv_heads", None) or heads)
    q_per_kv = heads // num_kv
    transformer = _get(lm, "transformer")
    head_w = _w(_get(lm, "lm_head"))
    ln_f = unwrap(transformer.ln_f)
    spec = DecoderSpec(
        family="falcon", hidden=cfg.hidden_size, head_dim=head_dim, norm="layernorm",
        eps=float(getattr(cfg, "layer_norm_epsilon", 1e-5)), rotary_dim=head_dim, rope_theta=_rope_theta(cfg),
        rope_interleaved=False, parallel_block=True, act="gelu", vocab_size=cfg.vocab_size,
        embed=_get(transformer, "word_embeddings").weight.detach(), pos_embed=None, pos_offset=0,
        final_ln_w=ln_f.weight.detach(), final_ln_b=ln_f.bias.detach(), head_w=head_w,
        head_split="vocab" if head_w.shape[1] == cfg.hidden_size else "hidden",
    )
    for layer in unwrap(transformer).h:
        layer = unwrap(layer)
        attn, mlp = _get(layer, "self_attention"), _get(layer, "mlp")
        fused = _w(attn.query_key_value)
        if multi_query:  # [local q heads | k | v]
            q_rows = fused.shape[0] - 2 * head_dim
            wq, wk, wv = fused[:q_rows], fused[q_rows : q_rows + head_dim], fused[q_rows + head_dim :]
        else:            # [local groups][q_per_kv | k | v]
            groups = fused.shape[0] // ((q_per_kv + 2) * head_dim)
            g = fused.view(groups, q_per_kv + 2, head_dim, fused.shape[1])
            wq = g[:, :q_per_kv].reshape(groups * q_per_kv * head_dim, -1)
            wk, wv = g[:, q_per_kv].reshape(groups * head_dim, -1), g[:, q_per_kv + 1].reshape(groups * head_dim, -1)
        if hasattr(layer, "ln_attn"):
            ln1, ln2 = unwrap(layer.ln_attn), unwrap(layer.ln_mlp)
        else:
            ln1, ln2 = unwrap(layer.input_layernorm), None
        spec.layers.append(LayerSpec(
            ln1_w=ln1.weight.detach(), ln1_b=ln1.bias.detach(), wq=wq, wk=wk, wv=wv, bq=None, bk=None, bv=None,
            wo=_w(attn.dense), bo=None,
            ln2_w=None if ln2 is None else ln2.weight.detach(), ln2_b=None if ln2 is None else ln2.bias.detach(),
            w_up=_w(mlp.dense_h_to_4h), b_up=None, w_gate=None, b_gate=None, w_down=_w(mlp.dense_4h_to_h), b_down=None,
        ))
    return spec


ADAPTERS: Dict[str, Callable] = {
    "llama": _llama_like, "mistral": _llama_like, "qwen2": _llama_like,
    "opt": _opt,
    "falcon": _falcon, "RefinedWeb": _falcon, "RefinedWebModel": _falcon,
}


def describe(shard, max_seq: int = 0) -> Optional[DecoderSpec]:
    """The :class:`DecoderSpec` of a causal-LM shard, or ``None`` when no adapter describes it exactly."""
    lm = unwrap(shard)
    cfg = getattr(lm, "config", None)
    adapter = ADAPTERS.get(getattr(cfg, "model_type", None))
    if adapter is None or not hasattr(lm, "lm_head"):
        return None
    try:
        spec = adapter(lm, cfg, max_seq)
    except (AttributeError, ValueError, KeyError, TypeError):
        return None
    if spec is None or not spec.layers:
        return None
    tensors = spec.parameters()
    if any(t.device.type != "cuda" or t.dtype != torch.bfloat16 for t in tensors):
        return None
    if spec.head_dim not in (64, 128) or spec.hidden % 8:
        return None
    return spec
