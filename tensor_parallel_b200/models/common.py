"""Shared pieces of the self-contained model zoo.

The models reproduce the module tree, parameter names and per-module attributes of the Hugging
Face classes of the era the reference's rule tables target (``src/tensor_parallel/slicing_configs.py``),
so the predefined tables apply unchanged and state dicts are key-compatible — independent of
whichever ``transformers`` version happens to be installed.  Compute goes through
``tensor_parallel_b200.ops.functional`` (hand-written kernels on B200, PyTorch elsewhere).
"""
from __future__ import annotations

from typing import Any, Optional, Tuple

import torch
from torch import nn

from tensor_parallel_b200.ops import functional as OF


class ShapedConfig:
    """Minimal stand-in for ``transformers.PretrainedConfig``: attribute bag with ``model_type``."""

    model_type = "generic"

    def __init__(self, **kwargs):
        for key, value in kwargs.items():
            setattr(self, key, value)

    def to_dict(self):
        return {"model_type": self.model_type, **{k: v for k, v in vars(self).items()}}

    def __repr__(self):
        return f"{type(self).__name__}({self.to_dict()})"


class ModelOutput(dict):
    """Dict with attribute access (``out.loss``, ``out.logits``, ``out.past_key_values``) and
    integer indexing over the non-``None`` values, like Hugging Face model outputs."""

    def __getattr__(self, name):
        try:
            return self[name]
        except KeyError:
            raise AttributeError(name) from None

    def __getitem__(self, key):
        if isinstance(key, int):
            return [v for v in self.values() if v is not None][key]
        return super().__getitem__(key)


class Linear(nn.Linear):
    """``nn.Linear`` whose forward runs the tcgen05 GEMM on B200."""

    def forward(self, x):
        return OF.linear(x, self.weight, self.bias)


class Conv1D(nn.Module):
    """GPT-2 style linear layer storing ``weight[in, out]`` and its width as ``nf``."""

    def __init__(self, nf: int, nx: int):
        super().__init__()
        self.nf = nf
        self.weight = nn.Parameter(torch.empty(nx, nf))
        self.bias = nn.Parameter(torch.zeros(nf))
        nn.init.normal_(self.weight, std=0.02)

    def forward(self, x):
        out = torch.addmm(self.bias, x.reshape(-1, x.shape[-1]), self.weight)
        return out.view(*x.shape[:-1], self.weight.shape[1])


class RMSNorm(nn.Module):
    def __init__(self, hidden: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden))
        self.variance_epsilon = eps

    def forward(self, x):
        return OF.rms_norm(x, self.weight, self.variance_epsilon)


class LayerNorm(nn.LayerNorm):
    def forward(self, x):
        return OF.layer_norm(x, self.weight, self.bias, self.eps)


def update_kv(past: Optional[Tuple[torch.Tensor, torch.Tensor]], k: torch.Tensor, v: torch.Tensor):
    """Append ``k, v`` (``[B, S, H, D]``) to a cache kept as ``(K, V)`` of shape ``[B, H, S_total, D]``
    and return ``(K_bshd, V_bshd, present)``."""
    k_cache, v_cache = k.transpose(1, 2), v.transpose(1, 2)
    if past is not None:
        if hasattr(past, "append"):  # pre-allocated static cache (decode fast path)
            return past.append(k, v)
        k_cache = torch.cat((past[0], k_cache), dim=2)
        v_cache = torch.cat((past[1], v_cache), dim=2)
    return k_cache.transpose(1, 2), v_cache.transpose(1, 2), (k_cache, v_cache)


def past_length(past) -> int:
    if past is None:
        return 0
    first = past[0] if not hasattr(past, "length") else past
    if hasattr(first, "length"):
        return first.length
    return first[0].shape[2] if isinstance(first, (tuple, list)) else first.shape[2]


def init_weights_(module: nn.Module, std: float = 0.02, seed: Optional[int] = None):
    """N(0, std) for matrices / embeddings, zeros for biases, ones for norm scales.  Parameters are
    filled in place on whatever device they live on (a 7B model initialises on the GPU in seconds);
    with ``seed`` the values are drawn on the CPU from a private generator instead."""
    gen = torch.Generator().manual_seed(seed) if seed is not None else None
    for name, p in module.named_parameters():
        if p.device.type == "meta":
            continue
        with torch.no_grad():
            if p.ndim >= 2:
                if gen is None:
                    p.normal_(0.0, std)
                else:
                    p.copy_(torch.randn(p.shape, generator=gen, dtype=torch.float32).mul_(std).to(p.dtype))
            elif name.endswith("bias"):
                p.zero_()


class CausalLMBase(nn.Module):
    """Loss handling and generation shared by the decoder-only models."""

    def lm_loss(self, logits: torch.Tensor, labels: Optional[torch.Tensor]):
        if labels is None:
            return None
        return OF.cross_entropy(logits[:, :-1], labels[:, 1:].to(logits.device))

    def head_and_loss(self, head: nn.Module, hidden: torch.Tensor, labels: Optional[torch.Tensor]):
        """``(logits, loss)``.  With ``config.fused_lm_loss`` and labels on a CUDA bf16 model the head GEMM is
        fused with a (vocab-parallel) cross-entropy and full logits are never formed: ``logits`` is then None."""
        inner = head.__dict__.get("tp_wrapped_module", head)
        fused = (
            labels is not None and getattr(self.config, "fused_lm_loss", False) and hidden.is_cuda
            and hidden.dtype == torch.bfloat16 and isinstance(inner, nn.Linear) and inner.bias is None
            and (inner.weight.shape[0] == self.config.vocab_size or "_tp_vocab_parallel" in self.__dict__)
        )
        if fused:
            from tensor_parallel_b200.ops.loss import lm_head_cross_entropy

            extra = self.__dict__.get("_tp_vocab_parallel", {})
            loss = lm_head_cross_entropy(hidden[:, :-1], inner.weight, labels[:, 1:], **extra)
            return None, loss
        logits = head(hidden)
        return logits, self.lm_loss(logits, labels)

    def generate(self, input_ids=None, **kwargs):
        from tensor_parallel_b200.models.generation import generate

        return generate(self, input_ids, **kwargs)

    @staticmethod
    def _reorder_cache(past, beam_idx):
        return tuple(tuple(t.index_select(0, beam_idx.to(t.device)) for t in layer) for layer in past)
