"""Operator front-end used by the self-contained models.

Every operator has a plain PyTorch definition (the numerical reference, and the CPU path) and,
for CUDA tensors, a hand-written sm_100a kernel from ``tensor_parallel_b200.ops.native``.
Dispatch rule: CUDA bf16/fp16/fp32 tensors go to the native kernel when the shape is
supported; if the native library cannot be loaded on a CUDA machine the call raises, unless
``TENSOR_PARALLEL_USE_NATIVE`` asks for stock PyTorch operators.
"""
from __future__ import annotations

import math
import os
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

_FORCE_TORCH = bool(os.environ.get("TENSOR_PARALLEL_USE_NATIVE"))


def _native(x: torch.Tensor):
    """The native module if ``x`` should run on hand-written kernels, else ``None``."""
    if not x.is_cuda or _FORCE_TORCH:
        return None
    from tensor_parallel_b200.ops import native  # raises if the library is missing on a GPU box

    return native


# -- reference definitions ---------------------------------------------------------------------


def rms_norm_ref(x, weight, eps: float):
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (y * weight.float()).to(x.dtype) if weight is not None else y.to(x.dtype)


def layer_norm_ref(x, weight, bias, eps: float):
    return F.layer_norm(x.float(), x.shape[-1:], None if weight is None else weight.float(), None if bias is None else bias.float(), eps).to(x.dtype)


def rope_tables(positions: torch.Tensor, rotary_dim: int, theta: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos / sin of shape ``[..., rotary_dim/2]`` in fp32 for integer ``positions``."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, device=positions.device, dtype=torch.float32) / rotary_dim))
    angles = positions.to(torch.float32)[..., None] * inv_freq
    return angles.cos(), angles.sin()


def apply_rope_ref(x, positions, theta: float, rotary_dim: Optional[int] = None, interleaved: bool = False):
    """Rotary embedding on ``x[B, S, H, D]`` with ``positions[B, S]``.  ``interleaved`` pairs
    ``(2i, 2i+1)`` (GPT-J / CodeGen); otherwise ``(i, i + rotary_dim/2)`` (Llama / NeoX / Falcon)."""
    d = x.shape[-1]
    rotary_dim = d if rotary_dim is None else rotary_dim
    cos, sin = rope_tables(positions, rotary_dim, theta)
    cos, sin = cos[:, :, None, :], sin[:, :, None, :]
    rot, keep = x[..., :rotary_dim].float(), x[..., rotary_dim:]
    if interleaved:
        a, b = rot[..., 0::2], rot[..., 1::2]
        out = torch.stack((a * cos - b * sin, b * cos + a * sin), dim=-1).flatten(-2)
    else:
        a, b = rot[..., : rotary_dim // 2], rot[..., rotary_dim // 2 :]
        out = torch.cat((a * cos - b * sin, b * cos + a * sin), dim=-1)
    return torch.cat((out.to(x.dtype), keep), dim=-1)


def attention_ref(q, k, v, causal: bool, bias=None, scale: Optional[float] = None):
    """``q[B,Sq,Hq,D]``, ``k/v[B,Sk,Hkv,D]`` -> ``[B,Sq,Hq,D]``.  With ``causal`` query *i* sees keys
    ``<= i + (Sk - Sq)`` (so a cached decode step sees the whole cache).  ``bias`` is added to the
    scores and broadcasts against ``[B,Hq,Sq,Sk]``.  Softmax in fp32."""
    b, sq, hq, d = q.shape
    sk, hkv = k.shape[1], k.shape[2]
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3)
    vf = v.float().permute(0, 2, 1, 3)
    if hkv != hq:
        kf = kf.repeat_interleave(hq // hkv, dim=1)
        vf = vf.repeat_interleave(hq // hkv, dim=1)
    scores = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if bias is not None:
        scores = scores + bias.float()
    if causal:
        i = torch.arange(sq, device=q.device)[:, None] + (sk - sq)
        j = torch.arange(sk, device=q.device)[None, :]
        scores = scores.masked_fill(j > i, float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    return torch.matmul(probs, vf).permute(0, 2, 1, 3).to(q.dtype)


def gelu_ref(x, approximate: str = "none"):
    return F.gelu(x, approximate=approximate)


def swiglu_ref(gate, up):
    return F.silu(gate) * up


def geglu_ref(gate, up, approximate: str = "tanh"):
    return F.gelu(gate, approximate=approximate) * up


# -- dispatching front-end ---------------------------------------------------------------------


def linear(x, weight, bias=None):
    nat = _native(x)
    if nat is not None and nat.gemm_supported(x, weight):
        return nat.linear(x, weight, bias)
    return F.linear(x, weight, bias)


def rms_norm(x, weight, eps: float = 1e-6):
    nat = _native(x)
    if nat is not None and nat.norm_supported(x):
        return nat.rms_norm(x, weight, eps)
    return rms_norm_ref(x, weight, eps)


def layer_norm(x, weight, bias, eps: float = 1e-5):
    nat = _native(x)
    if nat is not None and nat.norm_supported(x):
        return nat.layer_norm(x, weight, bias, eps)
    return layer_norm_ref(x, weight, bias, eps)


def apply_rope(x, positions, theta: float = 10000.0, rotary_dim: Optional[int] = None, interleaved: bool = False):
    nat = _native(x)
    if nat is not None and nat.rope_supported(x):
        return nat.rope(x, positions, theta, rotary_dim, interleaved)
    return apply_rope_ref(x, positions, theta, rotary_dim, interleaved)


def attention(q, k, v, causal: bool, bias=None, scale: Optional[float] = None):
    nat = _native(q)
    if nat is not None and nat.attention_supported(q, k, v, bias):
        return nat.attention(q, k, v, causal, bias, scale)
    return attention_ref(q, k, v, causal, bias, scale)


def gelu(x, approximate: str = "none"):
    nat = _native(x)
    if nat is not None and nat.elementwise_supported(x):
        return nat.gelu(x, approximate)
    return gelu_ref(x, approximate)


def relu(x):
    nat = _native(x)
    if nat is not None and nat.elementwise_supported(x):
        return nat.relu(x)
    return F.relu(x)


def swiglu(gate, up):
    nat = _native(gate)
    if nat is not None and nat.elementwise_supported(gate):
        return nat.swiglu(gate, up)
    return swiglu_ref(gate, up)


def geglu(gate, up, approximate: str = "tanh"):
    nat = _native(gate)
    if nat is not None and nat.elementwise_supported(gate):
        return nat.geglu(gate, up, approximate)
    return geglu_ref(gate, up, approximate)


def cross_entropy(logits, labels, ignore_index: int = -100):
    return F.cross_entropy(logits.float().reshape(-1, logits.shape[-1]), labels.reshape(-1), ignore_index=ignore_index)
