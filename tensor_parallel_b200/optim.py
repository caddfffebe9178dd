"""Fused AdamW for tensor-parallel models.

``tp.optim.AdamW(model.parameters(), ...)`` updates every TP slice and every ZeRO-3 flat shard with one
hand-written kernel per tensor (parameter, gradient, both moments and an optional fp32 master copy are
read and written exactly once).  CPU tensors and unsupported dtypes fall back to the same update written
with stock PyTorch operators.  The reference ships no optimizer; its notebook uses a user-supplied one
(``examples/training_flan-t5-xl.ipynb:184``).
"""
from __future__ import annotations

from typing import Iterable

import torch


class AdamW(torch.optim.Optimizer):
    def __init__(self, params: Iterable, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 1e-2,
                 master_weights: bool = True):
        """``master_weights``: keep an fp32 copy of bf16 parameters so that small updates are not lost to rounding."""
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, master_weights=master_weights)
        super().__init__(params, defaults)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            beta1, beta2 = group["betas"]
            for p in group["params"]:
                if p.grad is None or p.numel() == 0:
                    continue
                state = self.state[p]
                if not state:
                    state["step"] = 0
                    state["exp_avg"] = torch.zeros(p.shape, dtype=torch.float32, device=p.device)
                    state["exp_avg_sq"] = torch.zeros(p.shape, dtype=torch.float32, device=p.device)
                    if group["master_weights"] and p.dtype != torch.float32:
                        state["master"] = p.detach().float().clone()
                state["step"] += 1
                grad = p.grad
                native_ok = p.is_cuda and p.dtype in (torch.bfloat16, torch.float32) and grad.dtype in (torch.bfloat16, torch.float32) \
                    and p.is_contiguous() and grad.is_contiguous()
                if native_ok:
                    from tensor_parallel_b200.ops import native

                    with torch.cuda.device(p.device):
                        native.adamw_step(p, grad, state["exp_avg"], state["exp_avg_sq"], state["step"], group["lr"], beta1, beta2,
                                          group["eps"], group["weight_decay"], master=state.get("master"))
                    # the kernel wrote through data_ptr: bump the version counter (no kernel) so that ZeRO-3 re-gathers
                    # and a serving engine built from these weights notices
                    torch.autograd.graph.increment_version(p)
                    continue
                g = grad.float()
                m, v = state["exp_avg"], state["exp_avg_sq"]
                m.mul_(beta1).add_(g, alpha=1 - beta1)
                v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
                target = state.get("master", p if p.dtype == torch.float32 else p.float())
                target.mul_(1 - group["lr"] * group["weight_decay"])
                bc1, bc2 = 1 - beta1 ** state["step"], 1 - beta2 ** state["step"]
                target.addcdiv_(m / bc1, (v / bc2).sqrt_().add_(group["eps"]), value=-group["lr"])
                if target is not p:
                    p.copy_(target)
        return loss
