"""Vocab-parallel lm_head fused with a distributed cross-entropy.

The reference gathers (or all-reduces) full ``[tokens, vocab]`` logits onto every rank and computes the
loss redundantly (``src/tensor_parallel/slicing_configs.py:381,390``).  Here every rank
multiplies the hidden states with its vocabulary slice of the head on the tcgen05 GEMM, reduces each row
of its local logits to four numbers (max, sum-exp, target logit, ownership flag), exchanges only those
``[tokens, 4]`` floats, and turns the local logits in place into their gradient.  Every rank returns its own share
``dlogits_local @ W_local`` of ``grad(hidden)`` (the shares are summed by the adjoint of whichever collective
produced the replicated hidden state), ``grad(W_local)`` stays local.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from tensor_parallel_b200.ops import native
from tensor_parallel_b200.ops.native import LIB, c_float, c_int, c_ll, c_void_p, check

LIB.tpb_ce_stats.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_ll, c_int, c_int, c_void_p]
LIB.tpb_ce_grad.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_ll, c_int, c_int, c_void_p, c_void_p]


class _VocabParallelCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, labels, vocab_start, gather_stats, reduce_hidden_grad, ignore_index):
        x2d = hidden.reshape(-1, hidden.shape[-1])
        if not x2d.is_contiguous():
            x2d = x2d.contiguous()
        labels = labels.reshape(-1).to(device=x2d.device, dtype=torch.int64).contiguous()
        rows, cols = x2d.shape[0], weight.shape[0]
        logits = native.gemm_nt(x2d, weight)  # [rows, local vocab] bf16
        stats = torch.empty(rows, 4, dtype=torch.float32, device=x2d.device)
        check(LIB.tpb_ce_stats(logits.data_ptr(), labels.data_ptr(), stats.data_ptr(), rows, cols, logits.stride(0), vocab_start,
                               ignore_index, native._stream()), "tpb_ce_stats")
        native.launch_count += 1
        everyone = gather_stats(stats) if gather_stats is not None else stats[None]  # [world, rows, 4]
        gmax = everyone[..., 0].max(dim=0).values
        sumexp = (everyone[..., 1] * torch.exp(everyone[..., 0] - gmax)).sum(dim=0)
        lse = gmax + torch.log(sumexp)
        target = everyone[..., 2].sum(dim=0)
        valid = labels != ignore_index
        n_valid = valid.sum().clamp(min=1)
        loss = ((lse - target) * valid).sum() / n_valid
        ctx.save_for_backward(x2d, weight, labels, logits, lse, n_valid)
        ctx.meta = (vocab_start, reduce_hidden_grad, ignore_index, hidden.shape)
        return loss

    @staticmethod
    def backward(ctx, grad_loss):
        x2d, weight, labels, logits, lse, n_valid = ctx.saved_tensors
        vocab_start, reduce_hidden_grad, ignore_index, hidden_shape = ctx.meta
        rows, cols = logits.shape
        if reduce_hidden_grad is not None:
            # the loss value is replicated on every rank; its cotangent is the sum over all copies (ranks whose
            # output does not seed the backward pass contribute zero)
            grad_loss = reduce_hidden_grad(grad_loss.float().reshape(1))
        scale = (grad_loss.float() / n_valid).reshape(1).contiguous()
        check(LIB.tpb_ce_grad(logits.data_ptr(), labels.data_ptr(), lse.data_ptr(), rows, cols, logits.stride(0), vocab_start,
                              ignore_index, scale.data_ptr(), native._stream()), "tpb_ce_grad")
        native.launch_count += 1
        dlogits = logits  # overwritten in place
        gx = gw = None
        if ctx.needs_input_grad[0]:
            # this rank's share of d loss / d hidden (through its vocabulary slice).  It is NOT summed over ranks
            # here: the replicated hidden state receives partial cotangents on every rank, and the adjoint of the
            # collective that produced it (the previous row-parallel all-reduce, the embedding gather) adds them up.
            gx = native.linear_dgrad(dlogits, weight).view(hidden_shape)
        if ctx.needs_input_grad[1]:
            gw = native.linear_wgrad(dlogits, x2d)
        return gx, gw, None, None, None, None, None


def lm_head_cross_entropy(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, vocab_start: int = 0,
                          gather_stats: Optional[Callable] = None, reduce_hidden_grad: Optional[Callable] = None,
                          ignore_index: int = -100) -> torch.Tensor:
    """Mean cross-entropy of ``softmax(hidden @ W_full^T)`` against ``labels`` where this rank only owns
    ``weight = W_full[vocab_start : vocab_start + weight.shape[0]]``.

    ``gather_stats([rows, 4]) -> [world, rows, 4]`` and ``reduce_hidden_grad(x) -> sum over ranks`` (applied to the
    scalar loss cotangent only) are the two collectives (``None`` on a single rank).  Requires CUDA bf16 tensors."""
    return _VocabParallelCE.apply(hidden, weight, labels, vocab_start, gather_stats, reduce_hidden_grad, ignore_index)


def lm_head_cross_entropy_ref(hidden, weight_full, labels, ignore_index: int = -100):
    logits = hidden.float().reshape(-1, hidden.shape[-1]) @ weight_full.float().t()
    return torch.nn.functional.cross_entropy(logits, labels.reshape(-1), ignore_index=ignore_index)
