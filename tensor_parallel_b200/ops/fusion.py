"""Fusion planner: rewrites rule-matched sites of freshly built shards to fused native operators.

The rule tables stay the source of truth for what is split; this module only changes how a matched
pattern executes on CUDA bf16 shards.  Module names, wrapper placement and state-dict keys are untouched.

Sites recognised today:

* **row-parallel linear + ``"sum"``** (attention ``o_proj`` / ``dense`` / ``out_proj`` / ``c_proj``, MLP
  ``down_proj`` / ``fc2`` / ``dense_4h_to_h`` / ``wo``): the wrapper whose output rule sums entry 0 contains exactly
  one ``nn.Linear`` whose weight was split along its input dim.  That linear gets a fused forward - GEMM with the
  all-reduce in its epilogue for decode-sized inputs, GEMM into symmetric memory + device all-reduce otherwise -
  and the wrapper's own ``"sum"`` on entry 0 is dropped.
* **vocab-parallel lm_head + loss**: a head whose weight was split along the vocabulary gets the distributed
  cross-entropy of ``tensor_parallel_b200.ops.loss`` when ``config.fused_lm_loss`` is set on the model.
"""
from __future__ import annotations

import logging
from typing import Optional

import torch
from torch import nn

from tensor_parallel_b200.parallel.actions import Split, unit_bounds
from tensor_parallel_b200.parallel.surgery import TensorParallelWrapper

logger = logging.getLogger(__name__)


class _RowParallelFn(torch.autograd.Function):
    """out = all-reduce(x @ W^T) + world * bias_local   (bias_local holds bias / world)."""

    @staticmethod
    def forward(ctx, x, weight, bias, comm):
        from tensor_parallel_b200.ops import native

        x2d = x.reshape(-1, x.shape[-1])
        tokens, features = x2d.shape[0], weight.shape[0]
        if tokens <= 64 and comm.fits_fused(tokens, features, weight.shape[1]):
            out = comm.gemm_allreduce(x2d, weight, bias=bias, bias_scale=float(comm.world))
        else:
            if tokens * features <= comm._capacity(torch.bfloat16, 1, 1):  # the GEMM writes straight into symmetric memory
                staged = comm.staging_view("in", (tokens, features), torch.bfloat16)
                native.gemm_nt(x2d, weight, out=staged)
                out = comm.all_reduce(staged).clone()
            else:
                out = comm.all_reduce(native.gemm_nt(x2d, weight))
            if bias is not None:
                out += bias * comm.world
        ctx.save_for_backward(x2d, weight)
        ctx.comm, ctx.has_bias, ctx.shape = comm, bias is not None, x.shape
        return out.view(*x.shape[:-1], features)

    @staticmethod
    def backward(ctx, grad):
        from tensor_parallel_b200.ops import native

        x2d, weight = ctx.saved_tensors
        g = grad.reshape(-1, grad.shape[-1]).to(torch.bfloat16).contiguous()
        g = ctx.comm.all_reduce(g).clone()  # adjoint of the forward all-reduce
        gx = native.linear_dgrad(g, weight).view(ctx.shape) if ctx.needs_input_grad[0] else None
        gw = native.linear_wgrad(g, x2d) if ctx.needs_input_grad[1] else None
        gb = g.float().sum(0).to(grad.dtype) if ctx.has_bias and ctx.needs_input_grad[2] else None
        return gx, gw, gb, None


def _fused_row_parallel_forward(linear: nn.Linear, comm, process_group=None):
    plain_forward = linear.forward

    def forward(x):
        ok = x.is_cuda and x.dtype == torch.bfloat16 and linear.weight.dtype == torch.bfloat16 and linear.weight.shape[1] % 8 == 0
        if not ok:
            return comm_sum(plain_forward(x))
        return _RowParallelFn.apply(x, linear.weight, linear.bias, comm)

    from tensor_parallel_b200.ops.comm import DeviceAllReduce
    from tensor_parallel_b200.parallel.collectives import DistributedAllReduce

    comm_sum = DeviceAllReduce(comm, DistributedAllReduce(comm.world, process_group))
    return forward


def _fused_row_parallel_forward_threaded(linear: nn.Linear, comm, rule_sum, rank: int):
    """Single-process mode (one shard per GPU, one host thread per rank).  Without gradients the linear runs the fused
    GEMM + all-reduce kernel on this rank's symmetric heap - the rank threads never meet on the host.  With gradients it
    keeps the rule's own ``"sum"`` (whose autograd node spans all devices, as one backward pass has to)."""
    plain_forward = linear.forward

    def forward(x):
        fused = (not (torch.is_grad_enabled() and (x.requires_grad or linear.weight.requires_grad)) and x.is_cuda
                 and x.dtype == torch.bfloat16 and linear.weight.dtype == torch.bfloat16 and linear.weight.shape[1] % 8 == 0)
        if not fused:
            return rule_sum(plain_forward(x), rank)
        from tensor_parallel_b200.ops import native

        x2d = x.reshape(-1, x.shape[-1])
        tokens, features = x2d.shape[0], linear.weight.shape[0]
        comm.poll_status()
        with torch.cuda.device(comm.device):
            if tokens <= 64 and comm.fits_fused(tokens, features, linear.weight.shape[1]):
                out = comm.gemm_allreduce(x2d, linear.weight, bias=linear.bias, bias_scale=float(comm.world))
            else:
                if tokens * features <= comm._capacity(torch.bfloat16, 1, 1):
                    staged = comm.staging_view("in", (tokens, features), torch.bfloat16)
                    native.gemm_nt(x2d, linear.weight, out=staged)
                    out = comm.all_reduce(staged).clone()
                else:
                    out = comm.all_reduce(native.gemm_nt(x2d, linear.weight))
                if linear.bias is not None:
                    out += linear.bias * comm.world
        return out.view(*x.shape[:-1], features)

    return forward


def _row_parallel_linears(wrapped: nn.Module, prefix: str, config) -> list:
    found = []
    for name, sub in wrapped.named_modules():
        if not isinstance(sub, nn.Linear) or isinstance(sub, TensorParallelWrapper):
            continue
        full = f"{prefix}.{name}.weight" if name else f"{prefix}.weight"
        for pattern, action in config.state_rules.items():
            if pattern.search(full) is not None:
                if isinstance(action, Split) and action.dim in (1, -1):
                    found.append(sub)
                break
    return found


def _rewrite_threaded(tp_module, comms, config) -> int:
    """Row-parallel linear + ``"sum"`` sites of every shard of a single-process model (see
    :func:`_fused_row_parallel_forward_threaded`).  Returns the number of sites per shard."""
    from tensor_parallel_b200.ops.comm import ThreadDeviceAllReduce

    from tensor_parallel_b200.ops import native

    per_shard = []
    for rank, (shard, comm) in enumerate(zip(tp_module.module_shards, comms)):
        with torch.cuda.device(comm.device):  # every kernel the rank threads may launch concurrently is loaded up front
            native.check(native.LIB.tpb_gemm_preload(), "tpb_gemm_preload")
            native.check(native.LIB.tpb_comm_preload(), "tpb_comm_preload")
        sites = 0
        original_names = {}
        for name, sub in shard.named_modules():
            original_names[id(sub)] = name.replace("tp_wrapped_module.", "").replace(".tp_wrapped_module", "")
        for name, sub in list(shard.named_modules()):
            if not isinstance(sub, TensorParallelWrapper):
                continue
            action = sub.output_actions.get(0)
            if not isinstance(action, ThreadDeviceAllReduce):
                continue
            inner = sub.__dict__["tp_wrapped_module"]
            linears = _row_parallel_linears(inner, original_names[id(inner)], config)
            if len(linears) != 1 or getattr(linears[0], "_tp_fused_row_parallel", False):
                continue
            linears[0].forward = _fused_row_parallel_forward_threaded(linears[0], comm, action, rank)
            linears[0]._tp_fused_row_parallel = True
            sub.output_actions = {k: v for k, v in sub.output_actions.items() if k != 0}
            sites += 1
        per_shard.append(sites)
    if per_shard and per_shard[0]:
        logger.info("fusion planner rewrote %d site(s) per shard (single-process mode)", per_shard[0])
    return per_shard[0] if per_shard else 0


def rewrite(tp_module) -> int:
    """Apply the plan to ``tp_module`` (a ``DistributedTensorParallel``); returns the number of rewritten sites."""
    backend = getattr(tp_module, "_device_backend", None)
    comm = getattr(backend, "comm", None)
    config = getattr(tp_module, "_live_config", None)
    comms = getattr(backend, "comms", None)
    if config is not None and comms is not None and len(comms) == len(tp_module.module_shards) > 1:
        return _rewrite_threaded(tp_module, comms, config)
    if comm is None or config is None or len(tp_module.module_shards) != 1:
        return 0
    from tensor_parallel_b200.ops.comm import DeviceAllReduce

    shard = tp_module.module_shards[0]
    sites = 0
    original_names = {}
    for name, sub in shard.named_modules():
        original_names[id(sub)] = name.replace("tp_wrapped_module.", "").replace(".tp_wrapped_module", "")
    for name, sub in list(shard.named_modules()):
        if not isinstance(sub, TensorParallelWrapper):
            continue
        action = sub.output_actions.get(0)
        if not isinstance(action, DeviceAllReduce):
            continue
        inner = sub.__dict__["tp_wrapped_module"]
        prefix = original_names[id(inner)]
        linears = _row_parallel_linears(inner, prefix, config)
        if len(linears) != 1:
            continue
        linear = linears[0]
        if getattr(linear, "_tp_fused_row_parallel", False):
            continue
        linear.forward = _fused_row_parallel_forward(linear, comm, getattr(tp_module, "process_group", None))
        linear._tp_fused_row_parallel = True
        sub.output_actions = {k: v for k, v in sub.output_actions.items() if k != 0}
        sites += 1

    # vocab-parallel head + distributed cross-entropy
    root = shard.__dict__.get("tp_wrapped_module", shard)
    for head_name in ("lm_head", "embed_out"):
        head = getattr(root, head_name, None)
        if head is None:
            continue
        inner = head.__dict__.get("tp_wrapped_module", head) if isinstance(head, TensorParallelWrapper) else head
        if not isinstance(inner, nn.Linear) or inner.bias is not None:
            continue
        for pattern, action in config.state_rules.items():
            if pattern.search(f"{head_name}.weight") is not None:
                if type(action) is Split and action.dim == 0:
                    full_vocab = getattr(root.config, "vocab_size", None)
                    if full_vocab is None:
                        break
                    start, _ = unit_bounds(full_vocab, tp_module.world_size, tp_module.rank)
                    root.__dict__["_tp_vocab_parallel"] = dict(
                        vocab_start=start,
                        gather_stats=lambda stats, c=comm: c.all_gather(stats).clone(),
                        reduce_hidden_grad=lambda gx, c=comm: c.all_reduce(gx.contiguous()).clone(),
                    )
                    sites += 1
                break
    if sites:
        logger.info("fusion planner rewrote %d site(s)", sites)
    return sites
