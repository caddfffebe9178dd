"""Fusion planner: rewrites rule-matched sites of freshly built shards without changing what the rule
tables mean.  Module names, wrapper placement and therefore checkpoint keys are untouched.

Two passes:

* :func:`merge_parallel_block_reductions` (pure Python, every mode): blocks that compute attention and MLP
  from the same input and add both to the residual (Falcon, GPT-J, CodeGen, GPT-NeoX with parallel residual)
  carry two ``"sum"`` rules (reference: ``src/tensor_parallel/slicing_configs.py:450-451``).  Both partial outputs
  are added locally first and reduced once, halving the collectives of such layers.
* ``tensor_parallel_b200.ops.fusion.rewrite`` (CUDA, one process per GPU): row-parallel linear + ``"sum"`` becomes
  one GEMM + all-reduce kernel; a vocabulary-split head gets the distributed cross-entropy.
"""
from __future__ import annotations

import logging

from tensor_parallel_b200.parallel import collectives as C
from tensor_parallel_b200.parallel.surgery import TensorParallelWrapper

logger = logging.getLogger(__name__)


def _is_all_reduce(action) -> bool:
    if isinstance(action, (C.ThreadAllReduce, C.DistributedAllReduce)):
        return True
    return type(action).__name__ in ("DeviceAllReduce", "ThreadDeviceAllReduce")


def merge_parallel_block_reductions(tp_module) -> int:
    """Layers that declare ``parallel_block = True`` and hold exactly two wrapped children whose entry-0 output
    rule is an all-reduce get one reduction of the summed partial outputs instead."""
    merged = 0
    ranks = getattr(tp_module, "local_ranks", range(len(tp_module.module_shards)))
    for shard, rank in zip(tp_module.module_shards, ranks):
        for layer in shard.modules():
            if not getattr(layer, "parallel_block", False) or isinstance(layer, TensorParallelWrapper):
                continue
            summed = [child for child in layer.children()
                      if isinstance(child, TensorParallelWrapper) and _is_all_reduce(child.output_actions.get(0))]
            if len(summed) != 2 or summed[0].output_actions[0] is not summed[1].output_actions[0]:
                continue
            op = summed[0].output_actions[0]
            for child in summed:
                child.output_actions = {k: v for k, v in child.output_actions.items() if k != 0}
            layer.__dict__["_tp_block_reduce"] = (lambda x, op=op, rank=rank: op(x, rank))
            merged += 1
    return merged


def apply_fusion_plan(tp_module) -> int:
    """Returns how many sites were rewritten."""
    sites = merge_parallel_block_reductions(tp_module)
    try:
        from tensor_parallel_b200.ops import fusion
    except Exception as exc:  # native library absent (CPU-only machine)
        logger.debug("native fusion pass inactive: %r", exc)
        return sites
    return sites + fusion.rewrite(tp_module)
