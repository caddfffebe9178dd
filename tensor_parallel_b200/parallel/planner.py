"""Fusion planner: swap rule-matched sub-graphs for fused native operators.

The rule tables stay the source of truth for *what* is split; the planner only changes *how*
a matched pattern executes on B200, e.g. a row-parallel ``nn.Linear`` whose wrapper output
rule is ``"sum"`` becomes one GEMM+all-reduce kernel over peer memory.  Module names, wrapper
placement and therefore checkpoint keys are untouched.  Populated by
``tensor_parallel_b200.ops``; a no-op when the native library is absent.
"""
from __future__ import annotations

import logging

logger = logging.getLogger(__name__)


def apply_fusion_plan(tp_module) -> int:
    """Returns how many sites were rewritten."""
    try:
        from tensor_parallel_b200.ops import fusion
    except Exception as exc:
        logger.debug("fusion planner inactive: %r", exc)
        return 0
    return fusion.rewrite(tp_module)
