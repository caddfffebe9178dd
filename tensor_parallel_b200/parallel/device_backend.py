"""Selection of the device-side collective backend (symmetric heap + hand-written kernels).

Returns ``None`` whenever the native library or peer access is unavailable or the user set
``TENSOR_PARALLEL_USE_NATIVE``; callers then use the portable thread / process-group
collectives.
"""
from __future__ import annotations

import logging
import os
from typing import Optional, Sequence

import torch

logger = logging.getLogger(__name__)


def maybe_thread_backend(devices: Sequence[torch.device]):
    if os.environ.get("TENSOR_PARALLEL_USE_NATIVE"):
        return None
    try:
        from tensor_parallel_b200.ops import comm
    except Exception as exc:  # library not built
        logger.debug("device collectives unavailable: %r", exc)
        return None
    return comm.thread_backend(devices)


def maybe_process_backend(device: torch.device, process_group=None):
    if os.environ.get("TENSOR_PARALLEL_USE_NATIVE") or device.type != "cuda":
        return None
    try:
        from tensor_parallel_b200.ops import comm
    except Exception as exc:
        logger.debug("device collectives unavailable: %r", exc)
        return None
    return comm.process_backend(device, process_group)
