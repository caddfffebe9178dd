"""NVTX ranges around the collectives, the fused GEMM + collective calls and the engine phases.

Off by default (zero overhead beyond one attribute test); ``TPB_NVTX=1`` in the environment, or
``enable(True)``, turns them on so that a timeline profiler shows which kernels belong to which logical step.
The reference has no tracing at all (it only logs its parameter-memory overhead,
``src/tensor_parallel/tensor_parallel.py:90-99``).
"""
from __future__ import annotations

import contextlib
import functools
import os

_enabled = bool(os.environ.get("TPB_NVTX"))
_depth = 0  # ranges currently open (lets tests see the nesting without a GPU)


def enable(on: bool = True) -> None:
    global _enabled
    _enabled = bool(on)


def enabled() -> bool:
    return _enabled


def _push(name: str) -> None:
    global _depth
    _depth += 1
    try:
        import torch

        if torch.cuda.is_available():
            torch.cuda.nvtx.range_push(name)
    except Exception:  # tracing must never break the traced call
        pass


def _pop() -> None:
    global _depth
    _depth -= 1
    try:
        import torch

        if torch.cuda.is_available():
            torch.cuda.nvtx.range_pop()
    except Exception:
        pass


@contextlib.contextmanager
def nvtx_range(name: str):
    if not _enabled:
        yield
        return
    _push(name)
    try:
        yield
    finally:
        _pop()


def traced(name: str):
    """Decorator form of :func:`nvtx_range`."""

    def wrap(fn):
        @functools.wraps(fn)
        def inner(*args, **kwargs):
            if not _enabled:
                return fn(*args, **kwargs)
            _push(name)
            try:
                return fn(*args, **kwargs)
            finally:
                _pop()

        return inner

    return wrap
