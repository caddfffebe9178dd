"""Weight-slicing actions: how one tensor of the original model becomes one tensor per rank.

Every action is a callable ``action(tensor, rank) -> slice`` with an inverse
``undo(list_of_slices) -> tensor`` used when a model is saved "as if never split".
Semantics follow ``torch.tensor_split`` (the first ``n % world`` ranks get one extra unit,
trailing ranks may get zero-size slices).  Reference: ``src/tensor_parallel/state_actions.py:10-119``.
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Callable, List, Optional, Sequence

import torch
from torch import Tensor


def unit_bounds(num_units: int, world_size: int, rank: int):
    """[start, stop) of the units owned by ``rank`` under tensor_split partitioning."""
    base, extra = divmod(num_units, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


class StateAction(ABC):
    """Base class of all state (parameter / buffer) rules."""

    @abstractmethod
    def __call__(self, tensor: Tensor, rank: int) -> Tensor:
        ...

    @abstractmethod
    def undo(self, tensors: Sequence[Tensor]) -> Tensor:
        ...


class LegacyStateAction(StateAction):
    """Adapter for the deprecated rule forms: a bare callable or a ``(split, merge)`` pair."""

    def __init__(self, action: Callable[[Tensor, int], Tensor], reverse_action: Optional[Callable] = None):
        self.action, self.reverse_action = action, reverse_action

    def __call__(self, tensor: Tensor, rank: int) -> Tensor:
        return self.action(tensor, rank)

    def undo(self, tensors: Sequence[Tensor]) -> Tensor:
        if self.reverse_action is None:
            raise RuntimeError(f"state rule {self.action} was given without an inverse; cannot merge shards")
        return self.reverse_action(tensors)


class Split(StateAction):
    """Even-as-possible split of dimension ``dim`` (column- or row-parallel weights)."""

    def __init__(self, world_size: int, dim: int):
        self.world_size, self.dim = world_size, dim

    def __call__(self, tensor: Tensor, rank: int) -> Tensor:
        start, stop = unit_bounds(tensor.shape[self.dim], self.world_size, rank)
        return tensor.narrow(self.dim, start, stop - start)

    def undo(self, tensors: Sequence[Tensor]) -> Tensor:
        return torch.cat([t.detach().cpu() for t in tensors], dim=self.dim)

    def __repr__(self):
        return f"{type(self).__name__}(world_size={self.world_size}, dim={self.dim})"


class Scale(StateAction):
    """Divide by the world size, so that an all-reduce over ranks restores the value
    (bias of a row-parallel layer)."""

    def __init__(self, world_size: int):
        self.world_size = world_size

    def __call__(self, tensor: Tensor, rank: int) -> Tensor:
        return tensor / self.world_size

    def undo(self, tensors: Sequence[Tensor]) -> Tensor:
        return tensors[0] * self.world_size

    def __repr__(self):
        return f"Scale(world_size={self.world_size})"


class SplitInChunks(Split):
    """Split ``dim`` in whole blocks of ``chunk_size`` (attention heads, fused QKV triples, GQA groups)."""

    def __init__(self, world_size: int, dim: int, chunk_size: int, optional: bool = False):
        super().__init__(world_size, dim)
        self.chunk_size, self.optional = chunk_size, optional

    def __call__(self, tensor: Optional[Tensor], rank: int) -> Optional[Tensor]:
        if tensor is None and self.optional:
            return None
        extent = tensor.shape[self.dim]
        if extent % self.chunk_size:
            raise ValueError(f"dim {self.dim} of shape {tuple(tensor.shape)} is not a multiple of {self.chunk_size}")
        start, stop = unit_bounds(extent // self.chunk_size, self.world_size, rank)
        return tensor.narrow(self.dim, start * self.chunk_size, (stop - start) * self.chunk_size)

    def __repr__(self):
        return f"SplitInChunks(world_size={self.world_size}, dim={self.dim}, chunk_size={self.chunk_size})"


class SplitInGroupedChunks(Split):
    """``dim`` holds ``num_groups`` equal groups (e.g. Q|K|V); take the same chunk range out of each."""

    def __init__(self, world_size: int, dim: int, num_groups: int, chunk_size: int):
        super().__init__(world_size, dim)
        self.num_groups, self.chunk_size = num_groups, chunk_size

    def _grouped(self, tensor: Tensor) -> Tensor:
        dim = self.dim % tensor.ndim
        return tensor.unflatten(dim, (self.num_groups, tensor.shape[dim] // self.num_groups)), dim

    def __call__(self, tensor: Tensor, rank: int) -> Tensor:
        grouped, dim = self._grouped(tensor)
        start, stop = unit_bounds(grouped.shape[dim + 1] // self.chunk_size, self.world_size, rank)
        part = grouped.narrow(dim + 1, start * self.chunk_size, (stop - start) * self.chunk_size)
        return part.flatten(dim, dim + 1)

    def undo(self, tensors: Sequence[Tensor]) -> Tensor:
        pieces: List[Tensor] = []
        dim = None
        for t in tensors:
            grouped, dim = self._grouped(t.detach().cpu())
            pieces.append(grouped)
        return torch.cat(pieces, dim=dim + 1).flatten(dim, dim + 1)

    def __repr__(self):
        return (
            f"SplitInGroupedChunks(world_size={self.world_size}, dim={self.dim}, "
            f"num_groups={self.num_groups}, chunk_size={self.chunk_size})"
        )


def as_state_action(rule) -> StateAction:
    """Accept the modern and both legacy spellings of a state rule (reference:
    ``src/tensor_parallel/config.py:68-83``)."""
    import logging

    if isinstance(rule, StateAction):
        return rule
    log = logging.getLogger(__name__)
    if callable(rule):
        log.warning("callables in state_rules are deprecated; derive from StateAction instead")
        return LegacyStateAction(rule)
    if isinstance(rule, tuple) and len(rule) == 2 and all(callable(f) for f in rule):
        log.warning("(split, merge) tuples in state_rules are deprecated; derive from StateAction instead")
        return LegacyStateAction(*rule)
    raise TypeError(f"cannot interpret {rule!r} (type {type(rule).__name__}) as a state rule")
