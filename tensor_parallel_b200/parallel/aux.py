"""Helper actions used by the predefined model rule tables (heads, KV cache, ALiBi).

Reference: ``src/tensor_parallel/aux_actions.py:7-47``.
"""
from __future__ import annotations

import torch

from tensor_parallel_b200.parallel.actions import unit_bounds
from tensor_parallel_b200.parallel.kv import PerDeviceTensors
from tensor_parallel_b200.utils.nested import nested_map


def _is_cache_object(obj) -> bool:
    return hasattr(obj, "update") and hasattr(obj, "get_seq_length")


def gather_kv(*per_rank_kv, world_size: int):
    """Zip every rank's ``(key, value)`` into ``(PerDeviceTensors(keys), PerDeviceTensors(values))``.

    No data moves: the result only holds references, and the same object is handed to every rank.
    """
    if per_rank_kv[0] is None:
        return per_rank_kv
    if isinstance(per_rank_kv[0], torch.Tensor) or _is_cache_object(per_rank_kv[0]):
        # not a (key, value) pair: newer attention modules keep their cache in a stateful object (handled by the
        # runtime) and return something else at this position, e.g. T5's per-rank position bias - leave it alone
        return per_rank_kv
    zipped = tuple(PerDeviceTensors(*same_slot) for same_slot in zip(*per_rank_kv))
    return [zipped] * world_size


def select_kv_for_rank(kv_state, rank: int):
    """Replace every ``PerDeviceTensors`` leaf by this rank's element."""
    return nested_map(lambda leaf: leaf[rank] if isinstance(leaf, PerDeviceTensors) else leaf, kv_state)


def split_num_heads(num_heads: int, *, rank: int, world_size: int) -> int:
    """Heads owned by ``rank``; never 0 (a rank without heads keeps one dummy head of zero weights)."""
    start, stop = unit_bounds(num_heads, world_size, rank)
    return max(stop - start, 1)


def split_inner_dim(inner_dim: int, *, rank: int, num_heads: int, world_size: int) -> int:
    return split_num_heads(num_heads, rank=rank, world_size=world_size) * (inner_dim // num_heads)


def split_heads(tensor, *, dim: int, head_dim: int, rank: int, world_size: int, optional: bool = False):
    """Slice ``dim`` in whole heads; a rank left without heads gets zeros of one head's width."""
    if tensor is None and optional:
        return None
    dim = dim % tensor.ndim
    if tensor.shape[dim] % head_dim:
        raise ValueError(f"dim {dim} of {tuple(tensor.shape)} is not a multiple of head_dim={head_dim}")
    start, stop = unit_bounds(tensor.shape[dim] // head_dim, world_size, rank)
    if stop == start:
        shape = list(tensor.shape)
        shape[dim] = head_dim
        return torch.zeros(shape, dtype=tensor.dtype, device=tensor.device)
    return tensor.narrow(dim, start * head_dim, (stop - start) * head_dim)


def split_alibi(alibi: torch.Tensor, *, rank: int, num_heads: int, world_size: int) -> torch.Tensor:
    """ALiBi bias laid out ``[batch * num_heads, ...]``: keep this rank's heads of every batch item."""
    per_head = alibi.reshape(-1, num_heads, *alibi.shape[1:])
    start, stop = unit_bounds(num_heads, world_size, rank)
    return per_head[:, start:stop].reshape(-1, *alibi.shape[1:])
