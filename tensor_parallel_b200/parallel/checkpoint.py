"""Checkpoint helpers: save "as if never split", convert plain state dicts to the sharded
key layout, and derive a per-tensor device map.

Sharded key layout (``[wrapped_model.]`` only for the Hugging Face wrapper)::

    [wrapped_model.]module_shards.{rank}.{path with tp_wrapped_module. after every wrapped module}.{tensor}
    [wrapped_model.]_sanity_check_params.{rank}
    [wrapped_model.]sharding_manager.flat_shards.{rank}

Reference: ``src/tensor_parallel/dispatch.py:13-131``.
"""
from __future__ import annotations

import re
from contextlib import contextmanager
from typing import Dict, Mapping, Optional

import torch

from tensor_parallel_b200.parallel.rules import Config, get_parameter_name_mapping
from tensor_parallel_b200.utils.tied import find_tied_weight_aliases


@contextmanager
def save_tensor_parallel(model):
    """Inside this context ``model.state_dict()`` (and ``save_pretrained``) produce the original,
    world-size independent layout that loads into the unsplit model."""
    model.set_preserve_shards_when_saving(False)
    try:
        yield
    finally:
        model.set_preserve_shards_when_saving(True)


_RANK_IN_KEY = re.compile(r"(?:_sanity_check_params|module_shards|flat_shards)\.(\d+)(?:\.|$)")


def infer_sharded_data_device_id(name: str) -> int:
    hit = _RANK_IN_KEY.search(name)
    if hit is None:
        raise KeyError(f"'{name}' is not a tensor-parallel state key: cannot tell which rank owns it")
    return int(hit.group(1))


def infer_sharded_device_map(tp_model) -> Dict[str, torch.device]:
    """Name (and every tied alias) of each parameter / buffer -> device of the owning rank."""
    by_id = {}
    for name, tensor in list(tp_model.named_parameters()) + list(tp_model.named_buffers()):
        by_id[id(tensor)] = tp_model.devices[infer_sharded_data_device_id(name)]
    device_map = {}
    for tensor_id, aliases in find_tied_weight_aliases(tp_model).items():
        for alias in aliases:
            device_map[alias] = by_id[tensor_id]
    return device_map


def convert_state_dict_single_shard(state: Mapping, config: Config, world_size: int, rank: int) -> dict:
    names = get_parameter_name_mapping(state.keys(), config)
    out = {}
    for name, tensor in state.items():
        for pattern, action in config.state_rules.items():
            if pattern.search(name) is not None:
                tensor = action(tensor, rank=rank)
                break
        out[f"module_shards.{rank}.{names[name]}"] = tensor
    return out


def convert_state_dict(input_state_dict: Mapping, tensor_parallel_config: Config, world_size: int, for_pretrained: bool = False,
                       sharded_param_names=None) -> dict:
    """Plain (possibly partial) state dict -> sharded key layout for ``world_size`` ranks.

    Works chunk by chunk, which is what makes memory-efficient loading possible.  Tied weights
    present under several names are sliced under each name.

    ``sharded_param_names`` (the ``sharded_param_names`` of a model wrapped with ``sharded=True``, i.e. shard-side names
    in the order of its flat shards, or the output of :func:`replicated_parameter_names`) additionally produces the
    ZeRO-3 ``sharding_manager.flat_shards.{rank}`` entries and drops those parameters (and their tied aliases) from
    the per-rank entries, so that the result loads straight into a model created with ``sharded=True``.  The whole set
    of those parameters must then be present in ``input_state_dict`` (a flat shard cannot be assembled from a chunk).
    The reference cannot emit flat shards (``src/tensor_parallel/dispatch.py:79``)."""
    out = {}
    for rank in range(world_size):
        out.update(convert_state_dict_single_shard(input_state_dict, tensor_parallel_config, world_size, rank))
        out[f"_sanity_check_params.{rank}"] = torch.empty(0)
    if sharded_param_names:
        from tensor_parallel_b200.parallel.actions import unit_bounds

        shard_side = get_parameter_name_mapping(input_state_dict.keys(), tensor_parallel_config)
        original_of = {v: k for k, v in shard_side.items()}
        missing = [n for n in sharded_param_names if n not in original_of]
        if missing:
            raise KeyError(f"parameters of the flat shards are not in this state dict: {missing[:5]}")
        tensors = [input_state_dict[original_of[n]] for n in sharded_param_names]
        pieces_per_rank = [[t.detach().flatten()[slice(*unit_bounds(t.numel(), world_size, r))] for t in tensors] for r in range(world_size)]
        flat_len = max(sum(p.numel() for p in pieces) for pieces in pieces_per_rank)
        for r, pieces in enumerate(pieces_per_rank):
            pad = flat_len - sum(p.numel() for p in pieces)
            out[f"sharding_manager.flat_shards.{r}"] = torch.cat(pieces + [tensors[0].new_zeros(pad)])
        # the sharded parameters (under every name that aliases them) no longer live in the shard modules
        aliased = {id_: names for id_, names in _aliases_by_storage(input_state_dict).items()}
        drop = set()
        for n in sharded_param_names:
            for alias in aliased.get(_storage_key(input_state_dict[original_of[n]]), [original_of[n]]):
                drop.add(shard_side[alias])
        out = {k: v for k, v in out.items() if not any(k == f"module_shards.{r}.{d}" for r in range(world_size) for d in drop)}
    if for_pretrained:
        out = {"wrapped_model." + key: value for key, value in out.items()}
    return out


def _storage_key(t: torch.Tensor):
    return (t.data_ptr(), tuple(t.shape), tuple(t.stride())) if t.numel() else ("empty", id(t))


def _aliases_by_storage(state: Mapping):
    groups: Dict[tuple, list] = {}
    for name, t in state.items():
        groups.setdefault(_storage_key(t), []).append(name)
    return groups


def replicated_parameter_names(module, tensor_parallel_config: Config):
    """Shard-side names, sorted, of the parameters of ``module`` that no state rule splits - the ones ZeRO-3 puts into
    flat shards; what ``sharded=True`` computes on its own, for use with :func:`convert_state_dict`."""
    names = [n for n, _ in module.named_parameters()]
    mapping = get_parameter_name_mapping(names, tensor_parallel_config)
    return sorted(mapping[n] for n in names if not any(p.search(n) for p in tensor_parallel_config.state_rules))


def load_sharded_state_dict_(tp_model, state: Mapping, strict: bool = True):
    """Meta-aware loader: assign each tensor of a sharded-layout state dict to its slot on the
    owning rank's device (replaces ``accelerate.set_module_tensor_to_device`` loops)."""
    device_map = infer_sharded_device_map(tp_model)
    slots = {}
    for module_name, sub in tp_model.named_modules():
        for store in (sub._parameters, sub._buffers):
            for local, t in store.items():
                if t is not None:
                    slots[(module_name + "." if module_name else "") + local] = (sub, store, local)
    missing = [k for k in slots if k not in state]
    unexpected = [k for k in state if k not in slots]
    if strict and (unexpected or [k for k in missing if "_sanity_check" not in k]):
        raise KeyError(f"missing keys {missing[:5]}..., unexpected keys {unexpected[:5]}...")
    replaced = {}  # id(old tensor) -> new tensor, so that tied slots keep sharing one tensor
    with torch.no_grad():
        for key, value in state.items():
            if key not in slots:
                continue
            sub, store, local = slots[key]
            old = store[local]
            if id(old) in replaced:
                continue
            new = value.to(device_map[key])
            if isinstance(old, torch.nn.Parameter):
                new = torch.nn.Parameter(new, requires_grad=old.requires_grad)
            replaced[id(old)] = new
        for sub, store, local in slots.values():
            old = store[local]
            if id(old) in replaced:
                store[local] = replaced[id(old)]
    return missing, unexpected
