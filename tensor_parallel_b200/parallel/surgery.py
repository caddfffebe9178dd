"""Model surgery: build the shard of a module that one rank owns.

A shard is a structural copy of the module whose parameters / buffers are the rank's slices
(state rules), whose per-rank attributes are patched (attr rules), and whose matched
sub-modules are replaced by :class:`TensorParallelWrapper` objects that run input actions
before and output actions after the wrapped forward.  Reference:
``src/tensor_parallel/shard.py:16-187`` and ``src/tensor_parallel/wrapper.py:17-75``.
"""
from __future__ import annotations

import copy
import logging
from typing import Collection, Dict, Optional, Sequence, Set, Tuple

import torch
from torch import nn

from tensor_parallel_b200.parallel.actions import StateAction
from tensor_parallel_b200.parallel.rules import Config, MappedActions, get_parameter_name_mapping

logger = logging.getLogger(__name__)


# ------------------------------------------------------------------------------------------
# wrapper
# ------------------------------------------------------------------------------------------


def apply_action(value, action, *, rank: int, world_size: int):
    """Interpret one module-rule action on ``value``."""
    if isinstance(action, tuple):
        action = action[0]
    if isinstance(action, StateAction):
        return action(value, rank)
    if callable(action):
        return action(value, rank=rank)
    kind, *opts = action.split()
    if kind == "split":
        return torch.tensor_split(value, world_size, dim=int(opts[0]))[rank]
    if kind == "scale":
        return value / world_size
    raise ValueError(f"unknown action {action!r}; expected 'split <dim>', 'scale', a collective or a callable")


def process_input(input_actions: MappedActions, rank: int, world_size: int, *args, **kwargs):
    """Apply actions keyed by positional index or keyword name.  A keyword the caller did not
    pass is still set to ``action(None)`` (rule tables rely on ``None`` passing through)."""
    merged = dict(kwargs)
    merged.update(enumerate(args))
    for key, action in input_actions.items():
        merged[key] = apply_action(merged.get(key), action, rank=rank, world_size=world_size)
    positional = [merged.pop(i) for i in range(len(args))]
    extra_positional = sorted(k for k in merged if isinstance(k, int))
    for k in extra_positional:  # an index rule beyond the passed positionals has no slot to fill
        merged.pop(k)
    return positional, merged


def process_output(output, output_actions: MappedActions, *, rank: int, world_size: int):
    """Apply actions to a tensor (key 0), a sequence (by index) or a mapping (by key)."""
    if isinstance(output, torch.Tensor):
        return process_output({0: output}, output_actions, rank=rank, world_size=world_size)[0]
    if isinstance(output, Sequence) and not isinstance(output, (str, bytes)):
        as_dict = process_output(dict(enumerate(output)), output_actions, rank=rank, world_size=world_size)
        items = [as_dict[i] for i in range(len(output))]
        if hasattr(type(output), "_fields"):
            return type(output)(*items)
        return type(output)(items)
    for key, action in output_actions.items():
        output[key] = apply_action(output.get(key), action, rank=rank, world_size=world_size)
    return output


class TensorParallelWrapper(nn.Module):
    """Holds the original sub-module as ``tp_wrapped_module`` (this name is part of the
    checkpoint key layout) and pipes its inputs / outputs through rule actions."""

    def __init__(self, module: nn.Module, input_actions: MappedActions, output_actions: MappedActions, *, rank: int, world_size: int):
        super().__init__()
        self.tp_wrapped_module = module
        self.__dict__["tp_wrapped_module"] = module  # reachable without going through __getattr__
        self.input_actions, self.output_actions = input_actions, output_actions
        self.rank, self.world_size = rank, world_size

    def forward(self, *args, **kwargs):
        args, kwargs = process_input(self.input_actions, self.rank, self.world_size, *args, **kwargs)
        output = self.tp_wrapped_module(*args, **kwargs)
        return process_output(output, self.output_actions, rank=self.rank, world_size=self.world_size)

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(self.__dict__["tp_wrapped_module"], name)


# ------------------------------------------------------------------------------------------
# shard construction
# ------------------------------------------------------------------------------------------


def find_matching_actions(kind: str, name: str, rules) -> MappedActions:
    """Union of the action maps of all patterns that match ``name``; conflicting actions raise."""
    merged: MappedActions = {}
    for pattern, mapped in rules.items():
        if pattern.search(name) is None:
            continue
        for key, action in mapped.items():
            if isinstance(key, str) and key.strip().isdigit():
                key = int(key)
            if key in merged and merged[key] != action:
                raise ValueError(f"conflicting {kind} rules for module '{name}', key {key!r}: {merged[key]} vs {action}")
            merged[key] = action
    return merged


def _placeholder_for(tensor: torch.Tensor, device: torch.device) -> torch.Tensor:
    target = tensor.device if tensor.device.type == "meta" else device
    empty = torch.empty(0, dtype=tensor.dtype, device=target)
    if isinstance(tensor, nn.Parameter):
        return nn.Parameter(empty, requires_grad=tensor.requires_grad)
    return empty


def _named_state(module: nn.Module):
    yield from module.named_parameters()
    yield from module.named_buffers()


def make_shard(module: nn.Module, device: torch.device, config: Config, *, rank: int, world_size: int) -> Tuple[nn.Module, Set[str]]:
    """Return ``(shard, names)`` where ``names`` are the shard-side names of all tensors that a
    state rule sliced (everything else is a replica and is a candidate for ZeRO-3 sharding)."""
    if not any(True for _ in module.children()):
        raise ValueError("tensor parallelism needs a container module (e.g. nn.Sequential), not a single layer")
    originals: Dict[str, torch.Tensor] = dict(_named_state(module))
    # deepcopy with a memo that maps every tensor to an empty placeholder: the module tree is
    # duplicated without touching (or allocating) any weight bytes; ties are kept because the
    # memo is keyed by tensor identity
    memo = {id(t): _placeholder_for(t, device) for t in originals.values()}
    shard = copy.deepcopy(module, memo=memo)
    del memo

    sliced_names = fill_state_(shard, originals, config, rank=rank)
    del originals

    replacements: Dict[nn.Module, nn.Module] = {}
    with torch.no_grad():
        for name, sub in shard.named_modules():
            if sub in replacements:
                continue
            attr_actions = find_matching_actions("attr", name, config.attr_rules)
            if attr_actions:
                patch_attrs_(sub, attr_actions, rank=rank)
            in_actions = find_matching_actions("input", name, config.input_rules)
            out_actions = find_matching_actions("output", name, config.output_rules)
            if in_actions or out_actions:
                replacements[sub] = TensorParallelWrapper(sub, in_actions, out_actions, rank=rank, world_size=world_size)

    for parent in list(shard.modules()):
        if isinstance(parent, TensorParallelWrapper):
            continue
        for child_name, child in list(parent.named_children()):
            if child in replacements:
                setattr(parent, child_name, replacements[child])

    fix_general_attributes(shard)
    shard = replacements.get(shard, shard)
    mapped = get_parameter_name_mapping(sliced_names, config)
    return shard, set(mapped.values())


@torch.no_grad()
def fill_state_(shard: nn.Module, originals: Dict[str, torch.Tensor], config: Config, *, rank: int) -> Set[str]:
    """Materialise every parameter / buffer of ``shard`` from the original tensors: the first
    matching state rule decides the slice, unmatched tensors are replicated."""
    sliced: Set[str] = set()
    unused = set(config.state_rules.keys())
    for name, holder in _named_state(shard):
        source = originals[name]
        for pattern, action in config.state_rules.items():
            if pattern.search(name) is not None:
                source = action(source, rank=rank)
                sliced.add(name)
                unused.discard(pattern)
                break
        # .clone() so that the shard owns compact storage rather than a view of the full tensor
        holder.data = source.detach().clone().to(holder.device)
    if unused and rank == 0:
        logger.warning("state_rules patterns that matched nothing: %s", sorted(p.pattern for p in unused))
    return sliced


def patch_attrs_(module: nn.Module, actions: MappedActions, *, rank: int):
    if module.__dict__.get("_tp_attrs_patched", False):
        raise RuntimeError("attribute rules were applied twice to the same module")
    for attr, action in actions.items():
        if not hasattr(module, attr):  # newer model revisions dropped some per-module size attributes
            logger.debug("attribute rule for '%s' skipped: %s has no such attribute", attr, type(module).__name__)
            continue
        setattr(module, attr, action(getattr(module, attr), rank=rank))
    module.__dict__["_tp_attrs_patched"] = True


@torch.no_grad()
def fix_general_attributes(shard: nn.Module):
    """Keep well-known size attributes consistent with sliced weights."""
    for sub in shard.modules():
        if isinstance(sub, nn.Linear):
            sub.out_features, sub.in_features = sub.weight.shape[0], sub.weight.shape[1]


def make_distributed_shard(module: nn.Module, device: torch.device, config: Optional[Config] = None, **kwargs):
    """One-process-per-rank entry (``torchrun``): returns a module, see
    :class:`tensor_parallel_b200.parallel.distributed.DistributedTensorParallel`."""
    from tensor_parallel_b200.parallel.distributed import DistributedTensorParallel

    return DistributedTensorParallel(module, device, tensor_parallel_config=config, **kwargs)
