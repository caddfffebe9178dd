"""The declarative slicing config: four regex-keyed rule tables.

* ``state_rules``  : parameter / buffer name pattern -> :class:`StateAction`
* ``input_rules``  : module name pattern -> {positional index | kwarg name: action}
* ``output_rules`` : module name pattern -> {output index | key: action}
* ``attr_rules``   : module name pattern -> {attribute name: callable(value, rank=...)}

Patterns are matched with ``re.search`` (unanchored unless the pattern anchors itself).
Module-rule actions are the strings ``"split <dim>"``, ``"scale"``, ``"sum"``,
``"gather <dim>"``, ``"gather_kv"`` or any callable ``(value, rank=...) -> value``.
Reference: ``src/tensor_parallel/config.py:26-191``.
"""
from __future__ import annotations

import copy
import os
import re
from itertools import chain
from typing import Any, Callable, Dict, Iterable, Mapping, Optional, Sequence, Union

import torch
from torch import nn

from tensor_parallel_b200.parallel import collectives as C
from tensor_parallel_b200.parallel.actions import Split, StateAction, as_state_action
from tensor_parallel_b200.utils.tied import check_lora

Arg = Union[int, str]
Action = Callable[[Any, int], Any]
MappedActions = Dict[Arg, Action]

#: any non-empty value disables device-side / NCCL collectives and CUDA-stream fan-out
TENSOR_PARALLEL_USE_NATIVE = bool(os.environ.get("TENSOR_PARALLEL_USE_NATIVE"))

WRAPPED_PREFIX = "tp_wrapped_module."


def _compile_table(table: Mapping) -> Dict[re.Pattern, Any]:
    return {(key if isinstance(key, re.Pattern) else re.compile(key)): value for key, value in table.items()}


class Config:
    """Container of the four rule tables; keys are compiled to ``re.Pattern`` on construction."""

    def __init__(self, state_rules: Mapping, input_rules: Mapping, output_rules: Mapping, attr_rules: Mapping):
        self.state_rules = {p: as_state_action(a) for p, a in _compile_table(state_rules).items()}
        self.input_rules = _compile_table(input_rules)
        self.output_rules = _compile_table(output_rules)
        self.attr_rules = _compile_table(attr_rules)
        #: failure domain of the live collectives; set by :meth:`create_collective_ops`
        self.rank_group: Optional[C.RankGroup] = None
        self.op_factory = None

    def replace(self, **tables) -> "Config":
        clone = copy.copy(self)
        for name, table in tables.items():
            setattr(clone, name, table)
        return clone

    def create_collective_ops(
        self, devices: Sequence[torch.device], distributed: bool = True, *, process_group=None, backend=None
    ) -> "Config":
        """Copy of this config whose ``"sum"`` / ``"gather d"`` / ``"gather_kv"`` strings are live
        collective objects.  One object is shared by all rules that spell the action the same way."""
        world_size = len(devices)
        use_pg = bool(distributed and torch.distributed.is_available() and torch.distributed.is_initialized())
        group = C.RankGroup(world_size)
        factory = _OpFactory(world_size, devices, use_pg, process_group, group, backend)
        clone = self.replace(
            input_rules=factory.instantiate(self.input_rules), output_rules=factory.instantiate(self.output_rules)
        )
        clone.rank_group = group
        clone.op_factory = factory  # lets the fusion planner create further collectives in the same failure domain
        return clone

    def __repr__(self):
        return (
            f"Config(state_rules={len(self.state_rules)}, input_rules={len(self.input_rules)}, "
            f"output_rules={len(self.output_rules)}, attr_rules={len(self.attr_rules)})"
        )


class _OpFactory:
    def __init__(self, world_size, devices, use_pg, process_group, group, backend):
        self.world_size, self.devices, self.use_pg, self.pg, self.group = world_size, devices, use_pg, process_group, group
        self.backend = backend
        self._cache: Dict[str, Any] = {}

    def make(self, spec: str):
        """Live collective for an action string (cached per spelling)."""
        if spec not in self._cache:
            self._cache[spec] = self._make(spec)
        return self._cache[spec]

    def _make(self, spec: str):
        kind, *opts = spec.split()
        if kind == "sum":
            if self.backend is not None:
                return self.backend.all_reduce_op(self.group)
            return C.DistributedAllReduce(self.world_size, self.pg) if self.use_pg else C.ThreadAllReduce(self.group)
        if kind == "gather":
            dim = int(opts[0]) if opts else -1
            if self.backend is not None:
                return self.backend.all_gather_op(self.group, dim)
            if self.use_pg:
                return C.DistributedAllGather(self.world_size, dim, self.pg)
            return C.ThreadAllGather(self.group, dim)
        if kind == "gather_kv":
            return C.LocalGatherKV() if self.use_pg else C.ThreadGatherKV(self.group)
        return None  # "split d" / "scale" are interpreted at call time by the wrapper

    def instantiate(self, rules: Mapping) -> Dict[re.Pattern, MappedActions]:
        out = {}
        for pattern, mapped in rules.items():
            fresh = {}
            for key, action in mapped.items():
                if isinstance(action, str):
                    if action not in self._cache:
                        self._cache[action] = self._make(action)
                    fresh[key] = self._cache[action] if self._cache[action] is not None else action
                elif isinstance(action, C.CollectiveOperation):
                    ident = f"__op_{id(action)}"
                    if ident not in self._cache:
                        self._cache[ident] = C.LocalGatherKV() if self.use_pg else action.rebind(self.group)
                    fresh[key] = self._cache[ident]
                else:
                    fresh[key] = action
            out[pattern] = fresh
        return out


def add_lora_rules(model: nn.Module, config: Config) -> Config:
    """Extend ``config`` for LoRA-wrapped linears: a column-parallel base splits ``lora_B`` the
    same way; a row-parallel base feeds ``lora_A`` the gathered input and scales its output
    by 1/world so that the base layer's all-reduce restores it.  Reference:
    ``src/tensor_parallel/config.py:128-154``."""
    extra_state, extra_in, extra_out = {}, {}, {}
    for name, module in model.named_modules():
        if not check_lora(module):
            continue
        for pattern, action in config.state_rules.items():
            if pattern.search(name + ".weight") is None:
                continue
            if not isinstance(action, Split):
                raise ValueError(f"LoRA layer {name}: base weight rule {action!r} is not a Split; unsupported")
            escaped = re.escape(name)
            if action.dim == 0:
                extra_state[re.compile(rf"^{escaped}\.lora_B\.")] = action
            elif action.dim == 1:
                extra_in[re.compile(rf"^{escaped}\.lora_A\.[^.]+$")] = {0: "gather -1"}
                extra_out[re.compile(rf"^{escaped}\.lora_A\.[^.]+$")] = {0: "scale"}
            else:
                raise ValueError(f"LoRA layer {name}: cannot handle a base weight split along dim {action.dim}")
            break
    if not (extra_state or extra_in or extra_out):
        return config
    return config.replace(
        state_rules={**extra_state, **config.state_rules},
        input_rules={**config.input_rules, **extra_in},
        output_rules={**config.output_rules, **extra_out},
    )


def get_parameter_name_mapping(names: Iterable[str], config: Config) -> Dict[str, str]:
    """Original dotted name -> name inside a shard, where ``tp_wrapped_module.`` follows every
    path component whose module is matched by an input or output rule (such modules are
    replaced by a wrapper that holds the original as ``tp_wrapped_module``)."""
    names = list(names)
    patterns = list(chain(config.input_rules.keys(), config.output_rules.keys()))
    mapping = {}
    module_hit: Dict[str, bool] = {}
    root_wrapped = any(p.search("") is not None for p in patterns)
    for name in names:
        parts = name.split(".")
        rebuilt = [WRAPPED_PREFIX[:-1]] if root_wrapped else []
        for depth in range(len(parts)):
            rebuilt.append(parts[depth])
            if depth == len(parts) - 1:
                break  # the last component is the tensor itself
            module_name = ".".join(parts[: depth + 1])
            hit = module_hit.get(module_name)
            if hit is None:
                hit = module_hit[module_name] = any(p.search(module_name) is not None for p in patterns)
            if hit:
                rebuilt.append(WRAPPED_PREFIX[:-1])
        mapping[name] = ".".join(rebuilt)
    return mapping
