"""ZeRO-3 style sharding of the parameters that tensor parallelism left replicated.

Every such parameter is flattened and cut into ``world`` pieces (``tensor_split`` rule); rank
*r* keeps piece *r* of every parameter, concatenated in a fixed order and zero-padded to a
common length, as one trainable 1-D ``flat_shards[r]``.  The original entries are removed
from the shard modules.  Before a forward pass the flat shards are all-gathered and the
full tensors are re-installed as plain (non-leaf) attributes, so autograd carries their
gradients back into the flat shards *summed over ranks without any 1/world scaling* — which
is exactly what makes training of replicated parameters correct here, because each rank's
replica only sees the partial gradient that flowed through its own weight slices.

The gather is skipped while no flat shard changed (``_version`` check), e.g. across
gradient-accumulation micro-steps.  Parameter order is ``sorted(names)`` unless the caller
passes an explicit sequence, and the layout (names, shapes, per-rank piece sizes) is saved alongside
the shards as the module's extra state (key ``sharding_manager._extra_state``): loading flat shards
into a model whose layout differs raises instead of silently scrambling parameters - the reference
keeps the order of a Python ``set`` and saves nothing (``src/tensor_parallel/sharding.py:41-44``).
A checkpoint without that key (one written by the reference) still loads.
Reference: ``src/tensor_parallel/sharding.py:18-180``.
"""
from __future__ import annotations

import logging
from typing import Collection, Dict, List, Optional, Sequence, Tuple

import torch
from torch import nn

from tensor_parallel_b200.parallel.actions import unit_bounds

logger = logging.getLogger(__name__)


def _tensor_key(t: torch.Tensor):
    return (t.data_ptr(), t.storage_offset(), tuple(t.stride()), tuple(t.shape), str(t.device))


@torch.no_grad()
def find_all_occurences(shard: nn.Module, names: Sequence[str]) -> List[List[Tuple[nn.Module, str]]]:
    """For each name, every ``(module, attribute)`` slot that holds that parameter, tied aliases included."""
    wanted = set(names)
    canonical_by_key: Dict[tuple, str] = {}
    slots: List[Tuple[str, nn.Module, str, tuple]] = []
    for module_name, sub in shard.named_modules(remove_duplicate=True):
        for local, param in sub._parameters.items():
            if param is None:
                continue
            full = f"{module_name}.{local}" if module_name else local
            key = _tensor_key(param) if param.numel() else ("empty", id(param))
            slots.append((full, sub, local, key))
            if full in wanted:
                canonical_by_key[key] = full
    found: Dict[str, List[Tuple[nn.Module, str]]] = {name: [] for name in names}
    for full, sub, local, key in slots:
        owner = full if full in wanted else canonical_by_key.get(key)
        if owner is not None:
            found[owner].append((sub, local))
    missing = [name for name in names if not found[name]]
    if missing:
        raise KeyError(f"parameters not found in the shard: {missing}")
    return [found[name] for name in names]


class Sharded(nn.Module):
    """Owner of ``flat_shards`` and of the gather-before-forward step."""

    def __init__(self, module, world_size: Optional[int] = None, replicated_param_names: Optional[Collection[str]] = None):
        super().__init__()
        self.preserve_shards_when_saving = True
        shards = module.module_shards
        self.sharded_param_names: Tuple[str, ...] = ()
        self.comm = getattr(module, "comm", None)
        if len(shards) == 1 and not getattr(module, "is_distributed", False):
            return
        self.world_size = world_size if world_size is not None else len(shards)
        self.local_ranks: Sequence[int] = getattr(module, "local_ranks", range(len(shards)))

        if replicated_param_names is None:
            if any(p.device.type == "meta" for p in module.parameters()):
                raise RuntimeError(
                    "the model still holds 'meta' parameters: create it with sharded=False, load the weights, "
                    "then call .apply_sharding()"
                )
            every = {name for name, _ in shards[0].named_parameters()}
            replicated_param_names = sorted(every - set(module.modified_parameters_names))
        self.sharded_param_names = tuple(replicated_param_names)
        if not self.sharded_param_names:
            logger.warning("ZeRO-3: no replicated parameters to shard")
            return

        by_name = dict(shards[0].named_parameters())
        self._shapes = [tuple(by_name[name].shape) for name in self.sharded_param_names]
        numels = [by_name[name].numel() for name in self.sharded_param_names]
        # piece sizes per rank, then padding as the last entry (part of the saved layout)
        self._sizes_with_pad: List[List[int]] = []
        for r in range(self.world_size):
            sizes = [unit_bounds(n, self.world_size, r)[1] - unit_bounds(n, self.world_size, r)[0] for n in numels]
            self._sizes_with_pad.append(sizes)
        flat_len = max(sum(sizes) for sizes in self._sizes_with_pad)
        for sizes in self._sizes_with_pad:
            sizes.append(flat_len - sum(sizes))

        flats = []
        with torch.no_grad():
            for shard, r in zip(shards, self.local_ranks):
                params = dict(shard.named_parameters())
                pieces = []
                for name, n in zip(self.sharded_param_names, numels):
                    lo, hi = unit_bounds(n, self.world_size, r)
                    pieces.append(params[name].detach().flatten()[lo:hi])
                first = params[self.sharded_param_names[0]]
                pieces.append(torch.zeros(self._sizes_with_pad[r][-1], dtype=first.dtype, device=first.device))
                flats.append(torch.cat(pieces))
        self.flat_shards = nn.ParameterList([nn.Parameter(f) for f in flats])

        self.param_occurences_by_rank = [find_all_occurences(shard, self.sharded_param_names) for shard in shards]
        for per_shard in self.param_occurences_by_rank:
            for slots in per_shard:
                for sub, local in slots:
                    sub._parameters.pop(local, None)
                    setattr(sub, local, None)
        self._last_versions = None

    # -- gather ------------------------------------------------------------------------------

    def _gather(self, all_cuda: bool) -> List[torch.Tensor]:
        """Return, per local shard, the ``[world, flat_len]`` stack of every rank's flat shard."""
        if self.comm is not None:
            return self.comm.all_gather_flat(list(self.flat_shards))
        stacks = []
        for mine in self.flat_shards:
            stacks.append(torch.stack([other.to(mine.device, non_blocking=True) for other in self.flat_shards]))
        return stacks

    def synchronize_weights(self, all_cuda: bool = False):
        if not self.sharded_param_names:
            return
        versions = tuple(f._version for f in self.flat_shards) + (torch.is_grad_enabled(),)
        if versions == self._last_versions:
            logger.debug("ZeRO-3: flat shards unchanged, re-using gathered parameters")
            return
        logger.debug("ZeRO-3: gathering flat shards")
        for stacked, per_shard in zip(self._gather(all_cuda), self.param_occurences_by_rank):
            for value, slots in zip(self._combine(stacked), per_shard):
                for sub, local in slots:
                    setattr(sub, local, value)
        self._last_versions = tuple(f._version for f in self.flat_shards) + (torch.is_grad_enabled(),)

    def _combine(self, stacked: torch.Tensor) -> List[torch.Tensor]:
        """``[world, flat_len]`` -> full tensors: piece *i* of every rank, concatenated, reshaped."""
        per_rank = [torch.split_with_sizes(stacked[r], self._sizes_with_pad[r]) for r in range(self.world_size)]
        return [
            torch.cat([per_rank[r][i] for r in range(self.world_size)]).view(shape)
            for i, shape in enumerate(self._shapes)
        ]

    # -- saving ------------------------------------------------------------------------------

    def layout(self) -> dict:
        return {
            "names": list(self.sharded_param_names),
            "shapes": [list(s) for s in getattr(self, "_shapes", [])],
            "sizes_with_pad": getattr(self, "_sizes_with_pad", []),
        }

    def get_extra_state(self):
        return self.layout()

    def set_extra_state(self, state):
        """Refuses flat shards that were cut from a different parameter list or with different piece sizes."""
        if not state or not state.get("names"):
            return
        mine = self.layout()
        for key in ("names", "shapes", "sizes_with_pad"):
            if [list(x) if isinstance(x, (list, tuple)) else x for x in state.get(key, [])] != \
                    [list(x) if isinstance(x, (list, tuple)) else x for x in mine[key]]:
                raise RuntimeError(
                    f"the checkpoint's ZeRO-3 flat shards were built with a different layout ({key} differ): "
                    f"checkpoint has {len(state.get('names', []))} parameters starting with {state.get('names', [])[:3]}, this model "
                    f"{len(mine['names'])} starting with {mine['names'][:3]}.  Pass sharded_param_names=<the checkpoint's names> when "
                    "wrapping, or load an un-sharded checkpoint (save_tensor_parallel) instead."
                )

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        if prefix + "_extra_state" not in state_dict:  # a checkpoint written without layout metadata: trust the caller
            state_dict[prefix + "_extra_state"] = self.layout()
        return super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)

    def state_dict(self, *args, **kwargs):
        if self.preserve_shards_when_saving:
            return super().state_dict(*args, **kwargs)
        return kwargs.get("destination", args[0] if args else {})
