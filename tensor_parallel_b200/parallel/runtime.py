"""``TensorParallel``: the single-process runtime that owns one shard per device.

A forward call (1) re-gathers ZeRO-3 parameters if they changed, (2) replicates every tensor
leaf of the arguments to all devices, (3) runs all shards concurrently — one long-lived
worker thread per rank, so no thread is created per call — and (4) returns the output of
rank ``output_device_index``.  A rank that raises aborts the collectives of its peers (they
raise :class:`TPCollectiveError` instead of waiting forever) and its exception is re-raised
in the caller.  Reference: ``src/tensor_parallel/tensor_parallel.py:26-315``.
"""
from __future__ import annotations

import logging
import queue
import atexit
import threading
import weakref
from typing import Any, Collection, List, Optional, Sequence, Union

import torch
from torch import nn

from tensor_parallel_b200.parallel.autoconfig import get_default_config
from tensor_parallel_b200.parallel.collectives import TPCollectiveError
from tensor_parallel_b200.parallel.rules import WRAPPED_PREFIX, Config, add_lora_rules
from tensor_parallel_b200.parallel.serving import ServingMixin
from tensor_parallel_b200.parallel.surgery import make_shard
from tensor_parallel_b200.parallel.zero import Sharded
from tensor_parallel_b200.utils.nested import nested_flatten, nested_pack

logger = logging.getLogger(__name__)


def canonicalize_device(device: Union[torch.device, str, int]) -> torch.device:
    device = torch.device(device)
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", 0)
    return device


def check_device_ids(device_ids: Optional[Sequence]) -> tuple:
    """``None`` means every visible CUDA device (possibly none, which disables splitting)."""
    if device_ids is None:
        device_ids = list(range(torch.cuda.device_count())) if torch.cuda.is_available() else []
    return tuple(canonicalize_device(d) for d in device_ids)


def _is_stateful_cache(obj) -> bool:
    return hasattr(obj, "update") and hasattr(obj, "get_seq_length") and not isinstance(obj, (torch.Tensor, nn.Module, dict))


_MIRRORED_CACHE_CALLS = ("reorder_cache", "batch_select_indices", "batch_repeat_interleave", "crop", "reset")


def _attach_cache_siblings(cache, world_size: int, keep_rank: int, devices, existing=None):
    """``existing``: the caches that the other ranks already own (one per rank; the entry of ``keep_rank`` is ignored);
    without it the siblings start as copies of ``cache``."""
    import copy

    if existing is not None:
        siblings = [cache if r == keep_rank else existing[r] for r in range(world_size)]
    else:
        siblings = [cache if r == keep_rank else copy.deepcopy(cache) for r in range(world_size)]
    cache.__dict__["_tp_siblings"] = siblings
    for method_name in _MIRRORED_CACHE_CALLS:
        original = getattr(cache, method_name, None)
        if original is None:
            continue

        def mirrored(*args, __name=method_name, __original=original, **kwargs):
            for r, sibling in enumerate(siblings):
                if sibling is cache:
                    continue
                local = [a.to(devices[r]) if isinstance(a, torch.Tensor) else a for a in args]
                getattr(sibling, __name)(*local, **kwargs)
            return __original(*args, **kwargs)

        cache.__dict__[method_name] = mirrored


class _RankWorker(threading.Thread):
    """Long-lived thread bound to one rank; executes closures handed over through a queue."""

    def __init__(self, rank: int):
        super().__init__(name=f"tp-rank-{rank}", daemon=True)
        self.jobs: "queue.SimpleQueue" = queue.SimpleQueue()
        self.start()

    def run(self):
        while True:
            job = self.jobs.get()
            if job is None:
                return
            fn, box, done = job
            try:
                box.append(("ok", fn()))
            except BaseException as exc:  # delivered to the caller thread
                box.append(("err", exc))
            finally:
                done.set()


_live_executors: "weakref.WeakSet" = weakref.WeakSet()
_retiring_threads: "weakref.WeakSet" = weakref.WeakSet()  # told to stop (e.g. when their model was collected), maybe still unwinding


def _stop_rank_threads():
    """The rank threads are daemons parked on a queue; stopping and joining them before the interpreter finalises keeps
    the C++ runtime from tearing down thread-local state underneath a live thread (seen as ``terminate called without
    an active exception`` and exit status 134 at the end of short scripts)."""
    for executor in list(_live_executors):
        try:
            executor.shutdown(join=True)
        except Exception:
            pass
    for thread in list(_retiring_threads):
        if thread.is_alive() and thread is not threading.current_thread():
            thread.join(timeout=5.0)


atexit.register(_stop_rank_threads)


class RankExecutor:
    """Runs one callable per rank concurrently on persistent threads."""

    def __init__(self, world_size: int):
        self.world_size = world_size
        self._workers: List[_RankWorker] = []
        self._lock = threading.Lock()
        _live_executors.add(self)

    def __deepcopy__(self, memo):
        return RankExecutor(self.world_size)  # threads are not copied; the copy starts its own on first use

    def __reduce__(self):
        return (RankExecutor, (self.world_size,))

    def _ensure(self):
        with self._lock:
            while len(self._workers) < self.world_size:
                self._workers.append(_RankWorker(len(self._workers)))

    def run(self, fns: Sequence, on_error=None) -> List[Any]:
        self._ensure()
        boxes, events = [], []
        for worker, fn in zip(self._workers, fns):
            box, done = [], threading.Event()

            def guarded(fn=fn):
                try:
                    return fn()
                except BaseException as exc:
                    if on_error is not None and not isinstance(exc, TPCollectiveError):
                        on_error(exc)
                    raise

            worker.jobs.put((guarded, box, done))
            boxes.append(box)
            events.append(done)
        for done in events:
            done.wait()
        results = [box[0] for box in boxes]
        primary = [r for status, r in results if status == "err" and not isinstance(r, TPCollectiveError)]
        secondary = [r for status, r in results if status == "err"]
        if primary or secondary:
            raise (primary or secondary)[0]
        return [r for _, r in results]

    def shutdown(self, join: bool = False):
        with self._lock:
            workers, self._workers = self._workers, []
        for w in workers:
            w.jobs.put(None)
            _retiring_threads.add(w)
        if join:
            for w in workers:
                if w is not threading.current_thread():
                    w.join(timeout=5.0)

    def __del__(self):
        try:
            self.shutdown()
        except Exception:
            pass


def parallel_apply_simple(modules, inputs, kwargs_tup=None, devices=None, executor: Optional[RankExecutor] = None, group=None):
    """Run ``modules[i](*inputs[i], **kwargs_tup[i])`` for all ranks at once; grad mode and
    autocast state of the caller are propagated into the workers."""
    n = len(modules)
    kwargs_tup = kwargs_tup if kwargs_tup is not None else ({},) * n
    devices = devices if devices is not None else [None] * n
    grad_on = torch.is_grad_enabled()
    autocast_state = {
        kind: (torch.is_autocast_enabled(kind), torch.get_autocast_dtype(kind)) for kind in ("cpu", "cuda")
    }

    def make(i):
        module, args, kwargs, device = modules[i], inputs[i], kwargs_tup[i], devices[i]

        def call():
            torch.set_grad_enabled(grad_on)
            if not isinstance(args, (list, tuple)):
                call_args = (args,)
            else:
                call_args = args
            kind = device.type if device is not None and device.type in autocast_state else "cpu"
            enabled, dtype = autocast_state[kind]
            if device is not None and device.type == "cuda":
                torch.cuda.set_device(device)
            with torch.autocast(kind, dtype=dtype, enabled=enabled):
                return module(*call_args, **kwargs)

        return call

    own = executor is None
    executor = executor if executor is not None else RankExecutor(n)
    try:
        if group is not None:
            group.reset()
        return executor.run([make(i) for i in range(n)], on_error=group.abort if group is not None else None)
    finally:
        if own:
            executor.shutdown()


class TensorParallel(ServingMixin, nn.Module):
    def __init__(
        self,
        module: nn.Module,
        device_ids: Optional[Sequence[torch.device]] = None,
        output_device: Optional[torch.device] = None,
        output_device_index: Optional[int] = None,
        tensor_parallel_config: Optional[Config] = None,
        delay_init: bool = False,
        distributed: bool = True,
        sharded: bool = True,
        sharded_param_names: Optional[Collection[str]] = None,
        fuse: Optional[bool] = None,
    ):
        super().__init__()
        original_params = sum(p.numel() for p in module.parameters())
        if output_device is not None and output_device_index is not None:
            raise ValueError("pass either output_device or output_device_index, not both")
        devices = check_device_ids(device_ids)
        if output_device is not None:
            output_device = canonicalize_device(output_device)
            if output_device not in devices:
                raise ValueError(f"output device {output_device} is not one of {devices}")
            output_device_index = devices.index(output_device)
        elif output_device_index is None:
            output_device_index = 0

        self.module_shards = nn.ModuleList()
        self.devices = devices
        self.device_ids = [d.index if d.type == "cuda" else None for d in devices]
        self.output_device_index = output_device_index
        self.all_cuda = all(d.type == "cuda" for d in devices)
        self.need_delayed_init = delay_init
        self.sharding_manager = None
        self.preserve_shards_when_saving = True
        self._executor: Optional[RankExecutor] = None
        world_size = len(devices)

        if world_size <= 1:  # nothing to split: keep the module as the only "shard"
            self.module_shards.append(module)
            if world_size == 1 and not delay_init:
                self.module_shards[0].to(devices[0])
            return

        if tensor_parallel_config is None:
            tensor_parallel_config = get_default_config(module, devices)
            logger.info("using the automatic config: every linear / embedding / conv layer is split on its own")
        tensor_parallel_config = add_lora_rules(module, tensor_parallel_config)
        self.tensor_parallel_config = tensor_parallel_config

        backend = None
        if self.all_cuda and len(set(devices)) == world_size:
            from tensor_parallel_b200.parallel.device_backend import maybe_thread_backend

            backend = maybe_thread_backend(devices)
        self._device_backend = backend
        live = tensor_parallel_config.create_collective_ops(devices, distributed, backend=backend)
        self._rank_group = live.rank_group
        self._live_config = live

        self.modified_parameters_names = set()
        for rank, device in enumerate(devices):
            shard, sliced = make_shard(
                module, torch.device("cpu") if delay_init else device, live, rank=rank, world_size=world_size
            )
            self.module_shards.append(shard)
            self.modified_parameters_names.update(sliced)

        per_shard = [sum(p.numel() for p in s.parameters()) for s in self.module_shards]
        if sum(per_shard) < original_params:
            raise AssertionError("internal error: parameters were lost while sharding")
        self.param_fractions = tuple(n / max(original_params, 1) for n in per_shard)
        waste = (sum(self.param_fractions) - 1) / world_size
        logger.log(
            logging.DEBUG if waste < 0.1 else logging.WARNING,
            "model has %d parameters, shards hold %s: each device spends %.3f%% extra parameter memory",
            original_params, per_shard, waste * 100,
        )

        # one empty parameter per device: if the user moves the whole model with .cuda()/.to(),
        # these all land on one device and forward() can tell
        self._sanity_check_params = nn.ParameterList(
            [nn.Parameter(torch.empty(0, device=d), requires_grad=False) for d in devices]
        )
        if fuse is None or fuse:
            from tensor_parallel_b200.parallel.planner import apply_fusion_plan

            self.fused_sites = apply_fusion_plan(self)
        if sharded:
            self.apply_sharding(sharded_param_names)

    # -- ZeRO-3 -------------------------------------------------------------------------------

    def apply_sharding(self, replicated_param_names: Optional[Collection[str]] = None):
        if self.sharding_manager is not None:
            raise RuntimeError("sharding was already applied; pass sharded=False at construction to do it later")
        self.sharding_manager = Sharded(self, len(self.devices), replicated_param_names)

    @torch.no_grad()
    def reduce_replicated_gradients(self) -> int:
        """With ``sharded=False`` the parameters that no state rule splits stay replicated on every rank, and after
        ``backward()`` each replica only holds the part of the gradient that flowed through its own rank's slices
        downstream (the reference has the same property and leaves it there: replicated-parameter training is only
        correct with ZeRO-3 on).  This sums those partial gradients over the ranks and gives every replica the total,
        so that a per-replica optimizer keeps the replicas identical.  Returns the number of parameters reduced; a
        no-op when ZeRO-3 sharding is active (its flat shards are sum-reduced already)."""
        if self.sharding_manager is not None or len(self.module_shards) < 2:
            return 0
        named = [dict(shard.named_parameters()) for shard in self.module_shards]
        reduced = 0
        for name, first in named[0].items():
            if name in self.modified_parameters_names:
                continue
            replicas = [params.get(name) for params in named]
            if any(p is None for p in replicas) or not first.requires_grad or all(p.grad is None for p in replicas):
                continue
            total = torch.zeros_like(first)
            for p in replicas:
                if p.grad is not None:
                    total += p.grad.to(total.device)
            for p in replicas:
                p.grad = total.to(p.device).clone()
            reduced += 1
        return reduced

    # -- forward ------------------------------------------------------------------------------

    def prepare_args_kwargs_for_forward(self, *args, **kwargs):
        """Replicate every tensor leaf to every device; other leaves are shared by reference."""
        template = (args, kwargs)
        leaves = list(nested_flatten(template))
        per_rank = []
        for rank, device in enumerate(self.devices):
            moved = []
            for leaf in leaves:
                if isinstance(leaf, torch.Tensor):
                    leaf = leaf.to(device, non_blocking=True)
                elif _is_stateful_cache(leaf):
                    leaf = self._cache_for_rank(leaf, rank)
                moved.append(leaf)
            per_rank.append(nested_pack(moved, template))
        return zip(*per_rank)

    def _cache_for_rank(self, cache, rank: int):
        """Stateful KV-cache objects (``transformers.Cache``) are updated in place by the model, so
        every rank needs its own instance: the output rank keeps the caller's object, the other
        ranks get empty siblings that live as long as the caller's object and mirror its
        batch-reordering calls (beam search)."""
        if rank == self.output_device_index:
            siblings = cache.__dict__.get("_tp_siblings")
            if siblings is None:
                _attach_cache_siblings(cache, len(self.devices), self.output_device_index, self.devices)
            return cache
        if cache.__dict__.get("_tp_siblings") is None:
            _attach_cache_siblings(cache, len(self.devices), self.output_device_index, self.devices)
        return cache.__dict__["_tp_siblings"][rank]

    def _materialize(self):
        if self.need_delayed_init:
            for shard, device in zip(self.module_shards, self.devices):
                shard.to(device)
            self.need_delayed_init = False

    def run_shards(self, modules, args, kwargs):
        inputs, kwargs_tup = self.prepare_args_kwargs_for_forward(*args, **kwargs)
        if self._executor is None:
            self._executor = RankExecutor(len(self.devices))
        outputs = parallel_apply_simple(
            modules, inputs, kwargs_tup, self.devices, executor=self._executor, group=getattr(self, "_rank_group", None)
        )
        self._adopt_new_caches(outputs)
        return outputs[self.output_device_index]

    def _adopt_new_caches(self, outputs):
        """A model called with ``use_cache=True`` and no cache creates a stateful cache object on every rank, each holding
        that rank's heads.  Only the output rank's object reaches the caller; the others are tied to it here, so that a
        later call that passes the object back finds every rank's history."""
        mine = outputs[self.output_device_index]
        fields = getattr(mine, "keys", None)
        if fields is None:
            return
        for key in list(fields()):
            value = mine[key] if hasattr(mine, "__getitem__") else getattr(mine, key)
            if _is_stateful_cache(value) and value.__dict__.get("_tp_siblings") is None:
                others = []
                for out in outputs:
                    other = out[key] if hasattr(out, "__getitem__") else getattr(out, key, None)
                    others.append(other)
                if all(_is_stateful_cache(o) for o in others):
                    _attach_cache_siblings(value, len(self.devices), self.output_device_index, self.devices, existing=others)

    def check_status(self):
        """Raises ``TPCollectiveError`` if a kernel gave up waiting for a peer GPU (synchronises the devices)."""
        for comm in getattr(getattr(self, "_device_backend", None), "comms", None) or ():
            comm.check_status()

    def forward(self, *args, **kwargs):
        self._materialize()
        for comm in getattr(getattr(self, "_device_backend", None), "comms", None) or ():
            comm.poll_status()  # a device-side wait that gave up during an earlier call raises here, without a sync
        if self.sharding_manager is not None:
            self.sharding_manager.synchronize_weights(self.all_cuda)
        if len(self.module_shards) <= 1:
            return self.module_shards[0](*args, **kwargs)
        if any(p.device != d for p, d in zip(self._sanity_check_params, self.devices)):
            raise ValueError(
                "shards are no longer on their devices: was .cuda() or .to(device) called on the "
                "tensor-parallel model? Move the original model before wrapping instead."
            )
        return self.run_shards(list(self.module_shards), args, kwargs)

    # -- saving -------------------------------------------------------------------------------

    def set_preserve_shards_when_saving(self, value: bool):
        self.preserve_shards_when_saving = value
        if self.sharding_manager is not None:
            self.sharding_manager.preserve_shards_when_saving = value

    def state_dict(self, *args, **kwargs):
        state = super().state_dict(*args, **kwargs)
        if self.preserve_shards_when_saving or len(self.module_shards) <= 1:
            return state
        prefix = kwargs.get("prefix", "")
        world = len(self.module_shards)
        shard_prefix = prefix + "module_shards."

        for r in range(world):
            state.pop(f"{prefix}_sanity_check_params.{r}", None)

        # collect the per-rank pieces of every original tensor under its original name
        pieces = {}
        for key in [k for k in state if k.startswith(shard_prefix)]:
            rank_str, _, inner = key[len(shard_prefix):].partition(".")
            original = inner.replace(WRAPPED_PREFIX, "")
            pieces.setdefault(original, {})[int(rank_str)] = state.pop(key)

        for original, by_rank in pieces.items():
            tensors = [by_rank[r] for r in sorted(by_rank)]
            for pattern, action in self.tensor_parallel_config.state_rules.items():
                if pattern.search(original) is not None:
                    state[prefix + original] = action.undo(tensors)
                    break
            else:
                state[prefix + original] = tensors[0]
        return self.process_sharded_state_dict(state, prefix)

    def process_sharded_state_dict(self, destination, prefix: str = ""):
        """Add the full values of ZeRO-3 parameters (they live in no shard module's state)."""
        manager = self.sharding_manager
        if manager is not None and manager.sharded_param_names:
            with torch.no_grad():
                stacked = manager._gather(self.all_cuda)[0]
                full = manager._combine(stacked)
            for name, value in zip(manager.sharded_param_names, full):
                destination[prefix + name.replace(WRAPPED_PREFIX, "")] = value.detach()
        return destination

    def _load_from_state_dict(self, *args, **kwargs):
        return super()._load_from_state_dict(*args, **kwargs)
