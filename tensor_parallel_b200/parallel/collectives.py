"""Collective operations usable as rule actions: ``op(value, rank) -> value``.

Three families live here:

* thread collectives for the single-process mode (one Python thread per rank), built on an
  abortable, time-limited :class:`Rendezvous` instead of bare barriers, so that a rank that
  dies before reaching a collective turns into :class:`TPCollectiveError` on every other rank
  rather than a hang;
* ``torch.distributed`` collectives for the one-process-per-GPU mode, written as true adjoint
  pairs (all-reduce <-> all-reduce, all-gather <-> reduce-scatter) so gradients are exact;
* thin adaptors that route CUDA tensors to the device-side kernels in
  ``tensor_parallel_b200.ops.comm`` when a symmetric heap is attached.

Reference behaviour being re-designed: ``src/tensor_parallel/communications.py:16-191`` and
``src/tensor_parallel/cross_device_ops.py:15-109``.
"""
from __future__ import annotations

import os
import threading
import time
from typing import Any, Callable, List, Optional, Sequence

import torch
import torch.distributed as dist

DEFAULT_TIMEOUT_S = float(os.environ.get("TENSOR_PARALLEL_TIMEOUT", "600"))


class TPCollectiveError(RuntimeError):
    """A collective could not complete: a peer rank failed, or the wait timed out."""


class RankGroup:
    """Host-side failure domain shared by every collective of one tensor-parallel model."""

    def __init__(self, world_size: int, timeout: Optional[float] = None):
        self.world_size = world_size
        self.timeout = DEFAULT_TIMEOUT_S if timeout is None else timeout
        self._lock = threading.Lock()
        self._failure: Optional[BaseException] = None
        self._waiters: List["Rendezvous"] = []

    def register(self, rendezvous: "Rendezvous"):
        with self._lock:
            self._waiters.append(rendezvous)

    def __deepcopy__(self, memo):
        # a copy of a model gets a failure domain of its own (fresh lock, no history); the copied collectives find it
        # through the memo and register themselves again
        return RankGroup(self.world_size, self.timeout)

    def __reduce__(self):  # pickling (torch.save of a whole model): locks and history are not part of the state
        return (RankGroup, (self.world_size, self.timeout))

    @property
    def failure(self) -> Optional[BaseException]:
        return self._failure

    def abort(self, cause: BaseException):
        """Wake every rank blocked in a collective; they raise :class:`TPCollectiveError`."""
        with self._lock:
            if self._failure is None:
                self._failure = cause
            waiters = list(self._waiters)
        for r in waiters:
            r.wake()

    def reset(self):
        """Forget a past failure and drop half-finished exchanges (called before each forward)."""
        with self._lock:
            failed = self._failure is not None
            self._failure = None
            waiters = list(self._waiters)
        if failed:
            for r in waiters:
                r.clear()


class Rendezvous:
    """Reusable all-to-all exchange of Python objects between the rank threads."""

    def __init__(self, group: RankGroup):
        self.group = group
        self.world_size = group.world_size
        self._cond = threading.Condition()
        self._slots: List[Any] = [None] * self.world_size
        self._arrived = 0
        self._round = 0
        self._published: List[Any] = []
        group.register(self)

    def __deepcopy__(self, memo):
        import copy

        return Rendezvous(copy.deepcopy(self.group, memo))

    def __reduce__(self):
        return (Rendezvous, (self.group,))

    def wake(self):
        with self._cond:
            self._cond.notify_all()

    def clear(self):
        with self._cond:
            self._slots = [None] * self.world_size
            self._arrived = 0
            self._round += 1

    def _raise_if_failed(self):
        cause = self.group.failure
        if cause is not None:
            raise TPCollectiveError(f"a peer rank failed: {cause!r}") from cause

    def exchange(self, rank: int, value: Any) -> List[Any]:
        """Deposit ``value`` for ``rank``; return every rank's value (index = rank)."""
        deadline = time.monotonic() + self.group.timeout
        with self._cond:
            self._raise_if_failed()
            my_round = self._round
            self._slots[rank] = value
            self._arrived += 1
            if self._arrived == self.world_size:
                self._published = self._slots
                self._slots = [None] * self.world_size
                self._arrived = 0
                self._round += 1
                self._cond.notify_all()
                return self._published
            while self._round == my_round:
                self._raise_if_failed()
                remaining = deadline - time.monotonic()
                if remaining <= 0:
                    err = TPCollectiveError(
                        f"rank {rank} waited {self.group.timeout:.1f}s in a collective; "
                        f"{self._arrived}/{self.world_size} ranks arrived"
                    )
                    self._cond.release()
                    try:
                        self.group.abort(err)
                    finally:
                        self._cond.acquire()
                    raise err
                self._cond.wait(min(remaining, 1.0))
            self._raise_if_failed()
            return self._published


class CollectiveBase:
    def __call__(self, x, rank: int):
        raise NotImplementedError


class CollectiveOperation(CollectiveBase):
    """Run ``func(in_0, ..., in_{W-1}) -> (out_0, ..., out_{W-1})`` once per call on rank
    ``authoritative_rank`` and hand output *r* to rank *r*.  An exception inside ``func`` is
    re-raised on every rank (reference: ``src/tensor_parallel/communications.py:21-52``)."""

    def __init__(self, world_size: int, func: Callable, authoritative_rank: int = 0, group: Optional[RankGroup] = None):
        self.world_size, self.func, self.authoritative_rank = world_size, func, authoritative_rank
        self.group = group if group is not None else RankGroup(world_size)
        self._inputs = Rendezvous(self.group)
        self._outputs = Rendezvous(self.group)

    def rebind(self, group: RankGroup) -> "CollectiveOperation":
        return CollectiveOperation(self.world_size, self.func, self.authoritative_rank, group)

    def __call__(self, x, rank: int):
        inputs = self._inputs.exchange(rank, x)
        payload = None
        if rank == self.authoritative_rank:
            try:
                payload = ("ok", self.func(*inputs))
            except Exception as exc:  # forwarded to every rank below
                payload = ("err", exc)
        status, result = self._outputs.exchange(rank, payload)[self.authoritative_rank]
        if status == "err":
            raise result
        return result[rank]


class ThreadAllGather(CollectiveBase):
    """Concatenate every rank's tensor along ``dim`` (slices may differ in length)."""

    def __init__(self, group: RankGroup, dim: int = -1):
        self.group, self.dim = group, dim
        self._rv = Rendezvous(group)

    def __call__(self, x: torch.Tensor, rank: int) -> torch.Tensor:
        parts = self._rv.exchange(rank, x)
        return torch.cat([p.to(x.device, non_blocking=True) for p in parts], dim=self.dim)


class ThreadAllReduce(CollectiveBase):
    """Sum over ranks as reduce-scatter + all-gather: rank *r* adds up slice *r* of everyone's
    flattened tensor (in rank order, so the result is bit-identical on all ranks), then the
    reduced slices are exchanged.  Differentiable: it is composed of ordinary torch ops."""

    def __init__(self, group: RankGroup):
        self.group = group
        self._scatter, self._gather = Rendezvous(group), Rendezvous(group)

    def __call__(self, x: torch.Tensor, rank: int) -> torch.Tensor:
        world = self.group.world_size
        everyone = self._scatter.exchange(rank, x)
        mine = None
        for peer in everyone:
            piece = peer.flatten().tensor_split(world)[rank].to(x.device, non_blocking=True)
            mine = piece if mine is None else mine + piece
        reduced = self._gather.exchange(rank, mine)
        return torch.cat([p.to(x.device, non_blocking=True) for p in reduced]).view_as(x)


class ThreadGatherKV(CollectiveBase):
    """Zip per-rank ``(k, v)`` caches into :class:`PerDeviceTensors` (host-only, moves no data)."""

    def __init__(self, group: RankGroup):
        self.group = group
        self._rv = Rendezvous(group)

    def __call__(self, kv, rank: int):
        from tensor_parallel_b200.parallel.aux import gather_kv

        if kv is None:  # no cache was asked for: every rank sees None at this site, nothing to zip, no need to meet
            return None
        everyone = self._rv.exchange(rank, kv)
        return gather_kv(*everyone, world_size=self.group.world_size)[rank]


# --------------------------------------------------------------------------------------------
# torch.distributed (one process per rank)
# --------------------------------------------------------------------------------------------


def _pg_sizes(x: torch.Tensor, dim: int, pg) -> List[int]:
    world = dist.get_world_size(pg)
    mine = torch.tensor([x.shape[dim]], dtype=torch.int64, device=x.device if x.is_cuda else "cpu")
    everyone = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(everyone, mine, group=pg)
    return [int(t.item()) for t in everyone]


class _DistAllReduceFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, pg):
        ctx.pg = pg
        out = x.contiguous().clone()
        dist.all_reduce(out, group=pg)
        return out

    @staticmethod
    def backward(ctx, grad):
        grad = grad.contiguous().clone()
        dist.all_reduce(grad, group=ctx.pg)
        return grad, None


class _DistAllGatherFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim, sizes, pg):
        ctx.pg, ctx.dim, ctx.sizes = pg, dim, sizes
        ctx.rank = dist.get_rank(pg)
        x = x.contiguous()
        longest = max(sizes)
        if x.shape[dim] != longest:
            pad_shape = list(x.shape)
            pad_shape[dim] = longest - x.shape[dim]
            x = torch.cat([x, x.new_zeros(pad_shape)], dim=dim)
        parts = [torch.empty_like(x) for _ in sizes]
        dist.all_gather(parts, x, group=pg)
        return torch.cat([p.narrow(dim, 0, n) for p, n in zip(parts, sizes)], dim=dim)

    @staticmethod
    def backward(ctx, grad):
        grad = grad.contiguous().clone()
        dist.all_reduce(grad, group=ctx.pg)  # reduce-scatter written as all-reduce + slice (works on gloo too)
        start = sum(ctx.sizes[: ctx.rank])
        return grad.narrow(ctx.dim, start, ctx.sizes[ctx.rank]).contiguous(), None, None, None


class DistributedAllReduce(CollectiveBase):
    """All-reduce across processes; its backward is an all-reduce of the gradients."""

    def __init__(self, world_size: int, process_group=None):
        self.world_size, self.pg = world_size, process_group

    def __call__(self, x: torch.Tensor, rank: int = 0) -> torch.Tensor:
        return _DistAllReduceFn.apply(x, self.pg)


class DistributedAllGather(CollectiveBase):
    """All-gather along ``dim`` across processes (uneven slices allowed); backward is a
    summing reduce-scatter, so the result carries gradients."""

    def __init__(self, world_size: int, dim: int = -1, process_group=None):
        self.world_size, self.dim, self.pg = world_size, dim, process_group
        self._size_cache = {}

    def __call__(self, x: torch.Tensor, rank: int = 0) -> torch.Tensor:
        dim = self.dim % x.ndim
        key = (tuple(x.shape), dim)
        sizes = self._size_cache.get(key)
        if sizes is None:
            sizes = self._size_cache[key] = _pg_sizes(x, dim, self.pg)
        return _DistAllGatherFn.apply(x, dim, sizes, self.pg)


class LocalGatherKV(CollectiveBase):
    """One-process-per-rank counterpart of :class:`ThreadGatherKV`: the cache stays local."""

    def __call__(self, kv, rank: int = 0):
        return kv


class _ZeroGradFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return x.view_as(x)

    @staticmethod
    def backward(ctx, grad):
        return torch.zeros_like(grad)


def mute_gradient(tree):
    """Identity whose backward is zero.  In the multi-process mode only the output rank's copy
    of the (replicated) loss may seed the backward pass; the other ranks still run their
    backward graph so that the collectives pair up, but contribute zero cotangents.  This is
    the same convention the single-process mode follows (only one rank's output is returned)."""
    from tensor_parallel_b200.utils.nested import nested_map

    return nested_map(
        lambda leaf: _ZeroGradFn.apply(leaf) if isinstance(leaf, torch.Tensor) and leaf.requires_grad else leaf, tree
    )
