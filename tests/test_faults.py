"""Failure detection on the host: a rank that raises or never arrives must surface as an error
on every rank within the timeout, never as a hang.  No GPU is involved."""
import threading
import time

import pytest
import torch
from torch import nn

import tensor_parallel_b200 as tp
from tensor_parallel_b200.parallel.collectives import RankGroup, Rendezvous, ThreadAllReduce, TPCollectiveError


class FailsOnRank(nn.Module):
    """Raises inside the forward of one rank, before the next collective."""

    def __init__(self):
        super().__init__()
        self.bad_rank = None
        self.rank = None

    def forward(self, x):
        if self.rank is not None and self.rank == self.bad_rank:
            raise ValueError("injected failure")
        return x


def _build(world=3):
    model = nn.Sequential(nn.Linear(8, 16), FailsOnRank(), nn.Linear(16, 8))
    wrapped = tp.TensorParallel(model, ["cpu"] * world, sharded=False)
    for rank, shard in enumerate(wrapped.module_shards):
        shard[1].rank = rank
    return model, wrapped


def test_rank_exception_propagates_and_model_recovers():
    model, wrapped = _build()
    x = torch.randn(4, 8)
    for shard in wrapped.module_shards:
        shard[1].bad_rank = 1
    start = time.monotonic()
    with pytest.raises(ValueError, match="injected failure"):
        wrapped(x)
    assert time.monotonic() - start < 30
    for shard in wrapped.module_shards:
        shard[1].bad_rank = None
    torch.testing.assert_close(wrapped(x), model(x), atol=1e-6, rtol=1e-5)  # usable again after the failure


def test_missing_rank_times_out():
    group = RankGroup(world_size=2, timeout=0.5)
    op = ThreadAllReduce(group)
    start = time.monotonic()
    with pytest.raises(TPCollectiveError, match="waited"):
        op(torch.ones(4), rank=0)  # rank 1 never joins
    assert 0.4 < time.monotonic() - start < 10


def test_abort_wakes_waiting_ranks():
    group = RankGroup(world_size=3, timeout=60)
    rv = Rendezvous(group)
    errors = []

    def waiter(rank):
        try:
            rv.exchange(rank, rank)
        except TPCollectiveError as exc:
            errors.append(exc)

    threads = [threading.Thread(target=waiter, args=(r,)) for r in (0, 1)]
    for t in threads:
        t.start()
    time.sleep(0.2)
    group.abort(RuntimeError("rank 2 died"))
    for t in threads:
        t.join(timeout=10)
    assert len(errors) == 2 and all("rank 2 died" in repr(e.__cause__) for e in errors)
    group.reset()
    results = []
    threads = [threading.Thread(target=lambda r=r: results.append(rv.exchange(r, r))) for r in range(3)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=10)
    assert all(r == [0, 1, 2] for r in results)


def test_exception_inside_collective_function_reaches_all_ranks():
    def boom(*xs):
        raise KeyError("inside func")

    op = tp.CollectiveOperation(world_size=2, func=boom)
    errors = []

    def run(rank):
        try:
            op(torch.ones(1), rank)
        except KeyError as exc:
            errors.append(exc)

    threads = [threading.Thread(target=run, args=(r,)) for r in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=10)
    assert len(errors) == 2
