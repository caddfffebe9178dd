"""The flagged-word exchange of the fused GEMM + all-reduce kernel, run by CPU threads standing in for ranks
(host-side model in ``tensor_parallel_b200/utils/protocol_model.py``)."""
import pytest

from tensor_parallel_b200.utils import protocol_model as pm
from tensor_parallel_b200.utils import tracing


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sums_are_exact_under_random_schedules(world):
    calls = [(8, 256), (8, 256), (3, 384), (8, 256), (16, 128), (1, 256)]
    for seed in range(3):
        errs = pm.run_ranks(world, calls, tile_keyed=True, jitter=2e-4, seed=seed)
        assert max(errs) < 1e-9, errs


def test_interleaved_shapes_never_accept_a_stale_word():
    """A short shape advances the epochs of the low tiles only; the long shape that follows must not mistake the words
    it left behind for its own.  With words keyed by tile this holds for any interleaving."""
    long_shape, short_shape = (8, 384), (64, 128)  # 3 tiles / 1 tile
    calls = [long_shape] * 4 + [short_shape] * 2 + [long_shape] * 3 + [short_shape] + [long_shape] * 2
    errs = pm.run_ranks(2, calls, tile_keyed=True, jitter=1e-4, seed=1)
    assert max(errs) < 1e-9, errs


def test_shape_dependent_addresses_would_accept_stale_words():
    """The model reproduces why the kernel keys word addresses by tile: with the shape-dependent order a word written by
    another shape can sit where a later call polls, carrying exactly the epoch that call expects."""
    # half 0 sees calls 0, 2, 4: two long calls put the epochs of tiles 0..2 at 2; the short call writes flag 3 into words
    # of tile 0 that, in the long shape's addressing, belong to tile 1 (epoch 2 -> expected flag 3)
    long_shape, short_shape = (2, 384), (64, 128)
    calls = [long_shape, long_shape, long_shape, long_shape, short_shape, long_shape, long_shape]
    late = {(1, 6): 0.3}  # rank 1 starts the last call late: rank 0 polls while only the stale words are there
    errs = pm.run_ranks(2, calls, tile_keyed=False, seed=0, late=late)
    assert max(errs) > 1e-3, errs   # the shape-dependent order returns a wrong sum ...
    errs = pm.run_ranks(2, calls, tile_keyed=True, seed=0, late=late)
    assert max(errs) < 1e-9, errs   # ... the tile-keyed order waits for the straggler and gets it right


def test_nvtx_ranges_nest_and_are_free_when_off():
    calls = []

    @tracing.traced("outer")
    def outer():
        with tracing.nvtx_range("inner"):
            calls.append(tracing._depth)
        return 7

    tracing.enable(False)
    assert outer() == 7 and calls == [0]
    tracing.enable(True)
    try:
        assert outer() == 7 and calls[-1] == 2 and tracing._depth == 0
    finally:
        tracing.enable(False)
