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


@pytest.mark.parametrize("world", [2, 4, 8])
def test_small_all_reduce_is_exact_for_changing_sizes(world):
    """Sizes in changing order (a word is reused by calls of different extent; blocks that only large calls use keep
    lower epochs) and more calls than parities, under random thread schedules."""
    sizes = [3, 32, 100, 3, 8, 100, 17, 64, 100, 3]
    for seed in range(2):
        errs = pm.run_small_all_reduce(world, sizes, jitter=1e-4, seed=seed)
        assert max(errs) < 1e-9, errs


def test_small_all_reduce_needs_both_parities():
    """A rank that is slow to READ call 0 while its peer races ahead: with two alternating areas the peer's words of call
    1 land beside those of call 0, and the peer cannot start call 2 before the slow rank has sent call 1 (after its
    reads); with a single area the words of call 1 overwrite what the slow rank still has to read."""
    slow = {(1, 0): 0.3}
    errs = pm.run_small_all_reduce(2, [16, 16, 16], parities=2, read_delay=slow)
    assert max(errs) < 1e-9, errs
    with pytest.raises(TimeoutError):
        pm.run_small_all_reduce(2, [16, 16, 16], parities=1, read_delay=slow, timeout=1.0)


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


def _check_decomposition(grid, tiles, k_blocks, bound=None):
    per_cta = pm.stream_k_items(grid, tiles, k_blocks)
    covered = {}
    by_tile = {}
    for cta, items in enumerate(per_cta):
        for tile, kb0, kb1, ordinal, contributors in items:
            assert 0 <= kb0 < kb1 <= k_blocks
            for kb in range(kb0, kb1):
                assert (tile, kb) not in covered, "a unit was dealt out twice"
                covered[(tile, kb)] = cta
            by_tile.setdefault(tile, []).append((cta, ordinal, contributors))
    assert len(covered) == tiles * k_blocks, "a unit was left out"
    for tile, entries in by_tile.items():
        ctas = sorted(c for c, _, _ in entries)
        assert len(set(ctas)) == len(ctas), "a CTA holds two pieces of one tile"
        assert {o for _, o, _ in entries} == set(range(len(entries))), "ordinals must number the contributors 0..n-1"
        assert all(n == len(entries) for _, _, n in entries), "every contributor must know the same count"
        assert [o for _, o, _ in sorted(entries)] == list(range(len(entries))), "ordinals follow the CTA order (deterministic sum)"
        if bound is not None:
            assert len(entries) <= bound
    return per_cta


def test_stream_k_decomposition_covers_every_unit_once():
    import random

    rng = random.Random(0)
    for _ in range(300):
        tiles, k_blocks = rng.randint(1, 300), rng.randint(1, 200)
        grid = rng.randint(1, min(148, tiles * k_blocks))
        _check_decomposition(grid, tiles, k_blocks)


@pytest.mark.parametrize("features,k", [(4096, 4096), (12288, 4096), (22016, 4096), (4096, 11008), (32000, 4096), (1536, 4096),
                                        (2752, 4096), (4096, 1376), (4096, 512), (4000, 4096), (256, 64), (65024, 8192), (128, 16384)])
def test_stream_k_planner_bounds_the_contributors(features, k):
    """For the shapes of the Llama / Falcon layers (whole and sharded 2- to 8-way) the planner's grid keeps the number of
    CTAs that share one tile within the parking slots of the workspace."""
    tiles, kb64 = (features + 127) // 128, (k + 63) // 64
    plan = pm.stream_k_grid(tiles, kb64)
    if plan is None:
        return
    kbox, k_blocks, grid, bound = plan
    assert bound <= 8
    per_cta = _check_decomposition(grid, tiles, k_blocks, bound=bound)
    busy = [sum(kb1 - kb0 for _, kb0, kb1, _, _ in items) for items in per_cta]
    assert max(busy) - min(busy) <= 1, "every CTA streams the same number of units (give or take one)"
