"""Executable host-side model of the flagged-word exchange that the fused GEMM + all-reduce kernel uses for few-token
tiles (``csrc/gemm_sm100.cu``), so that the protocol itself can be exercised by CPU threads standing in for ranks.

What is modelled, word for word:

* every rank owns two workspace halves; consecutive calls alternate between them;
* half ``h`` of rank ``d`` holds one slot per source rank; a slot is an array of 16-byte words
  ``(values(t, t + 1), flag, values(t + 2, t + 3), flag)`` (each half is one 8-byte unit: two bf16 values and the
  flag) addressed ``tile * TILE_WORDS + quad * ROWS + row``
  (or, with ``tile_keyed=False``, the shape-dependent ``(tile * ROWS + row) * quads + quad`` order that an earlier
  version of the kernel used and that this model shows to be unsafe when shapes are interleaved);
* a call on tile ``t`` uses flag ``epoch[h][t] + 1`` and stores it back; epochs live with the rank and only grow;
* the sender stores its words into every rank's slot (in any order, a word at a time); the receiver polls the words of
  its own tile and accepts a word when both flags equal the flag it expects; values are summed in rank order.

The two halves are enough because a rank can run at most one call ahead of a peer: its call ``i + 1`` cannot complete
before that peer has pushed its own call ``i + 1``, which the peer does only after it has finished reading call ``i``.

The same module models the barrier-free small all-reduce of ``csrc/comm.cu`` (``SmallAllReduceRank``).
"""
from __future__ import annotations

import random
import threading
import time
from typing import Dict, List, Sequence, Tuple

ROWS = 128                    # feature rows per tile
TILE_WORDS = ROWS * 16        # words one tile owns (up to 16 token quads)


class Heap:
    """Flagged areas of all ranks: ``mem[dest][half][src]`` maps a word index to ``((a, b), f0, (c, d), f1)``."""

    def __init__(self, world: int):
        self.world = world
        self.mem: List[List[List[Dict[int, Tuple[float, int, float, int]]]]] = [
            [[dict() for _ in range(world)] for _ in range(2)] for _ in range(world)
        ]


def _word_index(tile: int, row: int, pair: int, pairs: int, tile_keyed: bool) -> int:
    if tile_keyed:
        return tile * TILE_WORDS + pair * ROWS + row
    return (tile * ROWS + row) * pairs + pair


class Rank:
    def __init__(self, heap: Heap, rank: int, tile_keyed: bool = True, jitter: float = 0.0, seed: int = 0):
        self.heap, self.rank, self.tile_keyed = heap, rank, tile_keyed
        self.epochs: List[Dict[int, int]] = [dict(), dict()]
        self.calls = 0
        self.rng = random.Random(seed * 7919 + rank)
        self.jitter = jitter

    def _pause(self):
        if self.jitter:
            time.sleep(self.rng.random() * self.jitter)

    def all_reduce(self, partial: Sequence[Sequence[float]], features: int, timeout: float = 5.0) -> List[List[float]]:
        """``partial[token][feature]`` of this rank; returns the sum over ranks (every rank gets the same lists)."""
        tokens = len(partial)
        pairs = (tokens + 3) // 4  # token quads: one 16-byte word each
        half = self.calls & 1
        self.calls += 1
        tiles = (features + ROWS - 1) // ROWS
        flags = {}
        for t in range(tiles):
            flags[t] = self.epochs[half].get(t, 0) + 1
        # push: every word of every tile to every rank (own memory included), word by word
        words = [(t, r, p) for t in range(tiles) for r in range(min(ROWS, features - t * ROWS)) for p in range(pairs)]
        self.rng.shuffle(words)
        for n, (t, r, p) in enumerate(words):
            f = t * ROWS + r
            tok = [partial[4 * p + j][f] if 4 * p + j < tokens else 0.0 for j in range(4)]
            v0, v1 = (tok[0], tok[1]), (tok[2], tok[3])
            idx = _word_index(t, r, p, pairs, self.tile_keyed)
            for dest in range(self.heap.world):
                self.heap.mem[dest][half][self.rank][idx] = (v0, flags[t], v1, flags[t])
            if n % 64 == 0:
                self._pause()
        for t in range(tiles):
            self.epochs[half][t] = flags[t]
        # poll and reduce in rank order
        out = [[0.0] * features for _ in range(tokens)]
        deadline = time.monotonic() + timeout
        for (t, r, p) in sorted(words, key=lambda w: (-w[0], w[1], w[2])):  # (tiles are polled concurrently on the GPU; any order is legal)
            f = t * ROWS + r
            idx = _word_index(t, r, p, pairs, self.tile_keyed)
            for src in range(self.heap.world):
                while True:
                    w = self.heap.mem[self.rank][half][src].get(idx)
                    if w is not None and w[1] == flags[t] and w[3] == flags[t]:
                        break
                    if time.monotonic() > deadline:
                        raise TimeoutError(f"rank {self.rank}: word {idx} of rank {src} never arrived")
                    time.sleep(0)
                for j, value in enumerate(w[0] + w[2]):
                    if 4 * p + j < tokens:
                        out[4 * p + j][f] += value
        return out


def run_ranks(world: int, calls: Sequence[Tuple[int, int]], tile_keyed: bool = True, jitter: float = 0.0, seed: int = 0,
              late: Dict[Tuple[int, int], float] = None):
    """Runs ``calls`` = [(tokens, features), ...] on ``world`` threads.  Rank ``k`` contributes ``(k + 1) * (1 + call +
    token / 16 + feature / 4096)``; returns, per call, the largest absolute error of any rank's result.
    ``late[(rank, call)]`` = seconds that rank sleeps before it starts that call (a straggler)."""
    heap = Heap(world)
    errors: List[List[float]] = [[] for _ in range(world)]
    failures: List[BaseException] = []

    def value(rank, call, tok, feat):
        return (rank + 1) * (1.0 + call + tok / 16.0 + feat / 4096.0)

    def body(rank):
        me = Rank(heap, rank, tile_keyed, jitter, seed)
        try:
            for c, (tokens, features) in enumerate(calls):
                if late and (rank, c) in late:
                    time.sleep(late[(rank, c)])
                part = [[value(rank, c, t, f) for f in range(features)] for t in range(tokens)]
                got = me.all_reduce(part, features)
                scale = sum(r + 1 for r in range(world))
                worst = max(abs(got[t][f] - scale * (1.0 + c + t / 16.0 + f / 4096.0)) for t in range(tokens) for f in range(features))
                errors[rank].append(worst)
        except BaseException as e:  # surfaced to the caller
            failures.append(e)

    threads = [threading.Thread(target=body, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if failures:
        raise failures[0]
    return [max(errors[r][c] for r in range(world)) for c in range(len(calls))]


# ---------------------------------------------------------------------------------------------------
# barrier-free small all-reduce (``ll_allreduce_kernel`` in csrc/comm.cu)
# ---------------------------------------------------------------------------------------------------

SMALL_BLOCKS = 4    # the kernel's LL_BLOCKS (64 there): block b owns the words i with (i // SMALL_THREADS) % SMALL_BLOCKS == b
SMALL_THREADS = 8   # the kernel's COMM_THREADS (512 there)


class SmallAllReduceHeap:
    """``mem[dest][parity][src]`` maps a word index to ``(value, flag)`` (the kernel's word carries the flag twice)."""

    def __init__(self, world: int, parities: int = 2):
        self.world, self.parities = world, parities
        self.mem = [[[dict() for _ in range(world)] for _ in range(parities)] for _ in range(world)]


class SmallAllReduceRank:
    """One rank of the small all-reduce: per-block epochs that only grow, ``parities`` alternating areas (2 in the
    kernel; 1 shows why one is not enough), no barrier: a word is accepted when its flag equals the block's epoch."""

    def __init__(self, heap: SmallAllReduceHeap, rank: int, jitter: float = 0.0, seed: int = 0):
        self.heap, self.rank = heap, rank
        self.epochs = [0] * SMALL_BLOCKS
        self.rng = random.Random(seed * 104729 + rank)
        self.jitter = jitter

    def _pause(self):
        if self.jitter:
            time.sleep(self.rng.random() * self.jitter)

    def all_reduce(self, values: Sequence[float], timeout: float = 2.0, read_delay: float = 0.0) -> List[float]:
        words, world = len(values), self.heap.world
        blocks = min(SMALL_BLOCKS, -(-words // SMALL_THREADS))
        out = [0.0] * words
        order = list(range(blocks))
        self.rng.shuffle(order)  # blocks of one launch run in any order
        owned = {b: [i for i in range(words) if (i // SMALL_THREADS) % SMALL_BLOCKS == b] for b in order}
        flags = {}
        for b in order:  # every block first sends all its words ...
            self.epochs[b] += 1
            flags[b] = self.epochs[b]
            par = flags[b] % self.heap.parities
            for i in owned[b]:
                for dest in range(world):
                    self.heap.mem[dest][par][self.rank][i] = (values[i], flags[b])
                self._pause()
        if read_delay:
            time.sleep(read_delay)
        deadline = time.monotonic() + timeout
        for b in order:  # ... then sums what arrives, in rank order
            par = flags[b] % self.heap.parities
            for i in owned[b]:
                acc = 0.0
                for src in range(world):
                    while True:
                        w = self.heap.mem[self.rank][par][src].get(i)
                        if w is not None and w[1] == flags[b]:
                            break
                        if time.monotonic() > deadline:
                            raise TimeoutError(f"rank {self.rank}: word {i} of rank {src} never showed flag {flags[b]} (found {w})")
                        time.sleep(0)
                    acc += w[0]
                out[i] = acc
        return out


def run_small_all_reduce(world: int, sizes: Sequence[int], parities: int = 2, jitter: float = 0.0, seed: int = 0,
                         read_delay: Dict[Tuple[int, int], float] = None, timeout: float = 2.0):
    """``sizes`` = words per call.  Rank ``k`` contributes ``(k + 1) * (call + 1 + i / 1024)``; returns the largest absolute
    error per call.  ``read_delay[(rank, call)]``: seconds that rank waits between its sends and its reads."""
    heap = SmallAllReduceHeap(world, parities)
    errors: List[List[float]] = [[] for _ in range(world)]
    failures: List[BaseException] = []

    def body(rank):
        me = SmallAllReduceRank(heap, rank, jitter, seed)
        try:
            for c, words in enumerate(sizes):
                vals = [(rank + 1) * (c + 1 + i / 1024.0) for i in range(words)]
                got = me.all_reduce(vals, timeout=timeout, read_delay=(read_delay or {}).get((rank, c), 0.0))
                scale = sum(r + 1 for r in range(world))
                errors[rank].append(max(abs(got[i] - scale * (c + 1 + i / 1024.0)) for i in range(words)))
        except BaseException as e:
            failures.append(e)

    threads = [threading.Thread(target=body, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if failures:
        raise failures[0]
    return [max(errors[r][c] for r in range(world)) for c in range(len(sizes))]


# ---------------------------------------------------------------------------------------------------
# stream-K work decomposition (``WorkIter`` in csrc/gemm_sm100.cu), in the kernel's integer arithmetic
# ---------------------------------------------------------------------------------------------------


def stream_k_items(grid: int, tiles: int, k_blocks: int):
    """Per CTA, the list of work items ``(tile, kb0, kb1, ordinal, contributors)`` that the kernel's ``WorkIter`` yields
    in stream-K mode: the ``tiles * k_blocks`` units are dealt out as one contiguous range per CTA
    (``boundary(c) = c * units // grid``) and a range is cut at tile boundaries."""
    units = tiles * k_blocks

    def boundary(c):
        return c * units // grid

    def owner(unit):
        c = unit * grid // units
        while boundary(c + 1) <= unit:
            c += 1
        return c

    per_cta = []
    for cta in range(grid):
        u, u_end, items = boundary(cta), boundary(cta + 1), []
        while u < u_end:
            tile, kb0 = divmod(u, k_blocks)
            length = min(k_blocks - kb0, u_end - u)
            if length == k_blocks:
                ordinal, contributors = 0, 1
            else:
                first = owner(tile * k_blocks)
                ordinal, contributors = cta - first, owner(tile * k_blocks + k_blocks - 1) - first + 1
            items.append((tile, kb0, kb0 + length, ordinal, contributors))
            u += length
        per_cta.append(items)
    return per_cta


def stream_k_grid(tiles: int, kb64: int, sms: int = 148, max_contributors: int = 8):
    """The planner's choice (``tpb_gemm_plan`` with stream-K enabled): k-blocks per stage, grid size and the bound on the
    CTAs that share one tile; ``None`` when whole tiles are balanced already."""
    kbox = 4
    while kbox > 1 and tiles * ((kb64 + kbox - 1) // kbox) < 4 * sms:
        kbox >>= 1
    k_blocks = (kb64 + kbox - 1) // kbox
    units = tiles * k_blocks
    grid = min(sms, max(units // 2, 1))
    if tiles >= grid and tiles % grid == 0:
        return None
    while True:
        per = units // grid
        contributors = (k_blocks + per - 1) // per + 1
        if contributors <= max_contributors or grid == 1:
            return kbox, k_blocks, grid, max(contributors, 2)
        grid -= 1
