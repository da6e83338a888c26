"""Sequence bin-packing used to form token-balanced micro-batches and DP shards.

Three algorithms with the behaviour of the reference's ``areal/utils/seqpack.py``:

* ``ffd_allocate``  (:234) first-fit-decreasing into bins of a token capacity, with a
  minimum number of bins;
* ``kk_allocate``   (:446) Karmarkar-Karp largest-differencing into exactly ``k`` balanced
  groups;
* ``balanced_greedy_partition`` (:540) longest-processing-time greedy into ``k`` groups
  with (optionally) equal item counts.

The implementations are written from the algorithm descriptions (heap-based), not from the
reference source.
"""
from __future__ import annotations

import heapq
from typing import Sequence

import numpy as np


def ffd_allocate(sizes: Sequence[int], capacity: int, min_groups: int = 1) -> list[list[int]]:
    """First-fit-decreasing. Returns groups of indices; every group's total is <= capacity
    (an item larger than the capacity gets a bin of its own). At least ``min_groups`` bins
    are returned when there are enough items (the largest bins are split)."""
    n = len(sizes)
    order = sorted(range(n), key=lambda i: -int(sizes[i]))
    bins: list[list[int]] = []
    loads: list[int] = []
    for i in order:
        s = int(sizes[i])
        placed = False
        for b in range(len(bins)):
            if loads[b] + s <= capacity:
                bins[b].append(i)
                loads[b] += s
                placed = True
                break
        if not placed:
            bins.append([i])
            loads.append(s)
    # honour min_groups by repeatedly splitting the heaviest multi-item bin
    while len(bins) < min(min_groups, n):
        cand = max((b for b in range(len(bins)) if len(bins[b]) > 1), key=lambda b: loads[b], default=None)
        if cand is None:
            break
        items = sorted(bins[cand], key=lambda i: -int(sizes[i]))
        a, c = [], []
        la = lc = 0
        for i in items:
            if la <= lc:
                a.append(i)
                la += int(sizes[i])
            else:
                c.append(i)
                lc += int(sizes[i])
        bins[cand], loads[cand] = a, la
        bins.append(c)
        loads.append(lc)
    for b in bins:
        b.sort()
    return bins


def kk_allocate(sizes: Sequence[int], k: int, equal_size: bool = False) -> list[list[int]]:
    """Karmarkar-Karp (largest differencing) k-way partition. Returns ``k`` index groups
    whose sums are as even as the heuristic gets. ``equal_size`` pads the item list so that
    every group receives the same number of items (needs ``len(sizes) % k == 0``)."""
    n = len(sizes)
    if k <= 0:
        raise ValueError("k must be positive")
    if equal_size and n % k != 0:
        raise ValueError("equal_size needs len(sizes) divisible by k")
    if n == 0:
        return [[] for _ in range(k)]

    # A state is a list of k (sum, items) sets sorted by sum descending. The heap is keyed by
    # the spread (max - min); merging two states pairs the largest set of one with the
    # smallest of the other.
    def make_state(idx):
        sets = [(int(sizes[idx]), [idx])] + [(0, []) for _ in range(k - 1)]
        return sets

    order = sorted(range(n), key=lambda i: -int(sizes[i]))
    counter = 0
    heap = []
    if equal_size:
        # process k items at a time so each group grows by exactly one item per round
        for r in range(0, n, k):
            chunk = order[r:r + k]
            sets = sorted(((int(sizes[i]), [i]) for i in chunk), key=lambda t: -t[0])
            heapq.heappush(heap, (-(sets[0][0] - sets[-1][0]), counter, sets))
            counter += 1
    else:
        for i in order:
            sets = make_state(i)
            heapq.heappush(heap, (-(sets[0][0] - sets[-1][0]), counter, sets))
            counter += 1
    while len(heap) > 1:
        _, _, a = heapq.heappop(heap)
        _, _, b = heapq.heappop(heap)
        merged = [(a[j][0] + b[k - 1 - j][0], a[j][1] + b[k - 1 - j][1]) for j in range(k)]
        merged.sort(key=lambda t: -t[0])
        heapq.heappush(heap, (-(merged[0][0] - merged[-1][0]), counter, merged))
        counter += 1
    final = heap[0][2]
    groups = [sorted(items) for _, items in final]
    return groups


def balanced_greedy_partition(sizes: Sequence[int], k: int, equal_count: bool = True) -> list[list[int]]:
    """Longest-processing-time greedy into ``k`` groups. With ``equal_count`` each group
    gets ``len(sizes) // k`` items (+1 for the first ``len % k`` groups to fill up)."""
    n = len(sizes)
    if k <= 0:
        raise ValueError("k must be positive")
    order = sorted(range(n), key=lambda i: -int(sizes[i]))
    groups: list[list[int]] = [[] for _ in range(k)]
    loads = [0] * k
    if equal_count:
        base, extra = divmod(n, k)
        quota = [base + (1 if g < extra else 0) for g in range(k)]
    else:
        quota = [n] * k
    for i in order:
        cand = [g for g in range(k) if len(groups[g]) < quota[g]]
        g = min(cand, key=lambda g: (loads[g], g))
        groups[g].append(i)
        loads[g] += int(sizes[i])
    for g in groups:
        g.sort()
    return groups


def get_allocate_fn(name: str):
    if name == "ffd":
        return ffd_allocate
    if name == "kk":
        return lambda sizes, capacity, min_groups=1: _kk_with_capacity(sizes, capacity, min_groups)
    raise ValueError(f"unknown packing algorithm {name}")


def _kk_with_capacity(sizes, capacity: int, min_groups: int) -> list[list[int]]:
    """KK into the smallest k >= min_groups whose heaviest group fits the capacity."""
    n = len(sizes)
    total = int(np.sum(sizes)) if n else 0
    k = max(min_groups, -(-total // max(capacity, 1)), 1)
    while True:
        groups = [g for g in kk_allocate(sizes, k) if g]
        if all(sum(int(sizes[i]) for i in g) <= capacity or len(g) == 1 for g in groups) or k >= n:
            return groups
        k += 1


def reorder_to_balanced_batches(seqlens: Sequence[int], n_seqs_per_batch: int) -> list[int]:
    """Order of samples such that consecutive batches of ``n_seqs_per_batch`` have similar
    token totals (long and short sequences interleaved)."""
    n = len(seqlens)
    k = max(1, n // max(1, n_seqs_per_batch))
    groups = balanced_greedy_partition(seqlens, k, equal_count=True)
    return [i for g in groups for i in g]
