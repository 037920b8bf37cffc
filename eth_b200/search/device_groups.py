"""Device placement: which nodes form which pipeline, in which order, and what that can yield at most.

Reference: eth/searching/device_groups.py -- stage-size enumeration (:73-136), contiguous splits of
the node list into k pipelines (:363-388) sorted by a TFLOPS-variance loss (:292-339), node-order
permutations so that "contiguous" covers every assignment of node types to pipelines (:527-637),
and an upper bound on a group's throughput from groups that dominate it device by device
(bipartite matching, :197-286).
"""
from __future__ import annotations

import itertools
from typing import Dict, Iterator, List, Sequence, Tuple


def compositions_pow2(total: int, parts: int, max_part: int) -> List[Tuple[int, ...]]:
    """Ordered ways to write `total` as a sum of `parts` powers of two (each <= max_part)."""
    sizes = [s for s in (1, 2, 4, 8, 16, 32, 64) if s <= max_part]
    out: List[Tuple[int, ...]] = []

    def rec(left: int, k: int, acc: Tuple[int, ...]):
        if k == 0:
            if left == 0:
                out.append(acc)
            return
        if left < k or left > k * max(sizes):
            return
        for s in sizes:
            if s <= left:
                rec(left - s, k - 1, acc + (s,))

    rec(total, parts, ())
    return out


def contiguous_splits(n: int, k: int) -> Iterator[List[Tuple[int, int]]]:
    for cuts in itertools.combinations(range(1, n), k - 1):
        yield [(a, b) for a, b in zip((0,) + cuts, cuts + (n,))]


def imbalance_loss(groups, tflops_of_node) -> float:
    """Variance of the pipelines' TFLOPS (balanced splits are tried first)."""
    sums = [sum(tflops_of_node[i] for i in range(a, b)) for a, b in groups]
    mean = sum(sums) / len(sums)
    return sum((s - mean) ** 2 for s in sums) / len(sums)


def node_orders(nodes: Sequence[dict], limit: int = 24) -> List[Tuple[int, ...]]:
    """Orderings of the node list that differ as sequences of (GPU type, GPU count): with
    contiguous splits on top, every way of dealing node kinds to pipelines and to positions inside
    a pipeline is reached. Nodes of one kind are interchangeable, so only distinct kind sequences
    are kept (at most `limit`, the given order first)."""
    kinds = [(n["GPU"], n["GPU_NUM"]) for n in nodes]
    if len(set(kinds)) <= 1:
        return [tuple(range(len(nodes)))]
    seen, out = set(), []
    by_kind: Dict[tuple, List[int]] = {}
    for i, k in enumerate(kinds):
        by_kind.setdefault(k, []).append(i)
    for perm in _distinct_permutations(kinds):
        if perm in seen:
            continue
        seen.add(perm)
        pools = {k: list(v) for k, v in by_kind.items()}
        out.append(tuple(pools[k].pop(0) for k in perm))
        if len(out) >= limit:
            break
    identity = tuple(range(len(nodes)))
    if identity in out:
        out.remove(identity)
    return [identity] + out


def _distinct_permutations(items: Sequence) -> Iterator[tuple]:
    """Permutations of a multiset in lexicographic order, each once."""
    a = sorted(items)
    n = len(a)
    while True:
        yield tuple(a)
        i = n - 2
        while i >= 0 and a[i] >= a[i + 1]:
            i -= 1
        if i < 0:
            return
        j = n - 1
        while a[j] <= a[i]:
            j -= 1
        a[i], a[j] = a[j], a[i]
        a[i + 1:] = reversed(a[i + 1:])


# ------------------------------------------------------------------------------------------
# domination bound
# ------------------------------------------------------------------------------------------
def dominates(big: Sequence[Tuple[float, float]], small: Sequence[Tuple[float, float]]) -> bool:
    """True if every device of `small` can be paired with its own device of `big` that is at least
    as fast and has at least as much memory ((tflops, memory) pairs). Then anything `small` can run,
    `big` can run at least as fast, so a known throughput of `big` bounds `small` from above."""
    if len(small) > len(big):
        return False
    covers = [[j for j, (f, m) in enumerate(big) if f >= sf and m >= sm] for sf, sm in small]
    match: Dict[int, int] = {}

    def place(i, banned):
        for j in covers[i]:
            if j in banned:
                continue
            banned.add(j)
            if j not in match or place(match[j], banned):
                match[j] = i
                return True
        return False

    return all(place(i, set()) for i in range(len(small)))


class ThroughputBounds:
    """Known best rates (samples / us) per device group, and bounds derived from them."""

    def __init__(self, tflops: Dict[str, float], memory: Dict[str, float]):
        self.tflops, self.memory = tflops, memory
        self.known: Dict[Tuple[str, ...], float] = {}

    def _devices(self, group: Tuple[str, ...]):
        return [(self.tflops[t], self.memory[t]) for t in group]

    def record(self, group: Tuple[str, ...], rate: float) -> None:
        self.known[tuple(group)] = max(rate, self.known.get(tuple(group), 0.0))

    def upper_bound(self, group: Tuple[str, ...]) -> float:
        """Smallest known rate among groups that dominate `group` (inf if none is known). A group
        that is merely as large in total TFLOPS is bounded by the TFLOPS ratio as a fallback."""
        group = tuple(group)
        if group in self.known:
            return self.known[group]
        mine = self._devices(group)
        bound = float("inf")
        for other, rate in self.known.items():
            if len(other) >= len(group) and dominates(self._devices(other), mine):
                bound = min(bound, rate)
        return bound
