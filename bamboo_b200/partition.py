"""Layer -> stage partitioning and the redundancy (shadow) map.

Must give the same answers as the reference for the same inputs:
``partition_uniform`` / ``partition_balanced`` (deepspeed/runtime/utils.py:470-551) and
``get_redundant_stage_ids`` / ``get_redundant_user_stage_ids``
(deepspeed/runtime/pipe/redundancy.py:7-31).

``partition_balanced`` here is a bisection on the bottleneck weight with a greedy
feasibility sweep over the prefix sums, like the reference, and reproduces its tie-breaking
(boundaries are pushed as far right as the current bottleneck allows).
"""
from bisect import bisect_left
from itertools import accumulate
from typing import List, Sequence, Tuple


def partition_uniform(num_items: int, num_parts: int) -> List[int]:
    """Boundaries ``parts[0..num_parts]`` of equally sized contiguous chunks; the last chunk
    absorbs the remainder."""
    if num_items <= num_parts:
        return [min(p, num_items) for p in range(num_parts + 1)]
    chunk = num_items // num_parts
    return [min(chunk * p, num_items) for p in range(num_parts)] + [num_items]


def _sweep(prefix: Sequence[float], num_parts: int, bottleneck: float) -> Tuple[List[int], bool]:
    """Greedy left-to-right packing: every part takes items while its weight stays below
    ``bottleneck``.  Returns the boundaries and whether the packing fits."""
    n = len(prefix)
    parts = [0] + [n] * num_parts
    target = bottleneck
    chunk = n // num_parts
    probe = chunk
    for p in range(1, num_parts):
        while probe < n and prefix[probe] < target:
            probe += chunk
        parts[p] = bisect_left(prefix, target, lo=probe - chunk, hi=min(probe, n))
        if parts[p] == n:
            return parts, (prefix[-1] - prefix[parts[p - 1]]) < bottleneck
        target = prefix[parts[p] - 1] + bottleneck
    return parts, target >= prefix[-1]


def partition_balanced(weights: Sequence[float], num_parts: int, eps: float = 1e-3) -> List[int]:
    """Contiguous partition minimising the heaviest part (to within ``eps``)."""
    n = len(weights)
    if n <= num_parts:
        return partition_uniform(n, num_parts)
    prefix = list(accumulate(weights))
    lo, hi = prefix[-1] / num_parts, prefix[-1]
    while hi > lo + eps:
        mid = lo + (hi - lo) / 2
        if _sweep(prefix, num_parts, mid)[1]:
            hi = mid
        else:
            lo = mid + eps
    parts, ok = _sweep(prefix, num_parts, hi)
    assert ok
    return parts


def get_redundant_stage_ids(redundant_level: int, stage_id: int, num_stages: int) -> List[int]:
    """Stages whose weights ``stage_id`` shadows: the next ``redundant_level`` stages, cyclically."""
    return [(stage_id + k) % num_stages for k in range(1, redundant_level + 1)]


def get_redundant_user_stage_ids(redundant_level: int, stage_id: int, num_stages: int) -> List[int]:
    """Stages that hold a shadow copy of ``stage_id``."""
    return [s for s in range(num_stages)
            if stage_id in get_redundant_stage_ids(redundant_level, s, num_stages)]
