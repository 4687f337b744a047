"""Token-count balancing of variable-length samples: Karmarkar-Karp (largest differencing) k-way partitioning, a
greedy fallback, and the first-fit estimate of how many micro-batches a token budget requires.

Same entry points as the reference (openrlhf/utils/seqlen_balancing.py:24-247); implementation is this project's own.
"""
from __future__ import annotations

import heapq
from typing import List


def karmarkar_karp(seqlen_list: List[int], k_partitions: int, equal_size: bool) -> List[List[int]]:
    """Largest-differencing method generalised to k parts.

    State: a heap of "k-tuples of partial sets" ordered by spread (largest sum minus smallest sum). Repeatedly merge
    the two tuples with the largest spread, pairing the heaviest set of one with the lightest of the other.
    With ``equal_size`` the items are first grouped into chunks of k (sorted), which keeps set sizes identical.
    """
    k = k_partitions
    n = len(seqlen_list)
    order = sorted(range(n), key=lambda i: (seqlen_list[i], i))

    def make_state(items):
        # items: list of (length, index) with at most k entries -> k sets sorted by descending sum
        sets = [([idx], ln) for ln, idx in items] + [([], 0)] * (k - len(items))
        sets.sort(key=lambda s: -s[1])
        return sets

    heap = []
    counter = 0
    if equal_size:
        if n % k != 0:
            raise AssertionError(f"{n} items cannot be split into {k} partitions of equal size")
        for s in range(0, n, k):
            st = make_state([(seqlen_list[i], i) for i in order[s:s + k]])
            heapq.heappush(heap, (-(st[0][1] - st[-1][1]), counter, st))
            counter += 1
    else:
        for i in order:
            st = make_state([(seqlen_list[i], i)])
            heapq.heappush(heap, (-(st[0][1] - st[-1][1]), counter, st))
            counter += 1
    while len(heap) > 1:
        _, _, a = heapq.heappop(heap)
        _, _, b = heapq.heappop(heap)
        merged = [(a[j][0] + b[k - 1 - j][0], a[j][1] + b[k - 1 - j][1]) for j in range(k)]
        merged.sort(key=lambda s: -s[1])
        heapq.heappush(heap, (-(merged[0][1] - merged[-1][1]), counter, merged))
        counter += 1
    final = heap[0][2] if heap else [([], 0)] * k
    parts = [list(s[0]) for s in final]
    if equal_size:
        assert all(len(p) == n // k for p in parts)
    return parts


def greedy_partition(seqlen_list: List[int], k_partitions: int, equal_size: bool) -> List[List[int]]:
    """Longest-first assignment to the currently lightest partition."""
    bias = sum(seqlen_list) + 1 if equal_size else 0
    parts: List[List[int]] = [[] for _ in range(k_partitions)]
    loads = [0] * k_partitions
    for i in sorted(range(len(seqlen_list)), key=lambda i: -seqlen_list[i]):
        j = min(range(k_partitions), key=lambda p: loads[p])
        parts[j].append(i)
        loads[j] += seqlen_list[i] + bias
    return parts


def get_seqlen_balanced_partitions(seqlen_list: List[int], k_partitions: int, equal_size: bool) -> List[List[int]]:
    """Indices of `seqlen_list` split into k non-empty partitions of near-equal token count (each sorted)."""
    if len(seqlen_list) < k_partitions:
        raise AssertionError(f"number of items {len(seqlen_list)} < number of partitions {k_partitions}")
    parts = karmarkar_karp(seqlen_list, k_partitions, equal_size)
    seen = sorted(i for p in parts for i in p)
    assert seen == list(range(len(seqlen_list))), "partitioning lost or duplicated an item"
    if any(len(p) == 0 for p in parts):
        parts = greedy_partition(seqlen_list, k_partitions, equal_size)
    return [sorted(p) for p in parts]


def log_seqlen_unbalance(seqlen_list: List[int], partitions: List[List[int]], prefix: str) -> dict:
    k = len(partitions)
    n = len(seqlen_list)
    per = n // k
    naive = [sum(seqlen_list[i * per:(i + 1) * per]) for i in range(k)]
    bal = [sum(seqlen_list[i] for i in p) for p in partitions]
    return {f"{prefix}/min": min(naive), f"{prefix}/max": max(naive), f"{prefix}/minmax_diff": max(naive) - min(naive),
            f"{prefix}/balanced_min": min(bal), f"{prefix}/balanced_max": max(bal),
            f"{prefix}/mean": sum(seqlen_list) / max(k, 1)}


def ceildiv(a: int, b: int) -> int:
    return -(a // -b)


def get_reverse_idx(idx_map: List[int]) -> List[int]:
    rev = [0] * len(idx_map)
    for new, old in enumerate(idx_map):
        rev[old] = new
    return rev


def get_minimum_num_micro_batch_size(total_lengths: List[int], max_tokens_per_gpu: int, ring_attn_size: int,
                                     ds_tensor_parallel_size: int) -> int:
    """First-fit count of micro-batches needed so none exceeds the token budget; the budget of one model replica is
    max_tokens_per_gpu x ring_attn_size x tensor_parallel_size."""
    budget = max_tokens_per_gpu * ring_attn_size * ds_tensor_parallel_size
    bins: List[int] = []
    for ln in total_lengths:
        for j, used in enumerate(bins):
            if used + ln <= budget:
                bins[j] = used + ln
                break
        else:
            bins.append(ln)
    return len(bins)
