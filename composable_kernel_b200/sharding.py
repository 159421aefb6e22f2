"""Host-side work partitioning for one-process-per-GPU runs.  The contraction path has no exchange
step: grouped GEMMs shard by whole groups, the convolution by batch, single GEMMs run as replicas."""
from __future__ import annotations

from typing import List, Sequence, Tuple


def lpt_partition(weights: Sequence[float], parts: int) -> List[List[int]]:
    """Longest-processing-time greedy: indices of `weights` split into `parts` lists with balanced sums.
    Deterministic, so every rank computes the same assignment without communicating."""
    order = sorted(range(len(weights)), key=lambda i: (-weights[i], i))
    loads = [0.0] * parts
    out: List[List[int]] = [[] for _ in range(parts)]
    for i in order:
        j = loads.index(min(loads))
        out[j].append(i)
        loads[j] += weights[i]
    return [sorted(p) for p in out]


def batch_shard(n: int, rank: int, world: int) -> Tuple[int, int]:
    """[begin, end) of the batch owned by `rank`; remainders go to the first ranks."""
    base, rem = divmod(n, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def grouped_gemm_shard(ms: Sequence[int], rank: int, world: int) -> List[int]:
    """Groups (by index) of a grouped GEMM with equal N and K owned by `rank`: FLOPs are proportional to M_g."""
    return lpt_partition(list(ms), world)[rank]
