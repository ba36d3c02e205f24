"""Work partitioning across the GPUs of one node.  The op is independent per (sequence, v-head), so
every split below needs no collective on the data path: v-head groups (with the k-heads they share),
whole sequences (token balanced) or batch rows."""
from __future__ import annotations

from typing import List, Sequence, Tuple


def head_shard(num_k_heads: int, num_v_heads: int, world: int, rank: int) -> Tuple[slice, slice]:
    """Contiguous k-head / v-head slices of rank `rank`; every rank keeps whole GQA groups."""
    if num_k_heads % world != 0:
        raise ValueError(f"num_k_heads={num_k_heads} is not divisible by world size {world}")
    hk = num_k_heads // world
    hv = num_v_heads // world
    return slice(rank * hk, (rank + 1) * hk), slice(rank * hv, (rank + 1) * hv)


def balance_sequences(lengths: Sequence[int], world: int) -> List[List[int]]:
    """Greedy longest-first assignment of sequences to ranks, balancing tokens.  Returns the list of
    sequence indices of every rank (each in increasing index order)."""
    loads = [0] * world
    out: List[List[int]] = [[] for _ in range(world)]
    for i in sorted(range(len(lengths)), key=lambda j: (-lengths[j], j)):
        r = min(range(world), key=lambda j: (loads[j], j))
        out[r].append(i)
        loads[r] += lengths[i]
    return [sorted(x) for x in out]


def batch_shard(batch: int, world: int, rank: int) -> slice:
    """Rows of a [B, ...] batch owned by `rank` (first ranks take the remainder)."""
    base, rem = divmod(batch, world)
    lo = rank * base + min(rank, rem)
    return slice(lo, lo + base + (1 if rank < rem else 0))
