"""How the KDA path is partitioned over the GPUs of one node.

Every (sequence, head) recurrence is independent in forward and backward, so the operator shards with no
data-path collective: heads first (every rank sees all sequences, which balances ragged packed batches), and
sequences (longest first, greedy) only when there are fewer heads than ranks.  Decode shards the batch.
"""

from __future__ import annotations

from typing import List, Sequence, Tuple


def head_shard(heads: int, world: int, rank: int) -> Tuple[int, int]:
    """[begin, end) of the heads owned by `rank`; requires world <= heads (remainder goes to the low ranks)."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("invalid world / rank")
    if world > heads:
        raise ValueError("more ranks than heads: shard sequences instead")
    base, rem = divmod(heads, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def sequence_shard(lengths: Sequence[int], world: int) -> List[List[int]]:
    """Greedy longest-first assignment of sequence indices to ranks (balanced total tokens)."""
    loads = [0] * world
    out: List[List[int]] = [[] for _ in range(world)]
    for idx in sorted(range(len(lengths)), key=lambda i: (-lengths[i], i)):
        r = min(range(world), key=lambda j: (loads[j], j))
        out[r].append(idx)
        loads[r] += lengths[idx]
    return [sorted(x) for x in out]


def batch_shard(batch: int, world: int, rank: int) -> Tuple[int, int]:
    """[begin, end) of the decode batch rows owned by `rank`."""
    base, rem = divmod(batch, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)
