"""Host-side partitioning of the hot path across the GPUs of one box (one process per GPU).

Every unit of the path is independent, so there is no data-path collective:
  * elementwise / norm / converter ops shard contiguous blocks of token rows (RMSNorm reduces inside a row only);
  * paged decode attention shards whole sequences — their KV pages live on the owning GPU — balanced by context length;
  * prefill attention shards (batch item, KV head) units: the query heads of a KV-head group travel together.
Only when a consumer needs the gathered output (config 5) do the ranks all-gather it over NCCL.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple


def row_shard(total_rows: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous [start, end) block of rows for `rank`; the first `total_rows % world` ranks get one extra row."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    base, extra = divmod(total_rows, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def modulation_rows(start: int, end: int, rows_per_batch: int) -> Tuple[int, int, int]:
    """For a row block [start, end) of a [B*rows_per_batch, C] tensor: (first batch item, number of batch items, and the
    rowsPerBatch to pass to the kernel).  A block must either cover whole batch items or stay inside one."""
    if end <= start:
        return 0, 0, rows_per_batch
    first, last = start // rows_per_batch, (end - 1) // rows_per_batch
    if first == last:
        return first, 1, end - start  # inside one batch item: every local row uses that item's modulation row
    if start % rows_per_batch or end % rows_per_batch:
        raise ValueError("a row block spanning several batch items must start and end on item boundaries")
    return first, last - first + 1, rows_per_batch


def lpt_assign(costs: Sequence[int], world: int) -> List[List[int]]:
    """Assignment of sequences (cost = context length) to ranks: longest-processing-time-first, then refined by exchanges.

    Returns, per rank, the indices it owns (in ascending index order).  A uniform split of U[512, 32768] contexts can be
    ~2x imbalanced; LPT keeps the maximum within 4/3 of optimal (1.3 % over the mean for the 64 seeded sequences on 8
    ranks).  The refinement then repeats, while it helps: take the heaviest rank and either move one of its sequences to
    another rank or exchange one with a sequence of another rank, whichever lowers the heavier of the two loads most.  It is
    deterministic (ties by index) and ends: every step strictly lowers the sorted vector of loads."""
    cost = [int(c) for c in costs]
    loads = [0] * world
    owned: List[List[int]] = [[] for _ in range(world)]
    for idx in sorted(range(len(cost)), key=lambda i: (-cost[i], i)):
        r = min(range(world), key=lambda k: (loads[k], k))
        loads[r] += cost[idx]
        owned[r].append(idx)
    for _ in range(16 * max(1, len(cost))):  # far more steps than ever taken; a guard, not a tuning knob
        heavy = max(range(world), key=lambda k: (loads[k], -k))
        best = None  # (new pair maximum, other rank, index given, index taken or -1)
        for other in range(world):
            if other == heavy:
                continue
            for give in owned[heavy]:
                for take in [-1] + owned[other]:
                    delta = cost[give] - (cost[take] if take >= 0 else 0)
                    if delta <= 0:
                        continue
                    pair_max = max(loads[heavy] - delta, loads[other] + delta)
                    if pair_max < loads[heavy] and (best is None or (pair_max, other, give, take) < best):
                        best = (pair_max, other, give, take)
        if best is None:
            break
        _, other, give, take = best
        owned[heavy].remove(give)
        owned[other].append(give)
        loads[heavy] -= cost[give]
        loads[other] += cost[give]
        if take >= 0:
            owned[other].remove(take)
            owned[heavy].append(take)
            loads[other] -= cost[take]
            loads[heavy] += cost[take]
    return [sorted(o) for o in owned]


def prefill_units(batch: int, kv_heads: int, world: int, rank: int) -> List[Tuple[int, int]]:
    """(batch item, KV head) units of equal cost, dealt round-robin: unit u -> rank u % world."""
    return [(u // kv_heads, u % kv_heads) for u in range(batch * kv_heads) if u % world == rank]
