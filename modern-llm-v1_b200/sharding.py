"""Partition of an attention problem over the GPUs of one box.

The unit of work is one (batch, KV head): it reads Q of the group's query heads and K, V
of that KV head, and writes O, dQ of those query heads and dK, dV of that KV head — the
group sum of dK/dV (llm/src/model/attention.cu:412-429) stays inside the unit.  Units
therefore never exchange data, in forward or backward; ranks only meet to gather
results or checksums for verification.
"""
from __future__ import annotations


def unit_range(n_units: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous block [lo, hi) of units owned by `rank`; sizes differ by at most one."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("rank must satisfy 0 <= rank < world")
    if n_units < 0:
        raise ValueError("n_units must be >= 0")
    base, rem = divmod(n_units, world)
    lo = rank * base + min(rank, rem)
    hi = lo + base + (1 if rank < rem else 0)
    return lo, hi


def unit_to_batch_head(unit: int, Hkv: int) -> tuple[int, int]:
    """Unit index -> (batch, KV head); units are numbered b * Hkv + h_kv."""
    return divmod(unit, Hkv)


def query_heads_of_unit(unit: int, Hq: int, Hkv: int) -> range:
    """Query heads served by the unit's KV head: consecutive heads share a KV head."""
    g = Hq // Hkv
    hk = unit % Hkv
    return range(hk * g, hk * g + g)


def gather_units(local, n_units: int, rank: int, world: int):
    """All-gathers per-unit results (leading axis = this rank's units, in unit order) into
    the full [n_units, ...] tensor on every rank.  Verification only: the data path of
    attention needs no collective.  Uses the default torch.distributed group (NCCL on GPUs,
    gloo on CPUs); shards of unequal size are padded to the largest and trimmed."""
    import torch
    import torch.distributed as dist

    sizes = [hi - lo for lo, hi in (unit_range(n_units, r, world) for r in range(world))]
    if local.shape[0] != sizes[rank]:
        raise ValueError("local tensor does not hold this rank's units")
    if world == 1:
        return local
    big = max(sizes)
    pad = local
    if local.shape[0] < big:
        pad = torch.cat([local, local.new_zeros((big - local.shape[0],) + tuple(local.shape[1:]))])
    parts = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(parts, pad.contiguous())
    return torch.cat([p[:n] for p, n in zip(parts, sizes)])
