"""Replica-per-GPU batch sharding.  HYDRA's eval forward never mixes sequences (causal conv halo, value shift,
attention and the MoD top-k all stay inside one sequence; the reference pins "batched == solo" in
tests/test_ccgqa_model.py:146-167), so a batch is split by sequence across ranks, every rank holds a full
weight replica, and the only collective is a gather of results AFTER the forward."""
from __future__ import annotations

from typing import Optional, Tuple

import torch


def shard_bounds(n_rows: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous, balanced split of n_rows over `world` ranks: the first n_rows % world ranks get one extra row.
    Sequences are never split."""
    if world < 1 or not (0 <= rank < world) or n_rows < 0:
        raise ValueError(f"bad shard request n_rows={n_rows} rank={rank} world={world}")
    base, extra = divmod(n_rows, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_batch(ids: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Rows of a [B, S] id batch owned by `rank`."""
    a, b = shard_bounds(ids.shape[0], rank, world)
    return ids[a:b]


def gather_rows(local: torch.Tensor, n_rows_total: int, group=None) -> torch.Tensor:
    """All-gather per-rank results [b_r, ...] (b_r from shard_bounds) into [n_rows_total, ...] on every rank.
    Uneven shards are padded to the largest shard for the collective and trimmed afterwards."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    sizes = [shard_bounds(n_rows_total, r, world) for r in range(world)]
    biggest = max(b - a for a, b in sizes)
    pad = torch.zeros((biggest,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    pad[: local.shape[0]] = local
    out = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(out, pad, group=group)
    return torch.cat([o[: b - a] for o, (a, b) in zip(out, sizes)], dim=0)
