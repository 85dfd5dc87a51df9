"""Batch sharding of the decode path across the GPUs of one node.

Every (batch row, KV head) is independent on this path, so a rank owns a contiguous block of
batch rows with its own cache pools and runs append and attention locally; the only exchange is
the gather of the attention outputs (one ``all_gather_into_tensor`` per step over NCCL/NVLink).
"""

from __future__ import annotations

from typing import Tuple

import torch
import torch.distributed as dist


def shard_rows(batch: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Half-open range of batch rows owned by ``rank``; the batch must divide evenly."""

    if world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError("rank must be in [0, world_size)")
    if batch % world_size:
        raise ValueError(f"batch {batch} does not divide evenly over {world_size} ranks")
    per_rank = batch // world_size
    return rank * per_rank, (rank + 1) * per_rank


def gather_outputs(local: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """All-gather per-rank outputs ``[B/N, ...]`` into ``[B, ...]`` in rank order (identity for one rank)."""

    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size() == 1:
        return local
    world = dist.get_world_size()
    if out is None:
        out = torch.empty((world * local.shape[0], *local.shape[1:]), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out, local.contiguous())
    return out
