"""Sharding of the decode path across the GPUs of one node, by batch row and KV head.

Every (batch row, KV head) is independent on this path, so a rank owns a rectangle of batch rows x KV
heads with its own cache pools and runs append and attention locally; the only exchange is the gather of
the attention outputs (one all-gather per step over NCCL/NVLink).  The partition rule itself lives in the
C library (``dartkv_shard_range``) so that non-Python hosts split the work the same way: the batch is split
first, unevenly if it must be (the first groups hold one row more); KV heads are split as well only when there
are more ranks than batch rows.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from ._lib import LIB, Shard as _CShard, check


@dataclass(frozen=True)
class Shard:
    """What one rank owns: batch rows ``[row_begin, row_end)`` x KV heads ``[head_begin, head_end)``."""

    row_begin: int
    row_end: int
    head_begin: int
    head_end: int
    batch_groups: int
    head_groups: int
    rows_padded: int

    @property
    def rows(self) -> int:
        return self.row_end - self.row_begin

    @property
    def heads(self) -> int:
        return self.head_end - self.head_begin

    def query_heads(self, total_query_heads: int, kv_heads: int) -> Tuple[int, int]:
        """Half-open range of query heads that attend to this shard's KV heads (GQA by contiguous groups)."""

        rep = total_query_heads // kv_heads
        return self.head_begin * rep, self.head_end * rep


def shard_plan(batch: int, kv_heads: int, world_size: int, rank: int) -> Shard:
    """The rectangle of (batch rows, KV heads) owned by ``rank``; raises ``ValueError`` if it cannot be split."""

    c = _CShard()
    check(LIB.dartkv_shard_range(int(batch), int(kv_heads), int(world_size), int(rank), ctypes.byref(c)))
    return Shard(c.row_begin, c.row_end, c.head_begin, c.head_end, c.batch_groups, c.head_groups, c.rows_padded)


def shard_rows(batch: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Half-open range of batch rows owned by ``rank`` when only the batch is split (``batch >= world_size``)."""

    if world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError("rank must be in [0, world_size)")
    if batch < world_size:
        raise ValueError(f"batch {batch} has fewer rows than {world_size} ranks: use shard_plan to split KV heads too")
    plan = shard_plan(batch, 1, world_size, rank)
    return plan.row_begin, plan.row_end


def gather_outputs(local: torch.Tensor, out: Optional[torch.Tensor] = None, *, shard: Optional[Shard] = None,
                   batch: Optional[int] = None, kv_heads: Optional[int] = None) -> torch.Tensor:
    """All-gather per-rank attention outputs into the full ``[B, Hq, ...]`` tensor (identity for one rank).

    Without ``shard`` every rank holds the same number of batch rows and all heads: the result is the
    concatenation in rank order (``out`` may be passed to receive it).  With ``shard`` (plus the global
    ``batch`` and ``kv_heads``) ``local`` is ``[rows, Hq_local, ...]`` of that rectangle; ranks may hold
    different row counts and different head groups, and the pieces are placed at their global position.
    """

    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size() == 1:
        return local
    world = dist.get_world_size()
    even = shard is None or (shard.head_groups == 1 and shard.rows_padded * shard.batch_groups == batch)
    if even:
        if out is None:
            out = torch.empty((world * local.shape[0], *local.shape[1:]), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(out, local.contiguous())
        return out
    if batch is None or kv_heads is None:
        raise ValueError("gather_outputs with a shard needs the global batch and kv_heads")
    padded = local.new_zeros((shard.rows_padded, *local.shape[1:]))
    padded[: local.shape[0]].copy_(local)
    flat = local.new_empty((world * shard.rows_padded, *local.shape[1:]))
    dist.all_gather_into_tensor(flat, padded)
    pieces = flat.view(world, *padded.shape)
    heads_local = local.shape[1]
    if out is None:
        out = local.new_empty((batch, heads_local * shard.head_groups, *local.shape[2:]))
    for r in range(world):
        peer = shard_plan(batch, kv_heads, world, r)
        h0 = (r % shard.head_groups) * heads_local
        out[peer.row_begin:peer.row_end, h0:h0 + heads_local].copy_(pieces[r, : peer.rows])
    return out


class PeerGather:
    """Gathered attention outputs delivered by the decode kernels themselves instead of an all-gather.

    Every rank allocates two gathered tensors ``[batch, query_heads, head_dim]`` and a flag array in symmetric
    memory (``torch.distributed._symmetric_memory``: each rank's allocation is mapped into every other rank of the
    node).  ``decode_attention(..., peer_gather=self)`` then makes the kernel that normalizes the output rows store
    them into all ranks' gathered tensors over NVLink, publish an arrival flag per peer and wait (bounded) for the
    peers' flags; the call returns this rank's gathered tensor for the step.  Two tensors alternate because a rank
    may run one step ahead of its slowest peer.  All ranks must make the same sequence of calls.
    """

    def __init__(self, shard: Shard, batch: int, query_heads: int, kv_heads: int, head_dim: int, dtype: torch.dtype,
                 device: torch.device, group=None) -> None:
        import os

        # plain peer mappings are all this needs: do not bind the allocations to an NVLink multicast object
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        from ._lib import MAX_PEERS, PeerScatter

        group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > MAX_PEERS:
            raise ValueError(f"at most {MAX_PEERS} ranks (one node) can exchange outputs this way")
        self.shard = shard
        self.gathered = [symm_mem.empty((batch, query_heads, head_dim), dtype=dtype, device=device) for _ in range(2)]
        self.flags = symm_mem.empty((max(self.world, 4),), dtype=torch.int32, device=device)
        self.flags.zero_()
        handles = [symm_mem.rendezvous(t, group) for t in self.gathered]
        flag_handle = symm_mem.rendezvous(self.flags, group)
        self._handles = handles + [flag_handle]   # keep the mappings alive
        q_lo, _ = shard.query_heads(query_heads, kv_heads)
        self._structs = []
        for handle in handles:
            st = PeerScatter()
            st.world_size, st.rank = self.world, self.rank
            st.dst_row_begin, st.dst_head_begin, st.dst_heads_total = shard.row_begin, q_lo, query_heads
            for peer in range(self.world):
                st.out[peer] = int(handle.buffer_ptrs[peer])
                st.flags[peer] = int(flag_handle.buffer_ptrs[peer])
            self._structs.append(st)
        self.epoch = 0
        torch.cuda.synchronize(device)
        dist.barrier(group)   # every rank's flags are zero before anyone publishes one

    def next_step(self):
        """(descriptor, gathered tensor) of the next step."""

        self.epoch += 1
        st = self._structs[self.epoch & 1]
        st.epoch = self.epoch
        return st, self.gathered[self.epoch & 1]
