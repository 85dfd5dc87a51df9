"""Seeded synthetic K/V/query generators for the benchmark and parity workloads.

No public dataset is involved anywhere on this path; every workload is defined
by a seed and a shape.  Values come from the PyTorch CPU generator so that the
same seed gives the same tensors on every machine with the same PyTorch build.
"""

from __future__ import annotations

from typing import Tuple

import torch


def make_kvq(
    seed: int,
    batch: int,
    kv_heads: int,
    tokens: int,
    head_dim: int,
    *,
    query_heads: int | None = None,
    dtype: torch.dtype = torch.bfloat16,
    outlier_fraction: float = 0.05,
    outlier_scale: float = 10.0,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """K, V ``[B,H,T,D]`` and a one-token query ``[B,Hq,1,D]`` on the CPU.

    V and the query are N(0,1).  K is N(0,1) with ``int(outlier_fraction * D)``
    channels per KV head (fixed across batch and tokens, drawn from the same
    generator) multiplied by ``outlier_scale``.
    """

    gen = torch.Generator(device="cpu").manual_seed(seed)
    keys = torch.randn(batch, kv_heads, tokens, head_dim, generator=gen, dtype=torch.float32)
    values = torch.randn(batch, kv_heads, tokens, head_dim, generator=gen, dtype=torch.float32)
    count = int(outlier_fraction * head_dim)
    if count and outlier_scale != 1.0:
        for head in range(kv_heads):
            channels = torch.randperm(head_dim, generator=gen)[:count]
            keys[:, head, :, channels] *= outlier_scale
    hq = query_heads if query_heads is not None else kv_heads
    query = torch.randn(batch, hq, 1, head_dim, generator=gen, dtype=torch.float32)
    return keys.to(dtype), values.to(dtype), query.to(dtype)
