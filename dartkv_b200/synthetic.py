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


# ---------------------------------------------------------------------------------------------------------------
# The benchmark workloads (long-context decode): 32 query heads / 8 KV heads, head_dim 128, 128-token pages,
# 2-bit values, 2-bit keys with a quarter of the channels promoted to 2+2 bits, key group 128, value group 64,
# 32 dense sink tokens, pages held until full.
HEADLINE_GEOMETRY = dict(query_heads=32, kv_heads=8, head_dim=128, page=128, key_group=128, value_group=64, sinks=32,
                         promote_ratio=0.25, bits=2)


def headline_cache_kwargs() -> dict:
    g = HEADLINE_GEOMETRY
    return dict(bits=g["bits"], promote_ratio=g["promote_ratio"], page_size=g["page"], key_group_size=g["key_group"],
                value_group_size=g["value_group"], sink_tokens=g["sinks"], hold_partial_pages=True)


def outlier_channels(seed: int, kv_heads: int, head_dim: int, fraction: float = 0.05) -> torch.Tensor:
    """``[kv_heads, int(fraction * head_dim)]`` channel indices per KV head, fixed by the seed."""

    gen = torch.Generator().manual_seed(seed)
    count = int(fraction * head_dim)
    return torch.stack([torch.randperm(head_dim, generator=gen)[:count] for _ in range(kv_heads)])


def build_headline_cache(rows, ctx: int, seed: int, device: torch.device, *, heads=None, keep_rows=None,
                         metadata_dtype: torch.dtype = torch.bfloat16, cache_overrides=None):
    """Fill a ``DartKVCache`` on ``device`` with ``ctx`` tokens of bf16 K/V for the global batch rows ``rows``.

    Every batch row has its own device generator, seeded from the workload seed and the row's global index, so
    a row's data does not depend on how the batch is sharded: any rank can rebuild any row.  The first append
    carries the 32 sink tokens, the rest arrive 1024 tokens at a time.  ``heads = (first, end)`` keeps only those
    KV heads of every row (and the query heads that attend to them).  Returns ``(cache, query [B,Hq,1,D])`` and,
    when ``keep_rows`` lists global rows, also their K and V ``[len(keep_rows), H, ctx, D]`` as generated.
    ``cache_overrides`` replaces fields of the cache configuration (code width, promotion ratio, group sizes) for
    runs of the same data off the headline geometry.
    """

    from .cache import DartKVCache, DartKVCacheConfig

    g = HEADLINE_GEOMETRY
    rows = list(rows)
    h0, h1 = heads if heads is not None else (0, g["kv_heads"])
    rep = g["query_heads"] // g["kv_heads"]
    keep = [rows.index(r) for r in keep_rows] if keep_rows is not None else []
    config = headline_cache_kwargs()
    config.update(cache_overrides or {})
    cache = DartKVCache(DartKVCacheConfig(metadata_dtype=metadata_dtype, **config), max_tokens=ctx + 256)
    gens = [torch.Generator(device=device).manual_seed(seed * 1000003 + 17 * row) for row in rows]
    mult = torch.ones(g["kv_heads"], g["head_dim"], device=device)
    mult.scatter_(1, outlier_channels(seed, g["kv_heads"], g["head_dim"]).to(device), 10.0)
    mult = mult.view(g["kv_heads"], 1, g["head_dim"])
    done = 0
    first = True
    kept_k, kept_v = [], []
    while done < ctx:
        step = g["sinks"] if first else min(1024, ctx - done)
        first = False
        shape = (g["kv_heads"], step, g["head_dim"])
        keys = torch.stack([(torch.randn(shape, generator=gn, device=device) * mult).to(torch.bfloat16)[h0:h1] for gn in gens])
        values = torch.stack([torch.randn(shape, generator=gn, device=device).to(torch.bfloat16)[h0:h1] for gn in gens])
        cache.append(keys, values)
        if keep:
            kept_k.append(keys[keep])
            kept_v.append(values[keep])
        done += step
    qshape = (g["query_heads"], 1, g["head_dim"])
    query = torch.stack([torch.randn(qshape, generator=gn, device=device).to(torch.bfloat16)[h0 * rep:h1 * rep] for gn in gens])
    torch.cuda.synchronize(device)
    if keep_rows is not None:
        return cache, query, torch.cat(kept_k, dim=2), torch.cat(kept_v, dim=2)
    return cache, query
