"""Dense and page-streamed attention entry points with the reference's signatures.

Mirrors ``src/dart/attention.py``.  ``dense_attention`` is plain fp32 PyTorch (it is the
uncompressed comparison point, not part of the packed path).  ``streamed_dart_attention``
keeps the reference's contract (any number of query tokens, no call to ``cache.get()``) and
evaluates every query token with the fused decode kernel.
"""

from __future__ import annotations

import math
from typing import Optional

import torch

from .cache import DartKVCache


def dense_attention(query: torch.Tensor, keys: torch.Tensor, values: torch.Tensor, *,
                    scale: Optional[float] = None) -> torch.Tensor:
    """Eager attention for ``[B, H, Q/T, D]`` tensors (reference attention.py:14-29)."""

    if query.ndim != 4 or keys.ndim != 4 or values.ndim != 4:
        raise ValueError("query, keys, and values must have shape [B, H, T, D]")
    if keys.shape != values.shape or query.shape[0] != keys.shape[0] or query.shape[-1] != keys.shape[-1]:
        raise ValueError("query/key/value batch, head_dim, and key/value shapes must be compatible")
    factor = scale if scale is not None else 1.0 / math.sqrt(query.shape[-1])
    logits = torch.matmul(query.float(), keys.float().transpose(-1, -2)) * factor
    return torch.matmul(torch.softmax(logits, dim=-1), values.float()).to(query.dtype)


def streamed_dart_attention(query: torch.Tensor, cache: DartKVCache, *, scale: Optional[float] = None) -> torch.Tensor:
    """Attend to the packed pages without materializing the cache (reference attention.py:32-87)."""

    from .fused_attention import decode_attention

    if query.ndim != 4:
        raise ValueError("query must have shape [B, Hq, Q, D]")
    if cache.get_seq_length() == 0 or cache.shape is None:
        raise ValueError("cache is empty")
    batch, kv_heads, _, head_dim = cache.shape
    if query.shape[0] != batch or query.shape[-1] != head_dim:
        raise ValueError("query batch and head_dim must match the cache")
    if query.shape[1] % kv_heads:
        raise ValueError("query heads must be divisible by cache KV heads")
    tokens = query.shape[2]
    if tokens == 1:
        return decode_attention(query[:, :, 0], cache, scale=scale).unsqueeze(2)
    # Several query tokens (no mask between them, like the reference): the tokens of a query head attend to the
    # same KV head, so t tokens x rep query heads are served by ONE launch as t * rep query heads of that KV head.
    # The tensor-core kernels take up to 4 of them per KV head, the generic kernel up to 16.
    rep = query.shape[1] // kv_heads
    per_launch = max(1, 16 // rep)
    if rep <= 4 and _tensor_core_plan(cache, query.dtype, kv_heads * rep * max(1, 4 // rep)):
        per_launch = max(1, 4 // rep)
    outputs = []
    for first in range(0, tokens, per_launch):
        chunk = query[:, :, first:first + per_launch]                      # [B, H*rep, t, D]
        t = chunk.shape[2]
        packed = chunk.reshape(batch, kv_heads, rep * t, head_dim)        # (head, token) pairs of one KV head together
        out = decode_attention(packed.reshape(batch, kv_heads * rep * t, head_dim), cache, scale=scale)
        outputs.append(out.view(batch, kv_heads * rep, t, head_dim))
    return torch.cat(outputs, dim=2) if len(outputs) > 1 else outputs[0]


def _tensor_core_plan(cache: DartKVCache, dtype: torch.dtype, query_heads: int) -> bool:
    """Whether a decode call with this many query heads would run on a tensor-core kernel."""

    import ctypes

    from . import _lib

    info = _lib.DecodePlanInfo()
    rc = _lib.LIB.dartkv_decode_plan(ctypes.byref(cache.descriptor), _lib.DTYPE_CODE[dtype], query_heads,
                                     _lib.DEQUANT_PER_OP, cache.seen_tokens, ctypes.byref(info))
    return rc == 0 and info.kernel != 0


__all__ = ["dense_attention", "streamed_dart_attention"]
