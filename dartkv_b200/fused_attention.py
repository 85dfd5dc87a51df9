"""Fused single-token decode attention over packed pages (reference ``fused_dart_attention``).

Mirrors ``src/dart/fused_attention.py:654-771``: same signature and validation, but one
split-K kernel walks the cache's device-side page metadata instead of a Python loop that
launches one Triton program per page.
"""

from __future__ import annotations

import ctypes
import math
from typing import Optional, Sequence

import torch

from . import _lib
from ._lib import LIB, check, ptr, require_cuda, stream_ptr, device_guard
from .cache import DartKVCache
from .page_table import DartPageRun, DartPageTable


def decode_attention(query: torch.Tensor, cache: DartKVCache, *, scale: Optional[float] = None,
                     flavour: int = _lib.DEQUANT_PER_OP, out: Optional[torch.Tensor] = None,
                     peer_gather=None, row_start: Optional[torch.Tensor] = None,
                     token_capacity: Optional[int] = None) -> torch.Tensor:
    """One query token per (batch, query head): ``query`` and the result are ``[B, Hq, D]``.

    ``row_start`` (``[B]`` integers, first live token of every batch row) serves left-padded batches: the tokens
    before a row's first live one get no weight and the pages that hold only such tokens are not read.
    ``token_capacity`` sizes the work split for that many tokens instead of the current length (the kernels read
    the exact length on the device): a call captured in a CUDA graph stays valid while the cache grows up to it.

    With ``peer_gather`` (a ``dartkv_b200.sharding.PeerGather``) the kernels also deliver this rank's rows to every
    rank of the node and the gathered tensor ``[B_total, Hq_total, D]`` of the step is returned instead.
    """

    if cache.shape is None or cache.seen_tokens == 0:
        raise ValueError("cache is empty")
    batch, kv_heads, seen, head_dim = cache.shape
    if token_capacity is not None:
        if token_capacity < seen:
            raise ValueError("token_capacity must be at least the number of tokens in the cache")
        seen = int(token_capacity)
    if query.ndim != 3 or query.shape[0] != batch or query.shape[-1] != head_dim:
        raise ValueError("query batch and head_dim must match the cache")
    if query.shape[1] % kv_heads:
        raise ValueError("query heads must be divisible by cache KV heads")
    if query.dtype not in _lib.DTYPE_CODE:
        raise TypeError("query must be float32, float16 or bfloat16")
    device = require_cuda(query)
    if device != cache._device:
        raise ValueError("query and cache must be on the same device")
    q = query.contiguous()
    rep = q.shape[1] // kv_heads
    if row_start is not None:
        if peer_gather is not None:
            raise ValueError("row_start and peer_gather cannot be combined")
        if row_start.shape != (batch,):
            raise ValueError("row_start must have shape [batch]")
        row_start = row_start.to(device=q.device, dtype=torch.int32).contiguous()
    if rep > 4 and peer_gather is None and _grouped_heads_pay_off(cache, q.dtype, kv_heads, flavour, seen):
        # The tensor-core kernels take up to four query heads per KV head.  Wider groups (5..16 heads per KV head)
        # are served four heads at a time: every pass streams the packed pages again, which is still far cheaper
        # than the CUDA-core kernel that would otherwise take the whole group.
        grouped = q.view(batch, kv_heads, rep, head_dim)
        result = out if out is not None else torch.empty_like(q)
        result_view = result.view(batch, kv_heads, rep, head_dim)
        for first in range(0, rep, 4):
            part = grouped[:, :, first:first + 4].reshape(batch, -1, head_dim)
            result_view[:, :, first:first + 4] = decode_attention(part, cache, scale=scale, flavour=flavour,
                                                                   row_start=row_start, token_capacity=token_capacity).view(
                batch, kv_heads, -1, head_dim)
        return result
    if out is None:
        out = torch.empty_like(q)
    factor = scale if scale is not None else 1.0 / math.sqrt(head_dim)
    workspace, capacity = cache.decode_workspace(q.shape[1])
    if peer_gather is not None:
        peers, gathered = peer_gather.next_step()
        with device_guard(device):
            check(LIB.dartkv_decode_attention_scatter(
                ctypes.byref(cache.descriptor), ptr(q), _lib.DTYPE_CODE[q.dtype], q.shape[1], float(factor), flavour,
                seen, ptr(workspace), workspace.numel(), ptr(out), ctypes.byref(peers), stream_ptr(device)))
        return gathered
    if row_start is not None:
        with device_guard(device):
            check(LIB.dartkv_decode_attention_padded(
                ctypes.byref(cache.descriptor), ptr(q), _lib.DTYPE_CODE[q.dtype], q.shape[1], float(factor), flavour,
                seen, ptr(row_start), ptr(workspace), workspace.numel(), ptr(out), stream_ptr(device)))
        return out
    with device_guard(device):
        check(LIB.dartkv_decode_attention(
            ctypes.byref(cache.descriptor), ptr(q), _lib.DTYPE_CODE[q.dtype], q.shape[1], float(factor), flavour,
            seen, ptr(workspace), workspace.numel(), ptr(out), stream_ptr(device)))
    return out


def _grouped_heads_pay_off(cache: DartKVCache, dtype: torch.dtype, kv_heads: int, flavour: int, seen: int) -> bool:
    """True when a call with four query heads per KV head would run on a tensor-core kernel."""

    info = _lib.DecodePlanInfo()
    rc = LIB.dartkv_decode_plan(ctypes.byref(cache.descriptor), _lib.DTYPE_CODE[dtype], 4 * kv_heads, flavour, seen,
                                ctypes.byref(info))
    return rc == 0 and info.kernel != 0


def fused_dart_attention(
    query: torch.Tensor,
    cache: DartKVCache,
    *,
    scale: Optional[float] = None,
    fallback: bool = True,
    page_table: Optional[DartPageTable] = None,
    page_runs: Optional[Sequence[DartPageRun]] = None,
    flavour: int = _lib.DEQUANT_PER_OP,
    row_start: Optional[torch.Tensor] = None,
    token_capacity: Optional[int] = None,
    out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Single-token page attention, ``query [B, Hq, 1, D] -> [B, Hq, 1, D]``.

    ``flavour`` picks the dequantization arithmetic: ``DEQUANT_PER_OP`` (default) reproduces the
    reference's streamed path, whose pages are dequantized with the multiply and the add each
    rounded to the metadata dtype; ``DEQUANT_FUSED`` reproduces the reference's Triton kernels
    (``fused_attention.py:149-262``), which keep ``code * scale + zero`` in fp32.

    ``fallback`` only decides what happens for more than one query token (the streamed
    per-token path, as in the reference); there is no CPU fallback.  ``page_table`` and
    ``page_runs`` are validated against the cache like the reference does and otherwise
    unused: the kernel reads the device-resident metadata.

    ``row_start`` (``[B]`` integers, not in the reference) masks the tokens before every row's first live one:
    left-padded batches of unequal prompts decode through the packed path instead of falling back to dense.
    It applies to the single-token call only.  ``token_capacity`` and ``out`` (a ``[B, Hq, D]`` tensor that takes
    the result) serve calls captured in a CUDA graph: see ``decode_attention``.
    """

    if query.ndim != 4:
        raise ValueError("query must have shape [B, Hq, 1, D]")
    if query.shape[-2] != 1:
        if fallback:
            from .attention import streamed_dart_attention

            return streamed_dart_attention(query, cache, scale=scale)
        raise ValueError("fused_dart_attention currently supports one query token")
    if not query.is_cuda:
        raise RuntimeError("fused_dart_attention requires CUDA (dartkv_b200 has no CPU fallback)")
    cache_shape = cache.shape
    if cache_shape is None or cache_shape[2] == 0:
        raise ValueError("cache is empty")
    batch, kv_heads, _, head_dim = cache_shape
    if query.shape[0] != batch or query.shape[-1] != head_dim:
        raise ValueError("query batch and head_dim must match the cache")
    if query.shape[1] % kv_heads:
        raise ValueError("query heads must be divisible by cache KV heads")
    if page_table is not None:
        rows = cache.segment_table()
        if page_table.page_count != len(rows) or page_table.seen_tokens != cache.seen_tokens:
            raise ValueError("page_table does not describe the current cache segments")
    if page_runs is not None:
        starts = set()
        total = len(cache.segment_table())
        for run in page_runs:
            run.validate()
            if run.first_page_index in starts:
                raise ValueError("page_runs contain duplicate first_page_index")
            if run.first_page_index < 0 or run.first_page_index + run.page_count > total:
                raise ValueError("page_run is outside the current cache page range")
            starts.add(run.first_page_index)
    return decode_attention(query[:, :, 0], cache, scale=scale, flavour=flavour, row_start=row_start,
                            token_capacity=token_capacity, out=out).unsqueeze(2)


__all__ = ["fused_dart_attention", "decode_attention"]
