"""Dart mixed-precision keys: 2-bit for every channel, two more bits for promoted channels.

Mirrors ``src/dart/mixed.py`` of the reference (``MixedQuantizedKey``, ``select_key_channels``,
``quantize_key_mixed``) with the arithmetic in ``libdartkv_b200.so``.

Channel selection ranks by (score descending, channel ascending).  The reference ranks with
``torch.topk``, which leaves the order among equal scores unspecified; pass ``indices=`` to
``quantize_key_mixed`` to reproduce one particular reference run byte for byte.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import LIB, check, ptr, require_cuda, stream_ptr, device_guard


@dataclass
class MixedQuantizedKey:
    """Packed key tensor with 2-bit values and promoted 4-bit channels (reference mixed.py:13-34)."""

    low_values: torch.Tensor
    high_values: torch.Tensor
    channel_indices: torch.Tensor
    scale: torch.Tensor
    zero_point: torch.Tensor
    original_shape: Tuple[int, ...]
    padded_tokens: int
    group_size: int
    low_bits: int
    promote_bits: int
    output_dtype: torch.dtype

    @property
    def groups(self) -> int:
        return self.padded_tokens // self.group_size

    @property
    def promoted_channels(self) -> int:
        return self.channel_indices.shape[-1]

    @property
    def head_dim(self) -> int:
        return self.original_shape[-1]

    @property
    def nbytes(self) -> int:
        tensors = (self.low_values, self.high_values, self.channel_indices, self.scale, self.zero_point)
        return sum(t.numel() * t.element_size() for t in tensors)

    @property
    def dense_nbytes(self) -> int:
        total = 1
        for size in self.original_shape:
            total *= size
        return total * torch.tensor([], dtype=self.output_dtype).element_size()

    @property
    def compression_ratio(self) -> float:
        return self.dense_nbytes / self.nbytes if self.nbytes else 1.0

    @property
    def promote_mask(self) -> torch.Tensor:
        mask = torch.zeros((*self.original_shape[:2], self.head_dim), dtype=torch.bool,
                           device=self.channel_indices.device)
        if self.promoted_channels:
            mask.scatter_(-1, self.channel_indices.long(), True)
        return mask

    def dequantize(self, *, dtype: Optional[torch.dtype] = None, flavour: int = _lib.DEQUANT_PER_OP) -> torch.Tensor:
        device = require_cuda(self.low_values, self.scale, self.zero_point)
        out_dtype = dtype or self.output_dtype
        if out_dtype not in _lib.DTYPE_CODE:
            raise TypeError(f"unsupported output dtype {out_dtype}")
        b, h, t, d = self.original_shape
        out = torch.empty(self.original_shape, dtype=out_dtype, device=device)
        low = self.low_values.contiguous()
        high = self.high_values.contiguous()
        idx = self.channel_indices.to(torch.int32).contiguous()
        scale = self.scale.contiguous()
        zero = self.zero_point.contiguous()
        with device_guard(device):
            check(LIB.dartkv_dequantize_key_mixed(
                ptr(low), ptr(high) if self.promoted_channels else 0, ptr(idx) if self.promoted_channels else 0,
                ptr(scale), ptr(zero), _lib.DTYPE_CODE[scale.dtype], b * h, t, d, self.group_size,
                self.promoted_channels, flavour, ptr(out), _lib.DTYPE_CODE[out_dtype], stream_ptr(device)))
        return out

    def to(self, device: torch.device | str) -> "MixedQuantizedKey":
        return MixedQuantizedKey(
            low_values=self.low_values.to(device), high_values=self.high_values.to(device),
            channel_indices=self.channel_indices.to(device), scale=self.scale.to(device),
            zero_point=self.zero_point.to(device), original_shape=self.original_shape,
            padded_tokens=self.padded_tokens, group_size=self.group_size, low_bits=self.low_bits,
            promote_bits=self.promote_bits, output_dtype=self.output_dtype)


def promoted_count(head_dim: int, promote_ratio: float) -> int:
    return min(head_dim, int(head_dim * promote_ratio + 1e-6))


def channel_scores(key_states: torch.Tensor, *, strategy: str = "magnitude") -> torch.Tensor:
    """Per-channel promotion score ``[B, H, D]`` in the input dtype (reference mixed.py:154-162)."""

    if key_states.ndim != 4:
        raise ValueError("key_states must have shape [B, H, T, D]")
    if strategy not in {"magnitude", "variance"}:
        raise ValueError("strategy must be 'magnitude', 'random', or 'variance'")
    if key_states.dtype not in _lib.DTYPE_CODE:
        raise TypeError("key_states must be floating point")
    device = require_cuda(key_states)
    keys = key_states.detach().contiguous()
    b, h, t, d = keys.shape
    scores = torch.empty((b, h, d), dtype=keys.dtype, device=device)
    with device_guard(device):
        check(LIB.dartkv_channel_scores(
            ptr(keys), _lib.DTYPE_CODE[keys.dtype], b * h, t, d, t * d, d,
            _lib.SCORE_MAGNITUDE if strategy == "magnitude" else _lib.SCORE_VARIANCE, ptr(scores), stream_ptr(device)))
    return scores


def select_key_channels(
    key_states: torch.Tensor,
    promote_ratio: float,
    *,
    strategy: str = "magnitude",
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Select the key channels to promote (reference ``select_key_channels``, mixed.py:119-163).

    Returns a boolean mask ``[B, H, D]`` and channel indices ``[B, H, K]`` (int64) ordered by
    (score descending, channel ascending).
    """

    if key_states.ndim != 4:
        raise ValueError("key_states must have shape [B, H, T, D]")
    if not 0.0 <= promote_ratio <= 1.0:
        raise ValueError("promote_ratio must be in [0, 1]")
    if strategy not in {"magnitude", "random", "variance"}:
        raise ValueError("strategy must be 'magnitude', 'random', or 'variance'")
    batch, heads, _, head_dim = key_states.shape
    count = promoted_count(head_dim, promote_ratio)
    device = require_cuda(key_states)
    mask = torch.zeros(batch, heads, head_dim, dtype=torch.bool, device=device)
    if count == 0:
        return mask, torch.empty(batch, heads, 0, dtype=torch.long, device=device)
    if count == head_dim:
        indices = torch.arange(head_dim, device=device).view(1, 1, -1).expand(batch, heads, -1)
        return torch.ones_like(mask), indices
    if strategy == "random":
        # one permutation per KV head, shared across the batch (reference mixed.py:145-153)
        per_head = torch.stack([torch.randperm(head_dim, device=device)[:count] for _ in range(heads)], dim=0)
        indices = per_head.unsqueeze(0).expand(batch, -1, -1)
        mask.scatter_(-1, indices, True)
        return mask, indices
    scores = channel_scores(key_states, strategy=strategy)
    idx32 = torch.empty((batch, heads, count), dtype=torch.int32, device=device)
    with device_guard(device):
        check(LIB.dartkv_select_channels(ptr(scores), _lib.DTYPE_CODE[scores.dtype], batch * heads, head_dim, count,
                                         ptr(idx32), stream_ptr(device)))
    indices = idx32.long()
    mask.scatter_(-1, indices, True)
    return mask, indices


def quantize_key_mixed(
    key_states: torch.Tensor,
    *,
    group_size: int = 128,
    promote_ratio: float = 0.25,
    promote_bits: int = 4,
    strategy: str = "magnitude",
    metadata_dtype: Optional[torch.dtype] = None,
    indices: Optional[torch.Tensor] = None,
    check_finite: bool = True,
) -> MixedQuantizedKey:
    """Quantize a key chunk with 2-bit storage and channel promotion (reference mixed.py:166-244).

    ``indices`` (``[B, H, K]``) overrides the channel selection; ``check_finite=False`` skips the
    host synchronization of the finite-input check.
    """

    if key_states.ndim != 4:
        raise ValueError("key_states must have shape [B, H, T, D]")
    if not torch.is_floating_point(key_states):
        raise TypeError("key_states must be floating point")
    if key_states.shape[-2] == 0 or key_states.shape[-1] == 0:
        raise ValueError("key_states sequence and head dimensions must be non-empty")
    if not isinstance(group_size, int) or group_size <= 0:
        raise ValueError("group_size must be a positive integer")
    if promote_bits != 4:
        raise ValueError("the reference mixed representation currently supports promote_bits=4")
    if key_states.dtype not in _lib.DTYPE_CODE:
        raise TypeError("key_states must be float32, float16 or bfloat16")
    meta_dtype = metadata_dtype or (key_states.dtype if key_states.dtype in (torch.float16, torch.bfloat16) else torch.float32)
    if meta_dtype not in (torch.float16, torch.bfloat16, torch.float32):
        raise TypeError("metadata_dtype must be floating point")
    device = require_cuda(key_states)
    keys = key_states.detach().contiguous()
    batch, heads, tokens, head_dim = keys.shape
    if indices is None:
        _, indices = select_key_channels(keys, promote_ratio, strategy=strategy)
    idx32 = indices.to(device=device, dtype=torch.int32).contiguous()
    promoted = idx32.shape[-1]
    groups = (tokens + group_size - 1) // group_size
    packed = (group_size + 3) // 4
    low = torch.empty((batch, heads, head_dim, groups, packed), dtype=torch.uint8, device=device)
    high = torch.empty((batch, heads, promoted, groups, packed), dtype=torch.uint8, device=device)
    scale = torch.empty((batch, heads, head_dim, groups), dtype=meta_dtype, device=device)
    zero = torch.empty_like(scale)
    flag = torch.zeros(1, dtype=torch.int32, device=device) if check_finite else None
    with device_guard(device):
        check(LIB.dartkv_quantize_key_mixed(
            ptr(keys), _lib.DTYPE_CODE[keys.dtype], batch * heads, tokens, head_dim, tokens * head_dim, head_dim,
            group_size, ptr(idx32) if promoted else 0, promoted, _lib.DTYPE_CODE[meta_dtype], ptr(low),
            ptr(high) if promoted else 0, ptr(scale), ptr(zero), ptr(flag), stream_ptr(device)))
    if check_finite and int(flag.item()):
        raise ValueError("key_states must contain finite values")
    return MixedQuantizedKey(
        low_values=low, high_values=high, channel_indices=idx32, scale=scale, zero_point=zero,
        original_shape=(batch, heads, tokens, head_dim), padded_tokens=groups * group_size, group_size=group_size,
        low_bits=2, promote_bits=promote_bits, output_dtype=keys.dtype)


__all__ = ["MixedQuantizedKey", "quantize_key_mixed", "select_key_channels", "channel_scores"]
