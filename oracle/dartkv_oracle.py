"""CPU restatement (NumPy) of the DartKV KV-cache hot path.  TEST INFRASTRUCTURE ONLY.

This module is the checker for the CUDA library, never the thing that ships or
is measured as the product: only the tests, the smoke entry point and the
``cpu_baseline`` / ``--impl reference`` legs of the benchmark may import it.

It restates, operation by operation, the arithmetic of the reference
implementation (paths are relative to the reference project root):

* ``src/dart/quantization.py:25-45``   bit packing / unpacking
* ``src/dart/quantization.py:134-204`` group-wise asymmetric quantizer
* ``src/dart/quantization.py:96-109``  dequantization (metadata-dtype arithmetic)
* ``src/dart/mixed.py:119-163``        promoted-channel selection
* ``src/dart/mixed.py:166-244``        mixed 2+2-bit key quantizer
* ``src/dart/mixed.py:72-94``          mixed key dequantization
* ``src/dart/cache.py:168-190,403-542`` paged cache lifecycle
* ``src/dart/cache.py:229-274``        K/V segment boundary union
* ``src/dart/attention.py:14-29,32-87`` dense and page-streamed attention
* ``src/dart/triton_ops.py:32-201``    fp32 single-rounding dequantization flavour

Parity pin: every function here is checked against vectors produced by running
the reference itself (``tests/golden/make_golden.py`` writes them,
``tests/test_oracle_golden.py`` checks them).

Numeric model.  The reference computes every elementwise step in the dtype of
its input tensor (PyTorch evaluates a bf16/fp16 op in fp32 and rounds the
result back).  Arrays are therefore carried as float32 together with a dtype
tag ('f32', 'f16', 'bf16') and every step is followed by ``round_to``.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple, Union

import numpy as np

DTYPES = ("f32", "f16", "bf16")
_ELEM_BYTES = {"f32": 4, "f16": 2, "bf16": 2}


# --------------------------------------------------------------------------- rounding
def round_to(x, dt: str) -> np.ndarray:
    """Round float32 values to ``dt`` (nearest-even) and return them as float32."""

    x = np.ascontiguousarray(x, dtype=np.float32)
    if dt == "f32":
        return x
    if dt == "f16":
        with np.errstate(over="ignore"):
            return x.astype(np.float16).astype(np.float32)
    if dt == "bf16":
        bits = x.view(np.uint32).astype(np.uint64)
        bits = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
        return bits.astype(np.uint32).view(np.float32).reshape(x.shape)
    raise TypeError(f"unsupported dtype tag {dt!r}")


def bf16_bits_to_f32(u16: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(u16).view(np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    return (round_to(x, "bf16").view(np.uint32) >> 16).astype(np.uint16)


def _eps(dt: str) -> np.float32:
    # quantization.py:181 / mixed.py:206
    return np.float32(1e-4) if dt in ("f16", "bf16") else np.float32(1e-6)


def _default_md(dt: str, md: Optional[str]) -> str:
    # quantization.py:48-53
    if md is not None:
        if md not in DTYPES:
            raise TypeError(f"metadata dtype must be floating point, got {md}")
        return md
    return dt if dt in ("f16", "bf16") else "f32"


# --------------------------------------------------------------------------- bit packing
def pack_bits(codes: np.ndarray, bits: int, packed_dim: Optional[int] = None) -> np.ndarray:
    """quantization.py:25-35: element i of a byte sits at bit (i % vpb) * bits."""

    vpb = 8 // bits
    codes = np.asarray(codes, dtype=np.uint8)
    n = codes.shape[-1]
    if packed_dim is None:
        packed_dim = -(-n // vpb) * vpb
    if packed_dim > n:
        pad = np.zeros(codes.shape[:-1] + (packed_dim - n,), dtype=np.uint8)
        codes = np.concatenate((codes, pad), axis=-1)
    lanes = codes.reshape(codes.shape[:-1] + (packed_dim // vpb, vpb)).astype(np.uint32)
    shifts = (np.arange(vpb, dtype=np.uint32) * bits)
    return ((lanes << shifts).sum(axis=-1) & 0xFF).astype(np.uint8)


def unpack_bits(packed: np.ndarray, bits: int, count: int) -> np.ndarray:
    """quantization.py:38-45."""

    vpb = 8 // bits
    packed = np.asarray(packed, dtype=np.uint8)
    shifts = (np.arange(vpb, dtype=np.uint8) * bits).astype(np.uint8)
    lanes = (packed[..., None] >> shifts) & np.uint8((1 << bits) - 1)
    return lanes.reshape(packed.shape[:-1] + (packed.shape[-1] * vpb,))[..., :count]


# --------------------------------------------------------------------------- uniform quantizer
@dataclass
class QTensor:
    values: np.ndarray          # uint8, packed along the last dim
    scale: np.ndarray           # float32 carrier, already rounded to ``md``
    zero_point: np.ndarray      # group minimum, same
    original_shape: Tuple[int, ...]
    original_dim: int
    padded_dim: int
    packed_dim: int
    group_size: int
    bits: int
    out_dt: str
    md: str
    axis: int

    @property
    def groups(self) -> int:
        return (self.padded_dim + self.group_size - 1) // self.group_size

    @property
    def nbytes(self) -> int:
        return int(self.values.size + (self.scale.size + self.zero_point.size) * _ELEM_BYTES[self.md])

    @property
    def dense_nbytes(self) -> int:
        return int(np.prod(self.original_shape)) * _ELEM_BYTES[self.out_dt]

    @property
    def tokens(self) -> int:
        return self.original_shape[-2]


def _check_common(bits: int, group_size) -> None:
    if bits not in (2, 4, 8):
        raise ValueError(f"bits must be one of (2, 4, 8), got {bits}")
    if not isinstance(group_size, int) or group_size <= 0:
        raise ValueError(f"group_size must be a positive integer, got {group_size}")


def _affine_codes(grouped: np.ndarray, qmax: np.ndarray, dt: str, div: str):
    """Shared min/max -> scale -> code recipe (quantization.py:178-186, mixed.py:200-209).

    ``grouped`` is [..., groups, group]; ``qmax`` broadcasts against [..., groups].
    """

    mn = grouped.min(axis=-1)
    mx = grouped.max(axis=-1)
    rng = round_to(mx - mn, dt)
    rng = np.maximum(rng, round_to(_eps(dt), dt))
    qmax32 = np.asarray(qmax, dtype=np.float32)
    if div == "true":
        scale = round_to(rng / qmax32, dt)
    elif div == "reciprocal":
        # PyTorch's CUDA kernel for tensor / python-scalar multiplies by 1/scalar.
        scale = round_to(rng * (np.float32(1.0) / qmax32), dt)
    else:
        raise ValueError("div must be 'true' or 'reciprocal'")
    shifted = round_to(grouped - mn[..., None], dt)
    ratio = round_to(shifted / scale[..., None], dt)
    codes = np.rint(ratio)
    codes = np.minimum(np.maximum(codes, np.float32(0.0)), qmax32[..., None] if qmax32.ndim else qmax32)
    return codes.astype(np.uint8), scale, mn


def quantize(
    data: np.ndarray,
    dt: str,
    *,
    bits: int = 2,
    group_size: int = 64,
    md: Optional[str] = None,
    axis: int = -1,
    div: str = "true",
) -> QTensor:
    """quantization.py:134-204."""

    _check_common(bits, group_size)
    data = np.asarray(data)
    if data.ndim == 0:
        raise ValueError("quantize expects a tensor with at least one dimension")
    if not np.issubdtype(data.dtype, np.floating):
        raise TypeError(f"quantize expects a floating-point tensor, got {data.dtype}")
    if data.shape[-1] == 0:
        raise ValueError("quantize does not support an empty final dimension")
    if not np.isfinite(data).all():
        raise ValueError("quantize expects all values to be finite")
    if not isinstance(axis, int) or not -data.ndim <= axis < data.ndim:
        raise ValueError(f"axis must be in [-{data.ndim}, {data.ndim}), got {axis}")
    original_shape = tuple(data.shape)
    axis = axis % data.ndim
    moved = np.ascontiguousarray(np.moveaxis(round_to(data, dt), axis, -1))
    n = moved.shape[-1]
    groups = -(-n // group_size)
    padded = groups * group_size
    flat = moved.reshape(-1, n)
    if padded > n:
        flat = np.concatenate((flat, np.repeat(flat[:, -1:], padded - n, axis=1)), axis=1)
    grouped = flat.reshape(-1, groups, group_size)
    qmax = np.float32((1 << bits) - 1)
    codes, scale, mn = _affine_codes(grouped, qmax, dt, div)
    codes = codes.reshape(moved.shape[:-1] + (padded,))
    vpb = 8 // bits
    packed_dim = -(-padded // vpb) * vpb
    meta = _default_md(dt, md)
    return QTensor(
        values=pack_bits(codes, bits, packed_dim),
        scale=round_to(scale.reshape(moved.shape[:-1] + (groups,)), meta),
        zero_point=round_to(mn.reshape(moved.shape[:-1] + (groups,)), meta),
        original_shape=original_shape,
        original_dim=n,
        padded_dim=padded,
        packed_dim=packed_dim,
        group_size=group_size,
        bits=bits,
        out_dt=dt,
        md=meta,
        axis=axis,
    )


def _affine_restore(codes_f32: np.ndarray, scale, zero, md: str, out_dt: str, flavour: str) -> np.ndarray:
    if flavour == "cpu":
        # quantization.py:103-106 / mixed.py:91-94: multiply and add each rounded to the metadata dtype
        restored = round_to(round_to(codes_f32 * scale, md) + zero, md)
        return round_to(restored, out_dt)
    if flavour == "fp32":
        # triton_ops.py:59,110,201: fp32 multiply-add, one rounding to the output dtype
        fused = (codes_f32.astype(np.float64) * scale.astype(np.float64) + zero.astype(np.float64)).astype(np.float32)
        return round_to(fused, out_dt)
    if flavour == "fused":
        # fused_attention.py:159,209,241: the Triton attention kernels keep code * scale + zero in fp32 and never
        # round it to the cache dtype
        return (codes_f32.astype(np.float64) * scale.astype(np.float64) + zero.astype(np.float64)).astype(np.float32)
    raise ValueError("flavour must be 'cpu', 'fp32' or 'fused'")


def dequantize(q: QTensor, *, out_dt: Optional[str] = None, flavour: str = "cpu") -> np.ndarray:
    """quantization.py:96-109 (flavour 'cpu') or triton_ops.py:32-110 (flavour 'fp32')."""

    codes = unpack_bits(q.values, q.bits, q.packed_dim)[..., : q.padded_dim]
    outer = codes.shape[:-1]
    grouped = codes.reshape(outer + (q.groups, q.group_size)).astype(np.float32)
    restored = _affine_restore(grouped, q.scale[..., None], q.zero_point[..., None], q.md, out_dt or q.out_dt, flavour)
    restored = restored.reshape(outer + (q.padded_dim,))[..., : q.original_dim]
    if q.axis != len(q.original_shape) - 1:
        restored = np.moveaxis(restored, -1, q.axis)
    return np.ascontiguousarray(restored)


# --------------------------------------------------------------------------- mixed key
@dataclass
class MixedKey:
    low_values: np.ndarray        # [B,H,D,G,ceil(Gk/4)] uint8
    high_values: np.ndarray       # [B,H,K,G,ceil(Gk/4)] uint8
    channel_indices: np.ndarray   # [B,H,K] int32
    scale: np.ndarray             # [B,H,D,G]
    zero_point: np.ndarray
    original_shape: Tuple[int, ...]
    padded_tokens: int
    group_size: int
    out_dt: str
    md: str

    @property
    def groups(self) -> int:
        return self.padded_tokens // self.group_size

    @property
    def nbytes(self) -> int:
        meta = (self.scale.size + self.zero_point.size) * _ELEM_BYTES[self.md]
        return int(self.low_values.size + self.high_values.size + self.channel_indices.size * 4 + meta)

    @property
    def dense_nbytes(self) -> int:
        return int(np.prod(self.original_shape)) * _ELEM_BYTES[self.out_dt]

    @property
    def tokens(self) -> int:
        return self.original_shape[-2]


def _mean_over_tokens(x: np.ndarray, dt: str) -> np.ndarray:
    """``tensor.mean(dim=-2)`` in dtype ``dt``: fp32 accumulation, one rounding."""

    total = x.astype(np.float64).sum(axis=-2).astype(np.float32)
    return round_to(total / np.float32(x.shape[-2]), dt)


def channel_scores(keys: np.ndarray, dt: str, strategy: str = "magnitude") -> np.ndarray:
    """mixed.py:154-162: per-channel score in the input dtype, [B,H,D]."""

    keys = round_to(keys, dt)
    if strategy == "magnitude":
        return _mean_over_tokens(np.abs(keys), dt)
    if strategy == "variance":
        mean = _mean_over_tokens(keys, dt)
        centered = round_to(keys - mean[..., None, :], dt)
        return _mean_over_tokens(round_to(centered * centered, dt), dt)
    raise ValueError("strategy must be 'magnitude', 'random', or 'variance'")


def promoted_count(head_dim: int, ratio: float) -> int:
    return min(head_dim, int(head_dim * ratio + 1e-6))


def select_key_channels(
    keys: np.ndarray, dt: str, ratio: float, *, strategy: str = "magnitude"
) -> Tuple[np.ndarray, np.ndarray]:
    """mixed.py:119-163.  Tie rule of this restatement: score descending, channel ascending.

    ``torch.topk`` leaves the choice and order among equal scores unspecified, so
    only the score vector and (absent a tie at the cut) the selected *set* are
    comparable with the reference; pass explicit indices to ``quantize_key_mixed``
    to reproduce a particular reference run byte for byte.
    """

    keys = np.asarray(keys)
    if keys.ndim != 4:
        raise ValueError("key_states must have shape [B, H, T, D]")
    if not 0.0 <= ratio <= 1.0:
        raise ValueError("promote_ratio must be in [0, 1]")
    if strategy not in ("magnitude", "random", "variance"):
        raise ValueError("strategy must be 'magnitude', 'random', or 'variance'")
    b, h, _, d = keys.shape
    count = promoted_count(d, ratio)
    mask = np.zeros((b, h, d), dtype=bool)
    if count == 0:
        return mask, np.zeros((b, h, 0), dtype=np.int64)
    if count == d:
        return np.ones_like(mask), np.broadcast_to(np.arange(d, dtype=np.int64), (b, h, d)).copy()
    if strategy == "random":
        raise ValueError("random selection depends on the caller's generator; pass indices explicitly")
    score = channel_scores(keys, dt, strategy)
    order = np.argsort(-score.astype(np.float64), axis=-1, kind="stable")
    indices = order[..., :count].astype(np.int64)
    np.put_along_axis(mask, indices, True, axis=-1)
    return mask, indices


def quantize_key_mixed(
    keys: np.ndarray,
    dt: str,
    *,
    group_size: int = 128,
    ratio: float = 0.25,
    promote_bits: int = 4,
    strategy: str = "magnitude",
    md: Optional[str] = None,
    indices: Optional[np.ndarray] = None,
) -> MixedKey:
    """mixed.py:166-244."""

    keys = np.asarray(keys)
    if keys.ndim != 4:
        raise ValueError("key_states must have shape [B, H, T, D]")
    if not np.issubdtype(keys.dtype, np.floating):
        raise TypeError("key_states must be floating point")
    if keys.shape[-2] == 0 or keys.shape[-1] == 0:
        raise ValueError("key_states sequence and head dimensions must be non-empty")
    if not isinstance(group_size, int) or group_size <= 0:
        raise ValueError("group_size must be a positive integer")
    if promote_bits != 4:
        raise ValueError("the reference mixed representation currently supports promote_bits=4")
    if not np.isfinite(keys).all():
        raise ValueError("key_states must contain finite values")
    keys = round_to(keys, dt)
    b, h, t, d = keys.shape
    if indices is None:
        mask, indices = select_key_channels(keys, dt, ratio, strategy=strategy)
    else:
        indices = np.asarray(indices, dtype=np.int64)
        mask = np.zeros((b, h, d), dtype=bool)
        if indices.shape[-1]:
            np.put_along_axis(mask, indices, True, axis=-1)
    groups = -(-t // group_size)
    padded = groups * group_size
    data = np.ascontiguousarray(np.swapaxes(keys, -1, -2))
    if padded > t:
        data = np.concatenate((data, np.repeat(data[..., -1:], padded - t, axis=-1)), axis=-1)
    grouped = data.reshape(b, h, d, groups, group_size)
    qmax = np.where(mask[..., None], np.float32(15.0), np.float32(3.0)).astype(np.float32)
    qmax = np.broadcast_to(qmax, (b, h, d, groups))
    codes, scale, mn = _affine_codes(grouped, qmax, dt, "true")
    low = pack_bits(codes & 0x3, 2)
    k = indices.shape[-1]
    if k:
        gather = np.broadcast_to(indices[..., None, None], (b, h, k, groups, group_size))
        high = pack_bits(np.take_along_axis(codes, gather, axis=2) >> 2, 2)
    else:
        high = np.zeros((b, h, 0, groups, low.shape[-1]), dtype=np.uint8)
    meta = _default_md(dt, md)
    return MixedKey(
        low_values=low,
        high_values=high,
        channel_indices=indices.astype(np.int32),
        scale=round_to(scale, meta),
        zero_point=round_to(mn, meta),
        original_shape=(b, h, t, d),
        padded_tokens=padded,
        group_size=group_size,
        out_dt=dt,
        md=meta,
    )


def dequantize_mixed(m: MixedKey, *, out_dt: Optional[str] = None, flavour: str = "cpu") -> np.ndarray:
    """mixed.py:72-94 (flavour 'cpu') or triton_ops.py:113-201 (flavour 'fp32')."""

    b, h, t, d = m.original_shape
    low = unpack_bits(m.low_values, 2, m.low_values.shape[-1] * 4)[..., : m.group_size]
    codes = low.astype(np.uint8).copy()
    if m.channel_indices.shape[-1]:
        high = unpack_bits(m.high_values, 2, m.high_values.shape[-1] * 4)[..., : m.group_size]
        full = np.zeros_like(codes)
        idx = np.broadcast_to(m.channel_indices.astype(np.int64)[..., None, None], high.shape)
        np.put_along_axis(full, idx, high, axis=2)
        codes = codes | (full << 2)
    restored = _affine_restore(
        codes.astype(np.float32), m.scale[..., None], m.zero_point[..., None], m.md, out_dt or m.out_dt, flavour
    )
    restored = restored.reshape(b, h, d, m.padded_tokens)[..., :t]
    return np.ascontiguousarray(np.swapaxes(restored, -1, -2))


Segment = Union[np.ndarray, QTensor, MixedKey]


def materialize(seg: Segment, flavour: str = "cpu") -> np.ndarray:
    if isinstance(seg, np.ndarray):
        return seg
    if isinstance(seg, MixedKey):
        return dequantize_mixed(seg, flavour=flavour)
    return dequantize(seg, flavour=flavour)


def segment_tokens(seg: Segment) -> int:
    return seg.shape[-2] if isinstance(seg, np.ndarray) else seg.original_shape[-2]


def segment_nbytes(seg: Segment, dt: str) -> int:
    return int(seg.size) * _ELEM_BYTES[dt] if isinstance(seg, np.ndarray) else seg.nbytes


# --------------------------------------------------------------------------- cache lifecycle
@dataclass(frozen=True)
class CacheConfig:
    """Field-for-field mirror of ``DartKVCacheConfig`` (cache.py:45-112); dtypes are tags."""

    bits: int = 2
    group_size: int = 64
    sink_tokens: int = 0
    metadata_dtype: str = "f16"
    key_bits: Optional[int] = None
    value_bits: Optional[int] = None
    key_group_size: Optional[int] = None
    value_group_size: Optional[int] = None
    page_size: int = 128
    hold_partial_pages: bool = False
    local_tokens: int = 0
    value_local_tokens: int = 0
    promote_bits: int = 4
    promote_ratio: float = 0.0
    channel_selection: str = "magnitude"

    @property
    def kbits(self) -> int:
        return self.key_bits if self.key_bits is not None else self.bits

    @property
    def vbits(self) -> int:
        return self.value_bits if self.value_bits is not None else self.bits

    @property
    def kgroup(self) -> int:
        return self.key_group_size if self.key_group_size is not None else self.group_size

    @property
    def vgroup(self) -> int:
        return self.value_group_size if self.value_group_size is not None else self.group_size


def _slice_q(q: QTensor, start: int, stop: int) -> QTensor:
    shape = list(q.original_shape)
    shape[-2] = stop - start
    return QTensor(q.values[..., start:stop, :], q.scale[..., start:stop, :], q.zero_point[..., start:stop, :],
                   tuple(shape), q.original_dim, q.padded_dim, q.packed_dim, q.group_size, q.bits, q.out_dt, q.md, q.axis)


def _merge_q(a: QTensor, b: QTensor) -> QTensor:
    shape = list(a.original_shape)
    shape[-2] = a.original_shape[-2] + b.original_shape[-2]
    return QTensor(np.concatenate((a.values, b.values), axis=-2), np.concatenate((a.scale, b.scale), axis=-2),
                   np.concatenate((a.zero_point, b.zero_point), axis=-2), tuple(shape), a.original_dim, a.padded_dim,
                   a.packed_dim, a.group_size, a.bits, a.out_dt, a.md, a.axis)


class OracleCache:
    """Restatement of ``DartKVCache`` append / segment bookkeeping (cache.py:115-542).

    ``channel_indices_provider`` lets a test feed the promoted channels chosen by
    a particular reference run (one [B,H,K] array per mixed key page, in order).
    """

    def __init__(self, config: Optional[CacheConfig] = None, dt: str = "f32", channel_indices_provider=None):
        self.config = config or CacheConfig()
        self.dt = dt
        self.key_segments: List[Segment] = []
        self.value_segments: List[Segment] = []
        self.pending_key: Optional[np.ndarray] = None
        self.pending_value: Optional[np.ndarray] = None
        self.seen_tokens = 0
        self.shape3: Optional[Tuple[int, int, int]] = None
        self._provider = channel_indices_provider
        self._mixed_pages = 0

    # cache.py:168-190
    def append(self, keys: np.ndarray, values: np.ndarray) -> None:
        keys = round_to(keys, self.dt)
        values = round_to(values, self.dt)
        if keys.ndim != 4 or values.ndim != 4:
            raise ValueError("key_states and value_states must have shape [B, H, T, D]")
        if keys.shape != values.shape:
            raise ValueError(f"key/value shapes must match, got {keys.shape} and {values.shape}")
        if keys.shape[-2] == 0 or keys.shape[-1] == 0:
            raise ValueError("key/value sequence and head dimensions must be non-empty")
        shape3 = (keys.shape[0], keys.shape[1], keys.shape[3])
        if self.shape3 is None:
            self.shape3 = shape3
        elif shape3 != self.shape3:
            raise ValueError("all updates must keep batch/head/head_dim, dtype, and device unchanged")
        t = keys.shape[-2]
        sink = min(max(0, self.config.sink_tokens - self.seen_tokens), t)
        if sink:
            self.key_segments.append(keys[..., :sink, :].copy())
            self.value_segments.append(values[..., :sink, :].copy())
        if sink < t:
            self._append_remainder(keys[..., sink:, :], values[..., sink:, :])
        self.seen_tokens += t

    # cache.py:403-422
    def _append_remainder(self, k: np.ndarray, v: np.ndarray) -> None:
        cfg = self.config
        if cfg.value_local_tokens:
            self._append_key_remainder(k)
            self._append_value_remainder(v)
            return
        if cfg.hold_partial_pages or cfg.local_tokens:
            if self.pending_key is not None:
                k = np.concatenate((self.pending_key, k), axis=-2)
                v = np.concatenate((self.pending_value, v), axis=-2)
            avail = max(0, k.shape[-2] - cfg.local_tokens)
            full = (avail // cfg.page_size) * cfg.page_size
            if full:
                self._quantize_pages(k[..., :full, :], v[..., :full, :])
            self.pending_key = k[..., full:, :].copy() if full < k.shape[-2] else None
            self.pending_value = v[..., full:, :].copy() if full < v.shape[-2] else None
            return
        for start in range(0, k.shape[-2], cfg.page_size):
            stop = min(start + cfg.page_size, k.shape[-2])
            self._quantize_pages(k[..., start:stop, :], v[..., start:stop, :])

    # cache.py:424-455
    def _append_key_remainder(self, k: np.ndarray) -> None:
        cfg = self.config
        if (self.seen_tokens > 0 and self.pending_key is None and cfg.local_tokens == 1 and k.shape[-2] == 1
                and self.key_segments and not isinstance(self.key_segments[-1], np.ndarray)):
            final_page = materialize(self.key_segments.pop())
            self._quantize_key_pages(final_page)
        if self.pending_key is not None:
            k = np.concatenate((self.pending_key, k), axis=-2)
        local = 0 if self.seen_tokens == 0 else cfg.local_tokens
        avail = max(0, k.shape[-2] - local)
        full = (avail // cfg.page_size) * cfg.page_size
        if full:
            self._quantize_key_pages(k[..., :full, :])
        self.pending_key = k[..., full:, :].copy() if full < k.shape[-2] else None

    # cache.py:457-470
    def _append_value_remainder(self, v: np.ndarray) -> None:
        cfg = self.config
        if self.pending_value is not None:
            v = np.concatenate((self.pending_value, v), axis=-2)
        quantized = max(0, v.shape[-2] - cfg.value_local_tokens)
        for start in range(0, quantized, cfg.page_size):
            stop = min(start + cfg.page_size, quantized)
            self._quantize_value_segment(v[..., start:stop, :])
        self.pending_value = v[..., quantized:, :].copy() if quantized < v.shape[-2] else None

    # cache.py:472-479
    def _quantize_pages(self, k: np.ndarray, v: np.ndarray) -> None:
        p = self.config.page_size
        for start in range(0, k.shape[-2], p):
            stop = min(start + p, k.shape[-2])
            self._quantize_key_pages(k[..., start:stop, :])
            self._quantize_value_segment(v[..., start:stop, :])

    # cache.py:481-503
    def _quantize_key_pages(self, k: np.ndarray) -> None:
        cfg = self.config
        for start in range(0, k.shape[-2], cfg.page_size):
            page = k[..., start:start + cfg.page_size, :]
            if cfg.promote_ratio > 0.0:
                indices = None
                if self._provider is not None:
                    indices = self._provider(self._mixed_pages)
                self._mixed_pages += 1
                seg: Segment = quantize_key_mixed(page, self.dt, group_size=cfg.kgroup, ratio=cfg.promote_ratio,
                                                  promote_bits=cfg.promote_bits, strategy=cfg.channel_selection,
                                                  md=cfg.metadata_dtype, indices=indices)
            else:
                seg = quantize(page, self.dt, bits=cfg.kbits, group_size=cfg.kgroup, md=cfg.metadata_dtype, axis=-2)
            self.key_segments.append(seg)

    # cache.py:505-542
    def _quantize_value_segment(self, v: np.ndarray) -> None:
        cfg = self.config
        seg = quantize(v, self.dt, bits=cfg.vbits, group_size=cfg.vgroup, md=cfg.metadata_dtype)
        if not self.value_segments or isinstance(self.value_segments[-1], np.ndarray):
            self.value_segments.append(seg)
            return
        prev = self.value_segments[-1]
        if prev.original_shape[-2] == cfg.page_size:
            self.value_segments.append(seg)
            return
        merged = _merge_q(prev, seg)
        total = merged.original_shape[-2]
        self.value_segments[-1] = _slice_q(merged, 0, min(cfg.page_size, total))
        if total > cfg.page_size:
            self.value_segments.append(_slice_q(merged, cfg.page_size, total))

    # cache.py:192-199
    def get(self) -> Tuple[np.ndarray, np.ndarray]:
        if self.seen_tokens == 0:
            raise RuntimeError("DartKVCache is empty; call update() before get()")
        ks = [materialize(s) for s in self.key_segments]
        vs = [materialize(s) for s in self.value_segments]
        if self.pending_key is not None:
            ks.append(self.pending_key)
        if self.pending_value is not None:
            vs.append(self.pending_value)
        return np.concatenate(ks, axis=-2), np.concatenate(vs, axis=-2)

    # cache.py:209-227
    @property
    def storage_bytes(self) -> int:
        total = sum(segment_nbytes(s, self.dt) for s in (*self.key_segments, *self.value_segments))
        for pending in (self.pending_key, self.pending_value):
            if pending is not None:
                total += int(pending.size) * _ELEM_BYTES[self.dt]
        return total

    @property
    def dense_bytes(self) -> int:
        if self.shape3 is None:
            return 0
        b, h, d = self.shape3
        return 2 * b * h * self.seen_tokens * d * _ELEM_BYTES[self.dt]

    # cache.py:229-274
    def iter_segments(self) -> List[Tuple[Segment, Segment]]:
        ks = list(self.key_segments)
        vs = list(self.value_segments)
        if self.pending_key is not None:
            ks.append(self.pending_key)
        if self.pending_value is not None:
            vs.append(self.pending_value)
        if not ks or not vs:
            return []
        pairs = []
        ki = vi = ko = vo = 0
        while ki < len(ks) and vi < len(vs):
            kl, vl = segment_tokens(ks[ki]), segment_tokens(vs[vi])
            take = min(kl - ko, vl - vo)
            pairs.append((self._slice(ks[ki], ko, ko + take), self._slice(vs[vi], vo, vo + take)))
            ko += take
            vo += take
            if ko == kl:
                ki, ko = ki + 1, 0
            if vo == vl:
                vi, vo = vi + 1, 0
        return pairs

    @staticmethod
    def _slice(seg: Segment, start: int, stop: int) -> Segment:
        if start == 0 and stop == segment_tokens(seg):
            return seg
        return np.ascontiguousarray(materialize(seg)[..., start:stop, :])

    def segment_table(self) -> List[Tuple[int, int, int, int]]:
        """(sequence_start, token_count, key_mode, value_mode); modes as page_table.py:24-26."""

        rows, start = [], 0
        for k, v in self.iter_segments():
            n = segment_tokens(k)
            rows.append((start, n, _mode(k), _mode(v)))
            start += n
        return rows


def _mode(seg: Segment) -> int:
    if isinstance(seg, np.ndarray):
        return 0
    return 2 if isinstance(seg, MixedKey) else 1


# --------------------------------------------------------------------------- attention
def dense_attention(query: np.ndarray, keys: np.ndarray, values: np.ndarray, q_dt: str,
                    scale: Optional[float] = None) -> np.ndarray:
    """attention.py:14-29 (fp32 softmax attention, result rounded to the query dtype)."""

    q = np.asarray(query, dtype=np.float32)
    k = np.asarray(keys, dtype=np.float32)
    v = np.asarray(values, dtype=np.float32)
    factor = np.float32(scale if scale is not None else 1.0 / np.sqrt(q.shape[-1]))
    logits = np.matmul(q, np.swapaxes(k, -1, -2)) * factor
    logits = logits - logits.max(axis=-1, keepdims=True)
    w = np.exp(logits)
    w = w / w.sum(axis=-1, keepdims=True)
    return round_to(np.matmul(w, v), q_dt)


def streamed_attention(query: np.ndarray, cache: OracleCache, q_dt: str, scale: Optional[float] = None,
                       *, flavour: str = "cpu", return_f32: bool = False,
                       row_start: Optional[np.ndarray] = None) -> np.ndarray:
    """attention.py:32-87: per-segment dequantize + fp32 online softmax, GQA by contiguous head groups.

    ``row_start`` ([B] ints) is not in the reference, whose streamed path takes no mask: tokens before a batch
    row's first live one get logit -inf, the additive mask the model's dense attention would apply to a
    left-padded batch.
    """

    q = np.asarray(query, dtype=np.float32)
    if q.ndim != 4:
        raise ValueError("query must have shape [B, Hq, Q, D]")
    if cache.seen_tokens == 0 or cache.shape3 is None:
        raise ValueError("cache is empty")
    b, h, d = cache.shape3
    if q.shape[0] != b or q.shape[-1] != d:
        raise ValueError("query batch and head_dim must match the cache")
    hq = q.shape[1]
    if hq % h:
        raise ValueError("query heads must be divisible by cache KV heads")
    rep = hq // h
    factor = np.float32(scale if scale is not None else 1.0 / np.sqrt(d))
    qg = q.reshape(b, h, rep, q.shape[2], d)
    run_max = np.full((b, h, rep, q.shape[2]), -np.inf, dtype=np.float32)
    run_sum = np.zeros_like(run_max)
    run_val = np.zeros((b, h, rep, q.shape[2], d), dtype=np.float32)
    seen = 0
    for kseg, vseg in cache.iter_segments():
        k = materialize(kseg, flavour).astype(np.float32)
        v = materialize(vseg, flavour).astype(np.float32)
        logits = np.einsum("bhrqd,bhtd->bhrqt", qg, k, optimize=True).astype(np.float32) * factor
        if row_start is not None:
            positions = seen + np.arange(k.shape[2])
            dead = positions[None, :] < np.asarray(row_start).reshape(b, 1)
            logits = np.where(dead[:, None, None, None, :], np.float32(-np.inf), logits)
        seen += k.shape[2]
        page_max = logits.max(axis=-1)
        new_max = np.maximum(run_max, page_max)
        ref_max = np.where(np.isneginf(new_max), np.float32(0), new_max)   # nothing live yet: all weights zero
        old_w = np.exp(run_max - ref_max)
        w = np.exp(logits - ref_max[..., None])
        run_val = run_val * old_w[..., None] + np.einsum("bhrqt,bhtd->bhrqd", w, v, optimize=True).astype(np.float32)
        run_sum = run_sum * old_w + w.sum(axis=-1)
        run_max = new_max
    out = (run_val / np.maximum(run_sum, np.float32(1e-20))[..., None]).reshape(b, hq, q.shape[2], d)
    return out if return_f32 else round_to(out, q_dt)
