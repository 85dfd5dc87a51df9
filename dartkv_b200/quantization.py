"""Group-wise affine quantization, B200 kernels behind the reference's function signatures.

Mirrors ``src/dart/quantization.py`` of the reference: ``quantize`` / ``quantize_axis`` /
``dequantize`` / ``QuantizedTensor`` with identical field names, shapes, byte layout and error
behaviour.  The arithmetic runs in ``libdartkv_b200.so``; tensors must live on a CUDA device.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import LIB, check, ptr, require_cuda, stream_ptr, device_guard

_SUPPORTED_BITS = (2, 4, 8)


def _validate_bits(bits: int) -> None:
    if bits not in _SUPPORTED_BITS:
        raise ValueError(f"bits must be one of {_SUPPORTED_BITS}, got {bits}")


def _numel(shape: Tuple[int, ...]) -> int:
    result = 1
    for size in shape:
        result *= size
    return result


def _metadata_dtype(data: torch.Tensor, requested: Optional[torch.dtype]) -> torch.dtype:
    if requested is not None:
        if requested not in (torch.float16, torch.bfloat16, torch.float32, torch.float64):
            raise TypeError(f"metadata dtype must be floating point, got {requested}")
        if requested == torch.float64:
            raise TypeError("metadata dtype float64 is not supported by the B200 kernels (use float32)")
        return requested
    return data.dtype if data.dtype in (torch.float16, torch.bfloat16) else torch.float32


def _pack(values: torch.Tensor, bits: int, packed_dim: int) -> torch.Tensor:
    """Pack a uint8 tensor along its final dimension (reference ``_pack``, quantization.py:25-35)."""

    _validate_bits(bits)
    device = require_cuda(values)
    vpb = 8 // bits
    n = values.shape[-1]
    if packed_dim < n or packed_dim % vpb:
        raise ValueError("packed_dim must be a multiple of the values per byte and cover the last dimension")
    flat = values.to(torch.uint8).contiguous().reshape(-1, n)
    out = torch.empty((*values.shape[:-1], packed_dim // vpb), dtype=torch.uint8, device=device)
    if packed_dim // vpb > (n + vpb - 1) // vpb:
        out.zero_()
        view = out.reshape(-1, packed_dim // vpb)[:, : (n + vpb - 1) // vpb]
        tmp = torch.empty((flat.shape[0], (n + vpb - 1) // vpb), dtype=torch.uint8, device=device)
        with device_guard(device):
            check(LIB.dartkv_pack(ptr(flat), flat.shape[0], n, bits, ptr(tmp), stream_ptr(device)))
        view.copy_(tmp)
        return out
    with device_guard(device):
        check(LIB.dartkv_pack(ptr(flat), flat.shape[0], n, bits, ptr(out), stream_ptr(device)))
    return out


def _unpack(packed: torch.Tensor, bits: int, packed_dim: int) -> torch.Tensor:
    """Unpack a bit-packed uint8 tensor along its final dimension (reference ``_unpack``, quantization.py:38-45)."""

    _validate_bits(bits)
    device = require_cuda(packed)
    flat = packed.contiguous().reshape(-1, packed.shape[-1])
    out = torch.empty((*packed.shape[:-1], packed_dim), dtype=torch.uint8, device=device)
    with device_guard(device):
        check(LIB.dartkv_unpack(ptr(flat), flat.shape[0], flat.shape[1], bits, packed_dim, ptr(out), stream_ptr(device)))
    return out


@dataclass
class QuantizedTensor:
    """A bit-packed affine-quantized tensor (fields as in the reference, quantization.py:56-79).

    ``zero_point`` stores the floating-point group minimum.  ``values`` is packed along the
    last dimension after the quantized ``axis`` has been moved last.
    """

    values: torch.Tensor
    scale: torch.Tensor
    zero_point: torch.Tensor
    original_shape: Tuple[int, ...]
    original_dim: int
    padded_dim: int
    packed_dim: int
    group_size: int
    bits: int
    output_dtype: torch.dtype
    axis: int = -1

    @property
    def groups(self) -> int:
        return (self.padded_dim + self.group_size - 1) // self.group_size

    @property
    def nbytes(self) -> int:
        return (self.values.numel() * self.values.element_size() + self.scale.numel() * self.scale.element_size()
                + self.zero_point.numel() * self.zero_point.element_size())

    @property
    def dense_nbytes(self) -> int:
        return _numel(self.original_shape) * torch.tensor([], dtype=self.output_dtype).element_size()

    @property
    def compression_ratio(self) -> float:
        return self.dense_nbytes / self.nbytes if self.nbytes else 1.0

    def dequantize(self, *, dtype: Optional[torch.dtype] = None, flavour: int = _lib.DEQUANT_PER_OP) -> torch.Tensor:
        """Reconstruct the tensor on the device of the packed values.

        ``flavour`` selects the reference's two dequantization arithmetics: per-op rounding in
        the metadata dtype (the PyTorch path, default) or one fp32 multiply-add (its Triton path).
        """

        device = require_cuda(self.values, self.scale, self.zero_point)
        out_dtype = dtype or self.output_dtype
        if out_dtype not in _lib.DTYPE_CODE:
            raise TypeError(f"unsupported output dtype {out_dtype}")
        axis = self.axis if self.axis >= 0 else len(self.original_shape) + self.axis
        outer = _numel(self.original_shape[:axis])
        inner = _numel(self.original_shape[axis + 1:])
        n = self.original_shape[axis]
        out = torch.empty(self.original_shape, dtype=out_dtype, device=device)
        values = self.values.contiguous()
        scale = self.scale.contiguous()
        zero = self.zero_point.contiguous()
        with device_guard(device):
            check(LIB.dartkv_dequantize(
                ptr(values), ptr(scale), ptr(zero), _lib.DTYPE_CODE[scale.dtype], outer, n, inner, self.bits,
                self.group_size, flavour, ptr(out), _lib.DTYPE_CODE[out_dtype], n * inner, inner, 1,
                stream_ptr(device)))
        return out

    def to(self, device: torch.device | str) -> "QuantizedTensor":
        return QuantizedTensor(
            values=self.values.to(device), scale=self.scale.to(device), zero_point=self.zero_point.to(device),
            original_shape=self.original_shape, original_dim=self.original_dim, padded_dim=self.padded_dim,
            packed_dim=self.packed_dim, group_size=self.group_size, bits=self.bits, output_dtype=self.output_dtype,
            axis=self.axis)


def quantize(
    data: torch.Tensor,
    *,
    bits: int = 2,
    group_size: int = 64,
    metadata_dtype: Optional[torch.dtype] = None,
    axis: int = -1,
    division: str = "true",
    check_finite: bool = True,
) -> QuantizedTensor:
    """Quantize ``data`` along ``axis`` (reference ``quantize``, quantization.py:134-204).

    ``division='reciprocal'`` evaluates ``range / qmax`` as ``range * (1/qmax)``, which is what
    PyTorch's CUDA kernel does for a Python-scalar divisor; the default true division matches
    the reference on CPU.  ``check_finite=False`` skips the host synchronization that the
    finite-input check needs.
    """

    _validate_bits(bits)
    if not isinstance(group_size, int) or group_size <= 0:
        raise ValueError(f"group_size must be a positive integer, got {group_size}")
    if data.ndim == 0:
        raise ValueError("quantize expects a tensor with at least one dimension")
    if not torch.is_floating_point(data):
        raise TypeError(f"quantize expects a floating-point tensor, got {data.dtype}")
    if data.shape[-1] == 0:
        raise ValueError("quantize does not support an empty final dimension")
    if not isinstance(axis, int) or not -data.ndim <= axis < data.ndim:
        raise ValueError(f"axis must be in [-{data.ndim}, {data.ndim}), got {axis}")
    if division not in ("true", "reciprocal"):
        raise ValueError("division must be 'true' or 'reciprocal'")
    if data.dtype not in _lib.DTYPE_CODE:
        raise TypeError(f"quantize supports float32, float16 and bfloat16 tensors, got {data.dtype}")
    meta_dtype = _metadata_dtype(data, metadata_dtype)
    device = require_cuda(data)
    original_shape = tuple(data.shape)
    axis = axis % data.ndim
    data = data.detach().contiguous()
    n = original_shape[axis]
    if n == 0:
        raise ValueError("quantize does not support an empty final dimension")
    outer = _numel(original_shape[:axis])
    inner = _numel(original_shape[axis + 1:])
    groups = (n + group_size - 1) // group_size
    padded_dim = groups * group_size
    vpb = 8 // bits
    packed_dim = ((padded_dim + vpb - 1) // vpb) * vpb
    moved_shape = tuple(s for i, s in enumerate(original_shape) if i != axis)
    values = torch.empty((*moved_shape, packed_dim // vpb), dtype=torch.uint8, device=device)
    scale = torch.empty((*moved_shape, groups), dtype=meta_dtype, device=device)
    zero = torch.empty((*moved_shape, groups), dtype=meta_dtype, device=device)
    flag = torch.zeros(1, dtype=torch.int32, device=device) if check_finite else None
    with device_guard(device):
        check(LIB.dartkv_quantize(
            ptr(data), _lib.DTYPE_CODE[data.dtype], outer, n, inner, n * inner, inner, 1, bits, group_size,
            _lib.DTYPE_CODE[meta_dtype], _lib.DIV_TRUE if division == "true" else _lib.DIV_RECIPROCAL,
            ptr(values), ptr(scale), ptr(zero), ptr(flag), stream_ptr(device)))
    if check_finite and int(flag.item()):
        raise ValueError("quantize expects all values to be finite")
    return QuantizedTensor(
        values=values, scale=scale, zero_point=zero, original_shape=original_shape, original_dim=n,
        padded_dim=padded_dim, packed_dim=packed_dim, group_size=group_size, bits=bits, output_dtype=data.dtype,
        axis=axis)


def dequantize(data: QuantizedTensor, *, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """Functional alias for :meth:`QuantizedTensor.dequantize`."""

    return data.dequantize(dtype=dtype)


def quantize_axis(
    data: torch.Tensor,
    axis: int,
    *,
    bits: int = 2,
    group_size: int = 64,
    metadata_dtype: Optional[torch.dtype] = None,
) -> QuantizedTensor:
    """Explicit spelling for quantization along a non-last tensor axis."""

    return quantize(data, bits=bits, group_size=group_size, metadata_dtype=metadata_dtype, axis=axis)


__all__ = ["QuantizedTensor", "dequantize", "quantize", "quantize_axis"]
