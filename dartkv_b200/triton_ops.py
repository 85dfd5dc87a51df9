"""Page dequantization entry point kept for drop-in compatibility with the reference.

The reference exposes ``triton_dequantize`` (``src/dart/triton_ops.py:310-324``), whose CUDA
path evaluates ``code * scale + zero`` in fp32 and rounds once to the output dtype.  Here the
same arithmetic is a flavour of the library's dequantize kernels; no Triton is involved.
"""

from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from .mixed import MixedQuantizedKey
from .quantization import QuantizedTensor

TRITON_AVAILABLE = False


def triton_available() -> bool:
    """Always False: this package ships CUDA kernels, not Triton programs."""

    return False


def triton_dequantize(data: QuantizedTensor | MixedQuantizedKey, *, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """fp32 single-rounding dequantization of a packed page (reference triton_ops.py:310-324)."""

    restored = data.dequantize(flavour=_lib.DEQUANT_FP32)
    return restored if dtype is None else restored.to(dtype)


__all__ = ["TRITON_AVAILABLE", "triton_available", "triton_dequantize"]
