"""dartkv_b200: the DartKV KV-cache hot path as hand-written B200 (sm_100a) CUDA kernels.

The public names are the reference package's (``src/dart/__init__.py:11-34``), so code written
against ``dart`` runs against this package by changing the import.
"""

from ._lib import DEQUANT_FP32, DEQUANT_FUSED, DEQUANT_PER_OP
from .cache import DartKVCache, DartKVCacheConfig, DartPageMetadata, DartSegmentLayout
from .attention import dense_attention, streamed_dart_attention
from .fused_attention import decode_attention, fused_dart_attention
from .page_table import DENSE_PAGE, MIXED_PAGE, QUANTIZED_PAGE, DartPageRun, DartPageTable
from .mixed import MixedQuantizedKey, channel_scores, quantize_key_mixed, select_key_channels
from .quantization import QuantizedTensor, dequantize, quantize, quantize_axis
from .triton_ops import TRITON_AVAILABLE, triton_available, triton_dequantize

__all__ = [
    "DartKVCache",
    "DartKVCacheConfig",
    "DartPageMetadata",
    "DartSegmentLayout",
    "dense_attention",
    "fused_dart_attention",
    "decode_attention",
    "DEQUANT_PER_OP",
    "DEQUANT_FP32",
    "DEQUANT_FUSED",
    "DENSE_PAGE",
    "MIXED_PAGE",
    "QUANTIZED_PAGE",
    "DartPageTable",
    "DartPageRun",
    "QuantizedTensor",
    "MixedQuantizedKey",
    "dequantize",
    "quantize",
    "quantize_axis",
    "quantize_key_mixed",
    "select_key_channels",
    "channel_scores",
    "streamed_dart_attention",
    "TRITON_AVAILABLE",
    "triton_available",
    "triton_dequantize",
]

__version__ = "0.1.0"
