"""Optional integrations with external model libraries (reference ``src/dart/integrations``)."""

from .graph_decode import DartGraphedDecoder
from .huggingface import DartHFCache
from .qwen3 import attach_dart_fused_attention, build_dart_qwen3_attention_class

__all__ = ["DartGraphedDecoder", "DartHFCache", "attach_dart_fused_attention", "build_dart_qwen3_attention_class"]
