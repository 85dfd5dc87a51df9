"""Adapters that let the UNMODIFIED reference package run against the Transformers release in this image.
TEST INFRASTRUCTURE ONLY: used by the fixture generators and the reference legs of the benchmark.

The reference pins transformers 4.53; two call sites differ in 5.x.  Both are patched from outside the package:

* ``Cache.__init__`` now requires ``layers`` (or a layer class): ``DartHFCache.__init__``
  (``src/dart/integrations/huggingface.py:32-37``) calls it with no argument;
* decoder layers pass the cache as ``past_key_values=`` and no longer as ``past_key_value=``
  (``src/dart/integrations/qwen3.py:37-45``).

No arithmetic is touched: the cache, the quantizers and the attention functions the hook reaches are the
reference's own.
"""

from __future__ import annotations


def patch_reference_integrations(dart) -> None:
    """Apply both adapters to an imported reference package (idempotent)."""

    from transformers.cache_utils import Cache

    from dart.integrations import huggingface as hf
    from dart.integrations import qwen3 as hook

    if getattr(hf.DartHFCache, "_compat_patched", False):
        return

    def cache_init(self, config=None):
        try:
            Cache.__init__(self)
        except (TypeError, ValueError):
            Cache.__init__(self, layers=[])
        self.dart_config = config or dart.DartKVCacheConfig()
        self._layers = {}
        self._last_update_prefill = {}
        self._seen_tokens = 0

    hf.DartHFCache.__init__ = cache_init
    hf.DartHFCache._compat_patched = True

    build_original = hook.build_dart_qwen3_attention_class

    def build_patched():
        base = build_original()

        class Adapted(base):
            def forward(self, hidden_states, position_embeddings, attention_mask=None, past_key_values=None,
                        past_key_value=None, cache_position=None, **kwargs):
                cache = past_key_values if past_key_values is not None else past_key_value
                return base.forward(self, hidden_states, position_embeddings, attention_mask, past_key_value=cache,
                                    cache_position=cache_position, **kwargs)

        Adapted.__name__ = base.__name__
        return Adapted

    hook.build_dart_qwen3_attention_class = build_patched
