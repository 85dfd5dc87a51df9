"""Hugging Face ``Cache`` facade over per-layer device-resident Dart caches.

Mirrors ``src/dart/integrations/huggingface.py:19-147`` of the reference: one ``DartKVCache`` per
layer, PostQuant return timing (the attention call of a step sees the K/V of that step before
they are packed), ``layer_for_attention`` / ``last_update_was_prefill`` for the fused decode hook,
page descriptors, beam reorder and byte accounting.  Works with Transformers 4.5x and 5.x, whose
``Cache`` constructors differ.
"""

from __future__ import annotations

import inspect
from typing import Dict, Optional

import torch

from ..cache import DartKVCache, DartKVCacheConfig

try:
    from transformers import Cache
except ImportError as exc:  # pragma: no cover - exercised only without the optional dependency
    raise ImportError("DartHFCache requires transformers; install the model dependencies first.") from exc


class _LayerDecodeGraph:
    """One layer's generation step as a CUDA graph: device-planned append of the new token + decode attention."""

    def __init__(self) -> None:
        self.graph = None
        self.k_in = self.v_in = self.q_in = self.out = self.row_start = None
        self.capacity = 0
        self.pointers = ()
        self.padded = False      # whether row_start currently holds a left padding

    @staticmethod
    def _pool_pointers(layer: DartKVCache):
        return tuple(pool.data_ptr() for pool in layer._pools.values())

    @classmethod
    def capture(cls, layer: DartKVCache, query, keys, values, scale: float, row_start, capacity: int):
        """Capture the step for ``layer`` with the current inputs and run it once (the caller has seen the layer
        take a device-planned append before)."""

        from ..fused_attention import fused_dart_attention

        self = cls()
        self.capacity = int(capacity)
        self.k_in, self.v_in, self.q_in = torch.empty_like(keys), torch.empty_like(values), torch.empty_like(query)
        self.out = torch.empty(query.shape[0], query.shape[1], query.shape[3], dtype=query.dtype, device=query.device)
        self.row_start = torch.zeros(query.shape[0], dtype=torch.int32, device=query.device)
        self._load(query, keys, values, row_start)
        layer.decode_workspace(query.shape[1])          # allocated outside the capture
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            layer.append_device_planned(self.k_in, self.v_in)
            fused_dart_attention(self.q_in, layer, scale=scale, fallback=False, row_start=self.row_start,
                                 token_capacity=self.capacity, out=self.out)
        self.graph = graph
        self.pointers = self._pool_pointers(layer)
        graph.replay()      # the capture recorded the step (and the bookkeeping counted it): now run it
        return self

    def _load(self, query, keys, values, row_start) -> None:
        self.q_in.copy_(query)
        self.k_in.copy_(keys)
        self.v_in.copy_(values)
        if row_start is not None:
            self.row_start.copy_(row_start)
            self.padded = True
        elif self.padded:
            self.row_start.zero_()
            self.padded = False

    def usable(self, layer: DartKVCache, query) -> bool:
        return (layer.seen_tokens + 1 <= self.capacity and query.shape == self.q_in.shape
                and self.pointers == self._pool_pointers(layer))

    def replay(self, layer: DartKVCache, query, keys, values, row_start) -> torch.Tensor:
        self._load(query, keys, values, row_start)
        layer.advance_device_planned(1)
        self.graph.replay()
        return self.output()

    def output(self) -> torch.Tensor:
        return self.out.unsqueeze(2)


class DartHFCache(Cache):
    """A Transformers cache whose layers are packed Dart caches.

    ``update`` returns dense tensors for the standard attention backends unless the caller passes
    ``{"dart_fused_attention": True}`` in ``cache_kwargs`` (the fused decode hook does), in which
    case only the new K/V come back and nothing is materialized.  ``max_tokens`` pre-sizes every
    layer's pools.  ``graph_decode=True`` (needs ``max_tokens``; not in the reference) lets the decode hook replay
    one CUDA graph per layer for the cache update and the attention of a generation step, see ``decode_step``.
    """

    is_compileable = False

    def __init__(self, config: Optional[DartKVCacheConfig] = None, *, max_tokens: Optional[int] = None,
                 graph_decode: bool = False) -> None:
        parameters = inspect.signature(Cache.__init__).parameters
        if "layers" in parameters:
            super().__init__(layers=[])      # Transformers 5.x wants an explicit (empty) layer list
        else:
            super().__init__()
        self.dart_config = config or DartKVCacheConfig()
        self._max_tokens = max_tokens
        self._layers: Dict[int, DartKVCache] = {}
        self._last_update_prefill: Dict[int, bool] = {}
        self._seen_tokens = 0
        if graph_decode and max_tokens is None:
            raise ValueError("graph_decode needs max_tokens: the pools of a captured graph cannot grow")
        self.graph_decode = bool(graph_decode)
        self._decode_graphs: Dict[int, "_LayerDecodeGraph"] = {}
        # set by DartGraphedDecoder while it runs or captures whole steps: True, or the [B] first live tokens of a
        # left-padded batch; decode steps then use device-planned appends and attention sized for max_tokens
        self.planned_decode = None

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, layer_idx: int,
               cache_kwargs: Optional[dict] = None, *args, **kwargs) -> tuple[torch.Tensor, torch.Tensor]:
        fused_update = bool(cache_kwargs and cache_kwargs.get("dart_fused_attention"))
        if layer_idx == 0:
            self._seen_tokens += key_states.shape[-2]
        layer = self._layers.get(layer_idx)
        if layer is None:
            layer = DartKVCache(self.dart_config, max_tokens=self._max_tokens)
            self._layers[layer_idx] = layer
            self._last_update_prefill[layer_idx] = True
            keys_to_return, values_to_return = key_states, value_states
        else:
            self._last_update_prefill[layer_idx] = False
            if fused_update:
                # the fused decode path reads the packed pages itself: nothing to materialize
                keys_to_return, values_to_return = key_states, value_states
            else:
                prior_keys, prior_values = layer.get()
                keys_to_return = torch.cat((prior_keys, key_states), dim=-2)
                values_to_return = torch.cat((prior_values, value_states), dim=-2)
        # append copies what it keeps (sink / ring rows) or packs it, so the inputs need no clone
        layer.append(key_states, value_states)
        return keys_to_return, values_to_return

    def decode_step(self, query_states: torch.Tensor, key_states: torch.Tensor, value_states: torch.Tensor,
                    layer_idx: int, *, scale: float, row_start: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Cache update and fused attention of one generation step of a layer: ``query [B,Hq,1,D]``, new
        ``key/value [B,H,1,D]`` -> attention output ``[B,Hq,1,D]``.

        With ``graph_decode`` the layer's first step after the prompt runs eagerly, the second tries the
        device-planned append, and the third is captured in a CUDA graph (device-planned append + decode attention
        sized for ``max_tokens``) that later steps replay: the inputs are copied into the graph's buffers, the host
        only advances its bookkeeping.  The result is a view of the graph's output
        buffer, valid until the layer's next step.  Steps the graph cannot take (the first one after the prompt,
        a configuration outside the device-planned append, tokens beyond ``max_tokens``) run eagerly.
        """

        from ..fused_attention import fused_dart_attention

        if layer_idx == 0:
            self._seen_tokens += key_states.shape[-2]
        layer = self.layer_for_attention(layer_idx)
        self._last_update_prefill[layer_idx] = False
        if self.planned_decode is not None:
            layer.append_device_planned(key_states, value_states)
            return fused_dart_attention(query_states, layer, scale=scale, fallback=False, row_start=row_start,
                                        token_capacity=self._max_tokens)
        single = key_states.shape[-2] == 1 and query_states.shape[-2] == 1
        graph = self._decode_graphs.get(layer_idx) if self.graph_decode and single else False
        if isinstance(graph, _LayerDecodeGraph):
            if graph.usable(layer, query_states):
                return graph.replay(layer, query_states, key_states, value_states, row_start)
        elif graph is None and getattr(layer, "_decoded_once", False):
            # second step after the prompt: see whether this layer takes device-planned appends at all
            try:
                layer.append_device_planned(key_states, value_states)
                self._decode_graphs[layer_idx] = "capture next"
            except ValueError:
                self._decode_graphs[layer_idx] = False      # eager from now on
                layer.append(key_states, value_states)
            return fused_dart_attention(query_states, layer, scale=scale, fallback=False, row_start=row_start)
        elif graph == "capture next" and layer.seen_tokens + 1 <= self._max_tokens:
            graph = _LayerDecodeGraph.capture(layer, query_states, key_states, value_states, scale, row_start,
                                              self._max_tokens)
            self._decode_graphs[layer_idx] = graph
            return graph.output()
        layer.append(key_states, value_states)
        layer._decoded_once = True
        return fused_dart_attention(query_states, layer, scale=scale, fallback=False, row_start=row_start)

    def advance_planned_decode_step(self) -> None:
        """Host bookkeeping of one replayed generation step (every layer appended one token on the device)."""

        self._seen_tokens += 1
        for layer in self._layers.values():
            layer.advance_device_planned(1)

    def has_layer(self, layer_idx: int) -> bool:
        """True once the layer's cache exists, i.e. after its prefill."""

        return layer_idx in self._layers

    def layer_for_attention(self, layer_idx: int) -> DartKVCache:
        """A layer's packed cache for the fused attention hook."""

        try:
            return self._layers[layer_idx]
        except KeyError as exc:
            raise RuntimeError(f"layer {layer_idx} has not been initialized") from exc

    def last_update_was_prefill(self, layer_idx: int) -> bool:
        """True when the last ``update`` of this layer was its prefill, i.e. the call that created its cache."""

        return self._last_update_prefill.get(layer_idx, False)

    def get_seq_length(self, layer_idx: Optional[int] = 0) -> int:
        if layer_idx is None:
            layer_idx = 0
        layer = self._layers.get(layer_idx)
        return layer.get_seq_length() if layer is not None else 0

    def get_max_cache_shape(self, *args, **kwargs) -> None:
        return None

    def get_mask_sizes(self, cache_position, layer_idx: int = 0):
        """(kv_length, kv_offset) for mask construction: everything cached plus the incoming tokens."""

        query_length = cache_position.shape[0] if hasattr(cache_position, "shape") else int(cache_position)
        return self.get_seq_length(layer_idx) + query_length, 0

    def page_table(self, layer_idx: int = 0, *, device: torch.device | str | None = None, rebuild: bool = False):
        layer = self._layers.get(layer_idx)
        return layer.page_table(device=device, rebuild=rebuild) if layer is not None else None

    def page_runs(self, layer_idx: int = 0, *, device: torch.device | str | None = None, rebuild: bool = False):
        layer = self._layers.get(layer_idx)
        return layer.page_runs(device=device, rebuild=rebuild) if layer is not None else None

    def reorder_cache(self, beam_idx: torch.LongTensor, *, requantize: bool = True) -> "DartHFCache":
        """Select beams.  ``requantize=True`` (default) rebuilds them from the dequantized contents like the
        reference (huggingface.py:117-127); ``requantize=False`` permutes the packed pools on the device
        instead, which keeps every packed byte and costs one gather per pool."""

        if not requantize:
            for layer in self._layers.values():
                layer.reorder_batch(beam_idx)
            self._last_update_prefill.clear()
            return self
        for layer_idx, layer in list(self._layers.items()):
            keys, values = layer.get()
            indices = beam_idx.to(keys.device)
            rebuilt = DartKVCache(self.dart_config, max_tokens=self._max_tokens)
            rebuilt.update(keys.index_select(0, indices), values.index_select(0, indices))
            self._layers[layer_idx] = rebuilt
        self._last_update_prefill.clear()
        return self

    @property
    def key_cache(self) -> list[torch.Tensor]:
        return [self._layers[index].key_states for index in sorted(self._layers)]

    @property
    def value_cache(self) -> list[torch.Tensor]:
        return [self._layers[index].value_states for index in sorted(self._layers)]

    @property
    def storage_bytes(self) -> int:
        return sum(layer.storage_bytes for layer in self._layers.values())

    @property
    def dense_bytes(self) -> int:
        return sum(layer.dense_bytes for layer in self._layers.values())

    @property
    def compression_ratio(self) -> float:
        return self.dense_bytes / self.storage_bytes if self.storage_bytes else 1.0

    def __len__(self) -> int:
        return len(self._layers)


__all__ = ["DartHFCache"]
