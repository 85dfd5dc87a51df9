"""A whole generation step of a Qwen3 model as one CUDA graph (no counterpart in the reference).

The packed cache makes this possible where the reference's cache cannot: every launch of a step has the same shape
whatever the length of the cache (the append is planned on the device, the decode attention is sized for the
capacity and reads the exact length on the device), so the model's forward for one new token is captured once and
replayed; the host only advances its copy of the four lifecycle integers per layer.
"""

from __future__ import annotations

from typing import Optional

import torch

from .huggingface import DartHFCache


class DartGraphedDecoder:
    """Greedy / sampled decoding helper: ``logits = decoder.step(token_ids)`` for ``token_ids [B, 1]``.

    ``cache`` is the ``DartHFCache(config, max_tokens=N)`` that already holds the prompt (run the prefill through the
    model as usual).  ``position_ids [B, 1]`` are the positions of the next token (default: the cache length for
    every row); ``row_start [B]`` marks left padding (first live token of every row), as the attention mask cannot
    be inspected while a stream is being captured.  The first steps run eagerly (the one-token step that
    re-quantizes a boundary page, then one warm-up step on the device-planned path), the next one is captured, and
    every later step is a replay.  The returned logits ``[B, vocab]`` are a view of the graph's output buffer, valid
    until the next step.
    """

    def __init__(self, model, cache: DartHFCache, *, position_ids: Optional[torch.Tensor] = None,
                 row_start: Optional[torch.Tensor] = None) -> None:
        if not isinstance(cache, DartHFCache) or cache._max_tokens is None:
            raise ValueError("DartGraphedDecoder needs a DartHFCache created with max_tokens")
        if len(cache) == 0:
            raise ValueError("run the prompt through the model first: the cache is empty")
        self.model, self.cache = model, cache
        first = cache.layer_for_attention(0)
        batch, device = first.shape[0], first._device
        length = cache.get_seq_length()
        self.positions = (position_ids.to(device=device, dtype=torch.long).clone() if position_ids is not None
                          else torch.full((batch, 1), length, dtype=torch.long, device=device))
        self.cache_position = torch.full((1,), length, dtype=torch.long, device=device)
        self.tokens = torch.zeros(batch, 1, dtype=torch.long, device=device)
        self.row_start = None if row_start is None else row_start.to(device=device, dtype=torch.int32).contiguous()
        self.logits = None
        self.graph = None
        self._warm = False

    # ------------------------------------------------------------------ one step, three ways
    def _forward(self) -> torch.Tensor:
        out = self.model(self.tokens, past_key_values=self.cache, use_cache=True, position_ids=self.positions,
                         cache_position=self.cache_position)
        self.positions.add_(1)
        self.cache_position.add_(1)
        return out.logits[:, -1]

    def _layers(self):
        return [self.cache.layer_for_attention(i) for i in sorted(self.cache._layers)]

    def _device_planned_ok(self) -> bool:
        if self.cache.get_seq_length() + 1 > self.cache._max_tokens:
            return False
        try:
            for layer in self._layers():
                layer._plan_device_step(1)      # raises for the step that re-quantizes a boundary page
        except ValueError:
            return False
        return True

    @torch.no_grad()
    def step(self, token_ids: torch.Tensor) -> torch.Tensor:
        self.tokens.copy_(token_ids.reshape(self.tokens.shape))
        cache = self.cache
        if self.graph is not None and cache.get_seq_length() + 1 <= cache._max_tokens:
            cache.advance_planned_decode_step()
            self.graph.replay()
            return self.logits
        if not self._device_planned_ok():
            cache.planned_decode = None          # host-planned appends: any step, pools may grow
            return self._forward()
        cache.planned_decode = self.row_start if self.row_start is not None else True
        try:
            if not self._warm:
                self._warm = True                # once eagerly: workspaces, kernel attributes, cuBLAS handles
                return self._forward()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                self.logits = self._forward()
            self.graph = graph
            graph.replay()                       # the capture recorded the step (and the bookkeeping counted it)
            return self.logits
        finally:
            if self.graph is None:
                cache.planned_decode = None


__all__ = ["DartGraphedDecoder"]
