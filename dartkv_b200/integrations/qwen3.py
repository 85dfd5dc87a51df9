"""Qwen3 attention adapter that decodes straight from the packed Dart cache.

Mirrors ``src/dart/integrations/qwen3.py:30-124`` of the reference: prefill goes through the
model's regular attention backend, one-token decode steps call ``fused_dart_attention`` on the
layer's packed pages.  The forward accepts both spellings of the cache argument
(``past_key_value`` up to Transformers 4.5x, ``past_key_values`` from 5.x on).
"""

from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from ..fused_attention import fused_dart_attention
from .huggingface import DartHFCache


def _qwen3_modules():
    from transformers.models.qwen3 import modeling_qwen3 as modules

    return modules


def decode_row_start(cache, attention_mask: Optional[torch.Tensor], kv_len: int):
    """What a decode step's attention mask means for the packed path.

    ``None``: nothing is masked.  An int32 ``[B]`` tensor: a left-padded batch, the first live token of every row
    (what ``fused_dart_attention(row_start=...)`` takes).  ``False``: any other mask, which only the dense path
    can honour.  The reference's adapter ignores the mask (``src/dart/integrations/qwen3.py:78-87``) and is
    therefore limited to uniform-length batches.  Telling the cases apart costs one host read per decode step:
    every layer of the step receives the same mask tensor, so the answer is kept on the cache object.
    """

    if attention_mask is None:
        return None
    key = (attention_mask.data_ptr(), tuple(attention_mask.shape), attention_mask._version)
    memo = getattr(cache, "_decode_mask_memo", None)
    if memo is not None and memo[0] == key:
        return memo[1]
    mask = attention_mask
    result = False
    if mask.ndim == 4:
        mask = mask[:, 0, -1, :]
    if mask.ndim == 2 and mask.shape[-1] >= kv_len:
        mask = mask[:, :kv_len]
        if mask.dtype == torch.bool:
            live = mask
        elif mask.dtype.is_floating_point:
            live = mask > torch.finfo(mask.dtype).min / 2      # additive mask: 0 where live
        else:
            live = mask != 0
        count = live.sum(-1)
        first = live.int().argmax(-1)
        unmasked, left_padded = torch.stack(
            [(count == kv_len).all(), ((first + count == kv_len) & (count > 0)).all()]).tolist()
        if unmasked:
            result = None
        elif left_padded:
            result = first.to(torch.int32)
    cache._decode_mask_memo = (key, result)
    return result


def build_dart_qwen3_attention_class():
    """Build the Qwen3 attention subclass against the installed Transformers."""

    modules = _qwen3_modules()
    base = modules.Qwen3Attention

    class _DartQwen3Attention(base):
        def forward(self, hidden_states: torch.Tensor, position_embeddings, attention_mask: Optional[torch.Tensor] = None,
                    past_key_values=None, cache_position: Optional[torch.LongTensor] = None, past_key_value=None,
                    **kwargs):
            cache = past_key_values if past_key_values is not None else past_key_value
            input_shape = hidden_states.shape[:-1]
            hidden_shape = (*input_shape, -1, self.head_dim)
            query_states = self.q_norm(self.q_proj(hidden_states).view(hidden_shape)).transpose(1, 2)
            key_states = self.k_norm(self.k_proj(hidden_states).view(hidden_shape)).transpose(1, 2)
            value_states = self.v_proj(hidden_states).view(hidden_shape).transpose(1, 2)
            cos, sin = position_embeddings
            query_states, key_states = modules.apply_rotary_pos_emb(query_states, key_states, cos, sin)

            use_dart_decode = isinstance(cache, DartHFCache)
            output_attentions = bool(kwargs.get("output_attentions", False))
            if (use_dart_decode and (cache.graph_decode or cache.planned_decode is not None)
                    and query_states.shape[-2] == 1 and not output_attentions and cache.has_layer(self.layer_idx)):
                # cache update + packed attention of the step in one call (a CUDA graph per layer after the first
                # steps, or part of a whole-step graph of DartGraphedDecoder, which cannot look into the mask)
                layer = cache.layer_for_attention(self.layer_idx)
                if cache.planned_decode is not None:
                    row_start = cache.planned_decode if torch.is_tensor(cache.planned_decode) else None
                else:
                    row_start = decode_row_start(cache, attention_mask, layer.get_seq_length() + 1)
                if row_start is not False:
                    attn_output = cache.decode_step(query_states, key_states, value_states, self.layer_idx,
                                                    scale=self.scaling, row_start=row_start).transpose(1, 2)
                    attn_output = attn_output.reshape(*input_shape, -1).contiguous()
                    return self.o_proj(attn_output), None
            if cache is not None:
                if use_dart_decode:
                    cache_kwargs = {"sin": sin, "cos": cos, "cache_position": cache_position, "dart_fused_attention": True}
                    key_states, value_states = cache.update(key_states, value_states, self.layer_idx, cache_kwargs)
                else:
                    key_states, value_states = cache.update(key_states, value_states, self.layer_idx)

            fused_decode = (use_dart_decode and not cache.last_update_was_prefill(self.layer_idx)
                            and query_states.shape[-2] == 1 and not output_attentions)
            row_start = None
            if fused_decode:
                layer = cache.layer_for_attention(self.layer_idx)
                row_start = decode_row_start(cache, attention_mask, layer.get_seq_length())
                if row_start is False:
                    # a mask the packed path cannot express: dense attention over the materialized layer
                    fused_decode = False
                    key_states, value_states = layer.get()
            if fused_decode:
                attn_output = fused_dart_attention(
                    query_states, layer, scale=self.scaling, fallback=True, row_start=row_start,
                ).transpose(1, 2).contiguous()
                attn_weights = None
            else:
                interface = modules.eager_attention_forward
                if self.config._attn_implementation != "eager":
                    interface = modules.ALL_ATTENTION_FUNCTIONS[self.config._attn_implementation]
                attn_output, attn_weights = interface(
                    self, query_states, key_states, value_states, attention_mask,
                    dropout=0.0 if not self.training else self.attention_dropout, scaling=self.scaling,
                    sliding_window=self.sliding_window, **kwargs)
            attn_output = attn_output.reshape(*input_shape, -1).contiguous()
            return self.o_proj(attn_output), attn_weights

    _DartQwen3Attention.__name__ = "DartQwen3Attention"
    return _DartQwen3Attention


def attach_dart_fused_attention(model: nn.Module) -> nn.Module:
    """Replace every Qwen3 self-attention module with the Dart adapter (weights are shared, not copied)."""

    attention_class = build_dart_qwen3_attention_class()
    layers = getattr(getattr(model, "model", None), "layers", None)
    if layers is None:
        raise TypeError("attach_dart_fused_attention expects a Qwen3 causal-LM model")
    for layer in layers:
        original = layer.self_attn
        original.__class__ = attention_class   # same parameters and buffers, new forward
    return model


__all__ = ["attach_dart_fused_attention", "build_dart_qwen3_attention_class", "decode_row_start"]
