"""Page descriptors with the reference's ``DartPageTable`` / ``DartPageRun`` interface.

Mirrors ``src/dart/page_table.py``.  The decode kernel walks device-side metadata owned by
the cache, so these objects are descriptive: they exist for callers that inspect or reorder
the logical page layout; ``uniform_quantized_runs`` stacks the run's fields page-major exactly
like the reference does.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import TYPE_CHECKING, Sequence

import torch

from .mixed import MixedQuantizedKey
from .quantization import QuantizedTensor

if TYPE_CHECKING:
    from .cache import DartKVCache

DENSE_PAGE = 0
QUANTIZED_PAGE = 1
MIXED_PAGE = 2
_VALID_PAGE_MODES = (DENSE_PAGE, QUANTIZED_PAGE, MIXED_PAGE)


@dataclass(frozen=True)
class DartPageTable:
    """Batch-indexed page descriptors on one device (reference page_table.py:30-48)."""

    page_ids: torch.Tensor
    sequence_starts: torch.Tensor
    token_counts: torch.Tensor
    key_modes: torch.Tensor
    value_modes: torch.Tensor
    valid: torch.Tensor
    seen_tokens: int
    page_size: int

    @classmethod
    def from_cache(cls, cache: "DartKVCache", *, device: torch.device | str | None = None) -> "DartPageTable":
        shape = cache.shape
        batch = shape[0] if shape is not None else 0
        rows = cache.segment_table() if shape is not None else []
        covered = sum(r[1] for r in rows)
        if covered != cache.seen_tokens:
            raise RuntimeError(f"page table covers {covered} tokens, expected {cache.seen_tokens}")
        if device is not None:
            target = torch.device(device)
        else:
            target = cache._device if cache._device is not None else torch.device("cpu")
        count = len(rows)
        page_ids = torch.arange(count, dtype=torch.int64, device=target).unsqueeze(0).expand(batch, -1).contiguous()
        return cls(
            page_ids=page_ids,
            sequence_starts=torch.tensor([r[0] for r in rows], dtype=torch.int32, device=target),
            token_counts=torch.tensor([r[1] for r in rows], dtype=torch.int32, device=target),
            key_modes=torch.tensor([r[2] for r in rows], dtype=torch.int8, device=target),
            value_modes=torch.tensor([r[3] for r in rows], dtype=torch.int8, device=target),
            valid=torch.ones((batch, count), dtype=torch.bool, device=target),
            seen_tokens=cache.seen_tokens,
            page_size=cache.config.page_size,
        )

    @property
    def batch_size(self) -> int:
        return self.page_ids.shape[0]

    @property
    def page_count(self) -> int:
        return self.page_ids.shape[1]

    @property
    def device(self) -> torch.device:
        return self.page_ids.device

    def __len__(self) -> int:
        return self.page_count

    def validate(self) -> "DartPageTable":
        """Check shape, mode, ID, order, and total-length invariants."""

        count = self.page_count
        if self.page_ids.ndim != 2 or self.valid.shape != self.page_ids.shape:
            raise ValueError("page_ids and valid must have shape [batch, page_count]")
        for name, tensor in (("sequence_starts", self.sequence_starts), ("token_counts", self.token_counts),
                             ("key_modes", self.key_modes), ("value_modes", self.value_modes)):
            if tensor.ndim != 1 or tensor.shape[0] != count:
                raise ValueError(f"{name} must have shape [page_count]")
        if self.page_size <= 0 or self.seen_tokens < 0:
            raise ValueError("page_size and seen_tokens must be non-negative/positive")
        if count == 0:
            if self.seen_tokens != 0:
                raise ValueError("an empty page table cannot cover non-empty cache")
            return self
        # one host read of the small per-page arrays instead of a sync per check
        starts = self.sequence_starts.tolist()
        counts = self.token_counts.tolist()
        expected, running = [], 0
        for n in counts:
            expected.append(running)
            running += n
        if starts != expected:
            raise ValueError("sequence_starts are not contiguous")
        if any(n <= 0 for n in counts):
            raise ValueError("token_counts must be positive")
        if running != self.seen_tokens:
            raise ValueError("token_counts do not cover seen_tokens")
        if any(m not in _VALID_PAGE_MODES for m in self.key_modes.tolist()):
            raise ValueError("key_modes contain an unsupported mode")
        if any(m not in _VALID_PAGE_MODES for m in self.value_modes.tolist()):
            raise ValueError("value_modes contain an unsupported mode")
        ids = self.page_ids[self.valid]
        if ids.numel() and (int(ids.min()) < 0 or int(ids.max()) >= count):
            raise ValueError("valid page IDs are outside the page range")
        return self

    def sequence_ranges(self) -> torch.Tensor:
        """Inclusive-exclusive ``[start, stop]`` ranges on the table device."""

        return torch.stack((self.sequence_starts, self.sequence_starts + self.token_counts), dim=-1)

    def reorder(self, batch_indices: torch.Tensor | Sequence[int]) -> "DartPageTable":
        """Reorder batch rows like a beam update without touching packed storage."""

        indices = torch.as_tensor(batch_indices, dtype=torch.long, device=self.device)
        if indices.ndim != 1:
            raise ValueError("batch_indices must be one-dimensional")
        if indices.numel() and bool(((indices < 0) | (indices >= self.batch_size)).any().item()):
            raise IndexError("batch_indices contain an invalid batch row")
        return DartPageTable(
            page_ids=self.page_ids.index_select(0, indices), sequence_starts=self.sequence_starts,
            token_counts=self.token_counts, key_modes=self.key_modes, value_modes=self.value_modes,
            valid=self.valid.index_select(0, indices), seen_tokens=self.seen_tokens, page_size=self.page_size)

    def to(self, device: torch.device | str) -> "DartPageTable":
        return DartPageTable(
            page_ids=self.page_ids.to(device), sequence_starts=self.sequence_starts.to(device),
            token_counts=self.token_counts.to(device), key_modes=self.key_modes.to(device),
            value_modes=self.value_modes.to(device), valid=self.valid.to(device), seen_tokens=self.seen_tokens,
            page_size=self.page_size)

    def uniform_quantized_runs(self, cache: "DartKVCache") -> tuple["DartPageRun", ...]:
        """Consecutive full uniform pages as page-major run tensors (reference page_table.py:181-211)."""

        rows = cache.segment_table()
        if len(rows) != self.page_count or cache.seen_tokens != self.seen_tokens:
            raise ValueError("cache and page_table describe different page lifecycles")
        segments = None
        runs: list[DartPageRun] = []
        start = 0
        page = self.page_size
        while start < len(rows):
            if not (rows[start][1] == page and rows[start][2] == QUANTIZED_PAGE and rows[start][3] == QUANTIZED_PAGE):
                start += 1
                continue
            end = start + 1
            while end < len(rows) and rows[end][1] == page and rows[end][2] == QUANTIZED_PAGE \
                    and rows[end][3] == QUANTIZED_PAGE:
                end += 1
            if segments is None:
                segments = cache.iter_segments()
            runs.append(_stack_uniform_run(self, segments[start:end], start))
            start = end
        return tuple(runs)


@dataclass(frozen=True)
class DartPageRun:
    """Page-major packed fields for one consecutive uniform quantized run."""

    first_page_index: int
    page_indices: torch.Tensor
    sequence_starts: torch.Tensor
    token_counts: torch.Tensor
    key_values: torch.Tensor
    key_scale: torch.Tensor
    key_zero_point: torch.Tensor
    value_values: torch.Tensor
    value_scale: torch.Tensor
    value_zero_point: torch.Tensor
    key_bits: int
    value_bits: int
    key_group_size: int
    value_group_size: int
    page_size: int

    @property
    def page_count(self) -> int:
        return self.page_indices.shape[0]

    @property
    def device(self) -> torch.device:
        return self.key_values.device

    def validate(self) -> "DartPageRun":
        if self.page_indices.ndim != 1:
            raise ValueError("page_indices must have shape [run_pages]")
        count = self.page_count
        if count == 0:
            raise ValueError("a page run cannot be empty")
        if self.first_page_index < 0:
            raise ValueError("first_page_index must be non-negative")
        for name, tensor in (("sequence_starts", self.sequence_starts), ("token_counts", self.token_counts)):
            if tensor.ndim != 1 or tensor.shape[0] != count:
                raise ValueError(f"{name} must have shape [run_pages]")
        for name, tensor in (("key_values", self.key_values), ("key_scale", self.key_scale),
                             ("key_zero_point", self.key_zero_point), ("value_values", self.value_values),
                             ("value_scale", self.value_scale), ("value_zero_point", self.value_zero_point)):
            if tensor.ndim < 1 or tensor.shape[0] != count:
                raise ValueError(f"{name} must be page-major with first dimension {count}")
        counts = self.token_counts.tolist()
        starts = self.sequence_starts.tolist()
        ids = self.page_indices.tolist()
        if any(n <= 0 for n in counts):
            raise ValueError("run token_counts must be positive")
        for i in range(1, count):
            if ids[i] != ids[i - 1] + 1:
                raise ValueError("page IDs in a run must be consecutive")
            if starts[i] != starts[i - 1] + counts[i - 1]:
                raise ValueError("run sequence_starts are not contiguous")
        if self.key_bits not in (2, 4, 8) or self.value_bits not in (2, 4, 8):
            raise ValueError("run bit widths must be 2, 4, or 8")
        if self.key_group_size <= 0 or self.value_group_size <= 0 or self.page_size <= 0:
            raise ValueError("run group sizes and page_size must be positive")
        return self

    def to(self, device: torch.device | str) -> "DartPageRun":
        moved = {name: getattr(self, name).to(device) for name in (
            "page_indices", "sequence_starts", "token_counts", "key_values", "key_scale", "key_zero_point",
            "value_values", "value_scale", "value_zero_point")}
        return DartPageRun(first_page_index=self.first_page_index, key_bits=self.key_bits, value_bits=self.value_bits,
                           key_group_size=self.key_group_size, value_group_size=self.value_group_size,
                           page_size=self.page_size, **moved)


def _stack_uniform_run(table: DartPageTable, segments, first_page_index: int) -> DartPageRun:
    keys = [pair[0] for pair in segments]
    values = [pair[1] for pair in segments]
    if not all(isinstance(seg, QuantizedTensor) for seg in (*keys, *values)):
        raise TypeError("uniform page runs require QuantizedTensor key/value segments")
    first_key, first_value = keys[0], values[0]
    device = first_key.values.device
    stop = first_page_index + len(segments)
    return DartPageRun(
        first_page_index=first_page_index,
        page_indices=table.page_ids[0, first_page_index:stop].to(device),
        sequence_starts=table.sequence_starts[first_page_index:stop].to(device),
        token_counts=table.token_counts[first_page_index:stop].to(device),
        key_values=torch.stack([seg.values for seg in keys], dim=0),
        key_scale=torch.stack([seg.scale for seg in keys], dim=0),
        key_zero_point=torch.stack([seg.zero_point for seg in keys], dim=0),
        value_values=torch.stack([seg.values for seg in values], dim=0),
        value_scale=torch.stack([seg.scale for seg in values], dim=0),
        value_zero_point=torch.stack([seg.zero_point for seg in values], dim=0),
        key_bits=first_key.bits, value_bits=first_value.bits, key_group_size=first_key.group_size,
        value_group_size=first_value.group_size, page_size=table.page_size).validate()


__all__ = ["DENSE_PAGE", "MIXED_PAGE", "QUANTIZED_PAGE", "DartPageTable", "DartPageRun"]
