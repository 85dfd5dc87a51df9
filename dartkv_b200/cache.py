"""Device-resident paged KV cache behind the reference's ``DartKVCache`` interface.

Mirrors ``src/dart/cache.py`` of the reference: the same configuration dataclass, the same
``append / update / get / iter_segments / page_metadata / page_table / page_runs`` surface and
the same error messages.  Storage is not a Python list of tensors: each cache owns a few pools
(sink rows, dense ring, key page slots, packed value rows) plus device-side page metadata, and
``append`` enqueues kernels that quantize and pack straight into those pools.  Segment objects
returned by ``iter_segments`` are views into the pools with the reference's field shapes.

Deviation kept on purpose: ``append`` does not synchronize with the host.  The reference's
finite-input check (``isfinite().all()``) is a device flag here; ``check_finite()`` reads it.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import TYPE_CHECKING, List, Optional, Sequence, Tuple, Union

import torch

from . import _lib
from ._lib import LIB, AppendPlan, CacheDesc, check, ptr, require_cuda, stream_ptr, device_guard
from .lifecycle import (LifecycleState, key_segment_list, plan_append, regular_pages, ring_rows, segment_table,
                        value_segment_list)
from .mixed import MixedQuantizedKey, promoted_count
from .quantization import QuantizedTensor

Segment = Union[torch.Tensor, QuantizedTensor, MixedQuantizedKey]

if TYPE_CHECKING:
    from .page_table import DartPageRun, DartPageTable


@dataclass(frozen=True)
class DartSegmentLayout:
    """Storage layout of one logical K/V segment: field names, shapes and element strides."""

    kind: str
    logical_shape: Tuple[int, ...]
    fields: Tuple[Tuple[str, Tuple[int, ...], Tuple[int, ...]], ...]


@dataclass(frozen=True)
class DartPageMetadata:
    """Sequence-order metadata for one page, sink segment, or pending buffer."""

    index: int
    sequence_start: int
    token_count: int
    key: DartSegmentLayout
    value: DartSegmentLayout


_PLAN_FIELDS = tuple(name for name, _ in AppendPlan._fields_ if name != "reserved")


@dataclass(frozen=True)
class DartKVCacheConfig:
    """Cache configuration; field for field the reference's dataclass (cache.py:45-112)."""

    bits: int = 2
    group_size: int = 64
    sink_tokens: int = 0
    metadata_dtype: torch.dtype = torch.float16
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

    def __post_init__(self) -> None:
        if self.bits not in (2, 4, 8):
            raise ValueError("bits must be one of 2, 4, or 8")
        if self.group_size <= 0:
            raise ValueError("group_size must be positive")
        if self.sink_tokens < 0:
            raise ValueError("sink_tokens must be non-negative")
        for name, value in (("key_bits", self.key_bits), ("value_bits", self.value_bits)):
            if value is not None and value not in (2, 4, 8):
                raise ValueError(f"{name} must be one of 2, 4, or 8")
        for name, value in (("key_group_size", self.key_group_size), ("value_group_size", self.value_group_size)):
            if value is not None and (not isinstance(value, int) or value <= 0):
                raise ValueError(f"{name} must be a positive integer")
        if self.page_size <= 0:
            raise ValueError("page_size must be positive")
        if not isinstance(self.local_tokens, int) or self.local_tokens < 0:
            raise ValueError("local_tokens must be a non-negative integer")
        if not isinstance(self.value_local_tokens, int) or self.value_local_tokens < 0:
            raise ValueError("value_local_tokens must be a non-negative integer")
        if self.promote_bits != 4:
            raise ValueError("the reference mixed representation currently supports promote_bits=4")
        if not 0.0 <= self.promote_ratio <= 1.0:
            raise ValueError("promote_ratio must be in [0, 1]")
        if self.channel_selection not in {"magnitude", "random", "variance"}:
            raise ValueError("channel_selection must be 'magnitude', 'random', or 'variance'")
        if self.metadata_dtype not in (torch.float16, torch.bfloat16, torch.float32, torch.float64):
            raise TypeError("metadata_dtype must be a floating-point torch dtype")

    @property
    def resolved_key_bits(self) -> int:
        return self.key_bits if self.key_bits is not None else self.bits

    @property
    def resolved_value_bits(self) -> int:
        return self.value_bits if self.value_bits is not None else self.bits

    @property
    def resolved_key_group_size(self) -> int:
        return self.key_group_size if self.key_group_size is not None else self.group_size

    @property
    def resolved_value_group_size(self) -> int:
        return self.value_group_size if self.value_group_size is not None else self.group_size


class DartKVCache:
    """Append-only KV cache with packed pages resident in device pools.

    Inputs use the Hugging Face layout ``[batch, kv_heads, sequence, head_dim]``.
    ``max_tokens`` (optional) pre-sizes the pools; they grow by doubling otherwise.
    """

    def __init__(self, config: Optional[DartKVCacheConfig] = None, *, max_tokens: Optional[int] = None) -> None:
        self.config = config or DartKVCacheConfig()
        if self.config.metadata_dtype == torch.float64:
            raise TypeError("metadata_dtype float64 is not supported by the B200 kernels (use float32)")
        self._max_tokens_hint = max_tokens
        self._reset()
        self._layout_version = 0

    def _reset(self) -> None:
        self._life = LifecycleState()
        self._shape: Optional[Tuple[int, int, int]] = None
        self._dtype: Optional[torch.dtype] = None
        self._device: Optional[torch.device] = None
        self._desc: Optional[CacheDesc] = None
        self._pools: dict = {}
        self._workspace: Optional[torch.Tensor] = None
        self._page_table_cache: dict = {}
        self._page_run_cache: dict = {}
        self._forced_indices: Optional[torch.Tensor] = None
        self._plan = AppendPlan()
        cfg = self.config
        self._c_cfg = _lib.LifecycleConfig(cfg.page_size, cfg.sink_tokens, cfg.local_tokens, cfg.value_local_tokens,
                                           int(cfg.hold_partial_pages))
        self._c_state = _lib.LifecycleStateC()

    # ------------------------------------------------------------------ simple accessors
    @property
    def seen_tokens(self) -> int:
        return self._life.seen

    @property
    def layout_version(self) -> int:
        """Monotonic descriptor version changed by append, clear, or device move."""

        return self._layout_version

    def get_seq_length(self) -> int:
        return self._life.seen

    @property
    def shape(self) -> Optional[Tuple[int, int, int, int]]:
        if self._shape is None:
            return None
        batch, heads, head_dim = self._shape
        return batch, heads, self._life.seen, head_dim

    def __len__(self) -> int:
        return self._life.seen

    @property
    def promoted_channels(self) -> int:
        if self._shape is None or self.config.promote_ratio <= 0.0:
            return 0
        return promoted_count(self._shape[2], self.config.promote_ratio)

    # ------------------------------------------------------------------ pools
    def _allocate(self, batch: int, heads: int, head_dim: int, dtype: torch.dtype, device: torch.device,
                  first_chunk: int) -> None:
        cfg = self.config
        d = CacheDesc()
        d.batch, d.kv_heads, d.head_dim = batch, heads, head_dim
        d.dtype = _lib.DTYPE_CODE[dtype]
        d.md_dtype = _lib.DTYPE_CODE[cfg.metadata_dtype]
        d.page_size = cfg.page_size
        d.key_group = cfg.resolved_key_group_size
        d.value_group = cfg.resolved_value_group_size
        d.key_bits = cfg.resolved_key_bits
        d.value_bits = cfg.resolved_value_bits
        mixed = cfg.promote_ratio > 0.0
        d.key_mode = _lib.MIXED_PAGE if mixed else _lib.QUANTIZED_PAGE
        d.promoted = promoted_count(head_dim, cfg.promote_ratio) if mixed else 0
        d.sink_tokens = cfg.sink_tokens
        d.ring_tokens = ring_rows(cfg)
        d.regular_pages = 1 if regular_pages(cfg) else 0
        d.max_key_pages = 1
        d.max_value_tokens = 1
        check(LIB.dartkv_cache_geometry(ctypes.byref(d)))
        self._desc = d
        with device_guard(device):
            self._pools = {
                "k_sink": torch.empty((batch, heads, max(1, cfg.sink_tokens), head_dim), dtype=dtype, device=device),
                "v_sink": torch.empty((batch, heads, max(1, cfg.sink_tokens), head_dim), dtype=dtype, device=device),
                "k_ring": torch.empty((batch, heads, d.ring_tokens, head_dim), dtype=dtype, device=device),
                "v_ring": torch.empty((batch, heads, d.ring_tokens, head_dim), dtype=dtype, device=device),
                "state": torch.zeros(32, dtype=torch.int32, device=device),   # 8 state words, then plan scratch
                "nonfinite": torch.zeros(1, dtype=torch.int32, device=device),
            }
        hint = self._max_tokens_hint or max(2 * first_chunk, first_chunk + 1024)
        self._ensure_capacity(-(-hint // cfg.page_size) + 1, hint)

    def _ensure_capacity(self, need_pages: int, need_rows: int) -> None:
        """(Re)allocate the key page slots / packed value rows so that they hold at least the given counts."""

        cfg, d, device = self.config, self._desc, self._device
        b, h = d.batch, d.kv_heads
        old = self._pools
        with device_guard(device):
            if "k_pages" not in old or need_pages > d.max_key_pages:
                pages = max(1, need_pages)
                k_pages = torch.empty((b, h, pages, d.key_page_bytes), dtype=torch.uint8, device=device)
                page_start = torch.zeros(pages, dtype=torch.int32, device=device)
                page_tokens = torch.zeros(pages, dtype=torch.int32, device=device)
                if "k_pages" in old:
                    n = old["k_pages"].shape[2]
                    k_pages[:, :, :n].copy_(old["k_pages"])
                    page_start[:n].copy_(old["page_start"])
                    page_tokens[:n].copy_(old["page_tokens"])
                old.update(k_pages=k_pages, page_start=page_start, page_tokens=page_tokens)
                d.max_key_pages = pages
            if "v_codes" not in old or need_rows > d.max_value_tokens:
                rows = -(-max(1, need_rows) // 128) * 128   # whole pages: keeps page slices 16-byte aligned
                v_codes = torch.empty((b, h, rows, d.value_row_bytes), dtype=torch.uint8, device=device)
                v_meta = torch.empty((b, h, rows, 2, d.value_groups), dtype=cfg.metadata_dtype, device=device)
                if "v_codes" in old:
                    n = old["v_codes"].shape[2]
                    v_codes[:, :, :n].copy_(old["v_codes"])
                    v_meta[:, :, :n].copy_(old["v_meta"])
                old.update(v_codes=v_codes, v_meta=v_meta)
                d.max_value_tokens = rows
        for name in ("k_sink", "v_sink", "k_ring", "v_ring", "k_pages", "v_codes", "v_meta", "page_start",
                     "page_tokens", "state"):
            setattr(d, name, old[name].data_ptr())
        self._workspace = None

    # ------------------------------------------------------------------ append / update
    def update(self, key_states: torch.Tensor, value_states: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Append a chunk and return the materialized cache contents."""

        self.append(key_states, value_states)
        return self.get()

    def append(self, key_states: torch.Tensor, value_states: torch.Tensor, *,
               channel_indices: Optional[torch.Tensor] = None) -> None:
        """Append a chunk: quantize + pack whatever the lifecycle releases, keep the rest dense.

        ``channel_indices`` (``[B, H, pages, K]`` int) forces the promoted channels of the key
        pages this call produces (a re-quantized boundary page first); used for byte parity
        with a recorded reference run.
        """

        self._validate_inputs(key_states, value_states)
        device = require_cuda(key_states, value_states)
        keys = key_states.detach()
        values = value_states.detach()
        if keys.stride(-1) != 1:
            keys = keys.contiguous()
        if values.stride(-1) != 1 or values.stride() != keys.stride():
            keys = keys.contiguous()
            values = values.contiguous()
        batch, heads, chunk, head_dim = keys.shape
        if self._desc is None:
            self._device = device
            self._allocate(batch, heads, head_dim, keys.dtype, device, chunk)
        # the kernels index chunk tokens with 16 bits: longer chunks are appended in pieces, which the lifecycle
        # treats exactly like one append of the whole chunk (pages are cut at the same absolute positions) as long
        # as the first piece carries the whole sink prefix
        limit = 65535 // self.config.page_size * self.config.page_size
        if chunk > limit and channel_indices is None and self.config.sink_tokens <= limit \
                and not self.config.value_local_tokens and (self.config.hold_partial_pages or self.config.local_tokens):
            for start in range(0, chunk, limit):
                self.append(keys[:, :, start:start + limit], values[:, :, start:start + limit])
            return
        if chunk > 65535:
            raise ValueError("append chunks longer than 65535 tokens must be split by the caller for this cache "
                             "configuration (its page boundaries depend on the chunk boundaries)")
        cfg = self.config
        if cfg.promote_ratio > 0.0 and cfg.channel_selection != "magnitude" and channel_indices is None:
            channel_indices = self._host_selected_indices(keys, chunk)
        d = self._desc
        plan = self._plan
        if channel_indices is None or not d.promoted:
            # common path, one call: the library plans the step from its own copy of the lifecycle state and appends.
            # It refuses (nothing launched, state unchanged) when the pools are too small: grow them and repeat.
            for attempt in range(2):
                with device_guard(device):
                    rc = LIB.dartkv_cache_append_step(
                        ctypes.byref(d), ctypes.byref(self._c_cfg), ctypes.byref(self._c_state), ptr(keys), ptr(values),
                        chunk, keys.stride(0), keys.stride(1), keys.stride(2), None, ptr(self._pools["nonfinite"]),
                        ctypes.byref(plan), stream_ptr(device))
                if rc != _lib.ELIMIT or attempt:
                    break
                rows_needed = plan.value_end - cfg.sink_tokens if plan.value_end > plan.value_begin else 0
                self._ensure_capacity(
                    2 * plan.key_pages_after if plan.key_pages_after > d.max_key_pages else d.max_key_pages,
                    2 * rows_needed if rows_needed > d.max_value_tokens else d.max_value_tokens)
            check(rc)
        else:
            # forced promoted channels: plan first (their page count has to match the step), then append
            state = _lib.LifecycleStateC(self._c_state.seen, self._c_state.k_packed_end, self._c_state.v_packed_end,
                                         self._c_state.key_pages)
            check(LIB.dartkv_lifecycle_plan(ctypes.byref(self._c_cfg), ctypes.byref(state), chunk, ctypes.byref(plan)))
            expected = plan.num_pages + plan.requantize_last_page
            idx = channel_indices.to(device=device, dtype=torch.int32).reshape(batch * heads, -1, d.promoted)
            if idx.shape[1] != expected:
                raise ValueError(f"channel_indices must carry {expected} pages, got {idx.shape[1]}")
            if plan.requantize_last_page:
                idx = torch.cat((idx[:, :1].reshape(-1), idx[:, 1:].reshape(-1)))
            idx = idx.contiguous()
            rows_needed = plan.value_end - cfg.sink_tokens if plan.value_end > plan.value_begin else 0
            if plan.key_pages_after > d.max_key_pages or rows_needed > d.max_value_tokens:
                self._ensure_capacity(
                    2 * plan.key_pages_after if plan.key_pages_after > d.max_key_pages else d.max_key_pages,
                    2 * rows_needed if rows_needed > d.max_value_tokens else d.max_value_tokens)
            with device_guard(device):
                check(LIB.dartkv_cache_append(
                    ctypes.byref(d), ctypes.byref(plan), ptr(keys), ptr(values), keys.stride(0), keys.stride(1),
                    keys.stride(2), ptr(idx), ptr(self._pools["nonfinite"]), stream_ptr(device)))
            self._c_state = state
        # the step was accepted: bring the host-side segment bookkeeping up to date from its plan
        life = self._life
        if plan.sink_copy:
            life.sink_pieces.append((plan.chunk_start, plan.sink_copy))
        page = cfg.page_size
        for i in range(plan.num_pages):
            life.pages.append((plan.page_token_start + i * page,
                               plan.last_page_tokens if i == plan.num_pages - 1 else page))
        life.seen = plan.seen_after
        life.k_packed_end = plan.k_packed_end_after
        life.v_packed_end = plan.v_packed_end_after
        self._layout_version += 1
        self._invalidate_page_descriptors()

    def append_device_planned(self, key_states: torch.Tensor, value_states: torch.Tensor) -> None:
        """``append`` whose step is planned on the device: every launch has the same shape whatever the state of the
        cache, so the call can sit in a CUDA graph (together with the decode attention) that is captured once and
        replayed for every new token.  No counterpart in the reference, whose page bookkeeping is Python.

        For the lifecycles that only pack full pages (``hold_partial_pages``, ``local_tokens``,
        ``value_local_tokens``) on the geometry of the page kernels (head_dim 128, 16-bit data, 128-token pages and
        key groups, magnitude selection) and an initialized cache: the first chunk goes through ``append``, and so
        does the one-token step that re-quantizes the boundary page right after a prompt (``ValueError`` here).  Pools cannot grow under a captured graph: create the cache
        with ``max_tokens``; outside a capture the pools grow here as in ``append``.  Under a capture this method
        records the launches once; on every replay call ``advance_device_planned(chunk)`` so that the host-side
        bookkeeping follows.
        """

        self._validate_inputs(key_states, value_states)
        device = require_cuda(key_states, value_states)
        if self._desc is None:
            raise ValueError("the first chunk of a cache goes through append(); device-planned appends follow it")
        keys, values = key_states.detach(), value_states.detach()
        if keys.stride(-1) != 1 or values.stride() != keys.stride():
            keys, values = keys.contiguous(), values.contiguous()
        cfg = self.config
        if cfg.promote_ratio > 0.0 and cfg.channel_selection != "magnitude":
            raise ValueError("device-planned appends select promoted channels by magnitude")
        chunk = keys.shape[2]
        state = self._plan_device_step(chunk)
        d = self._desc
        with device_guard(device):
            check(LIB.dartkv_cache_append_device_planned(
                ctypes.byref(d), ctypes.byref(self._c_cfg), ptr(keys), ptr(values), chunk, keys.stride(0), keys.stride(1),
                keys.stride(2), ptr(self._pools["nonfinite"]), stream_ptr(device)))
        self._commit_step(state)

    def advance_device_planned(self, chunk: int) -> None:
        """Host-side bookkeeping of one device-planned append of ``chunk`` tokens (the device plans the same step
        from its own copy of the state): call it once per replay of a graph that holds ``append_device_planned``."""

        self._commit_step(self._plan_device_step(chunk))

    def _plan_device_step(self, chunk: int):
        """The step's plan on a copy of the lifecycle state (left in ``self._plan``), pools grown if it needs that."""

        cfg, d, plan = self.config, self._desc, self._plan
        state = _lib.LifecycleStateC(self._c_state.seen, self._c_state.k_packed_end, self._c_state.v_packed_end,
                                     self._c_state.key_pages)
        check(LIB.dartkv_lifecycle_plan(ctypes.byref(self._c_cfg), ctypes.byref(state), chunk, ctypes.byref(plan)))
        if plan.requantize_last_page:
            raise ValueError("this step re-quantizes the boundary page (the first one-token append after a prompt that "
                             "ended on a page boundary): run it through append()")
        rows_needed = plan.value_end - cfg.sink_tokens if plan.value_end > plan.value_begin else 0
        if plan.key_pages_after > d.max_key_pages or rows_needed > d.max_value_tokens:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("the cache pools are too small for this step and cannot grow under a graph capture: "
                                   "create the cache with max_tokens")
            self._ensure_capacity(
                2 * plan.key_pages_after if plan.key_pages_after > d.max_key_pages else d.max_key_pages,
                2 * rows_needed if rows_needed > d.max_value_tokens else d.max_value_tokens)
        return state

    def _commit_step(self, state) -> None:
        """The step in ``self._plan`` was accepted: bring the host-side bookkeeping up to date."""

        cfg, plan = self.config, self._plan
        self._c_state = state
        life = self._life
        if plan.sink_copy:
            life.sink_pieces.append((plan.chunk_start, plan.sink_copy))
        page = cfg.page_size
        for i in range(plan.num_pages):
            life.pages.append((plan.page_token_start + i * page,
                               plan.last_page_tokens if i == plan.num_pages - 1 else page))
        life.seen = plan.seen_after
        life.k_packed_end = plan.k_packed_end_after
        life.v_packed_end = plan.v_packed_end_after
        self._layout_version += 1
        self._invalidate_page_descriptors()

    def _host_selected_indices(self, keys: torch.Tensor, chunk: int) -> Optional[torch.Tensor]:
        """Promoted channels for the 'random' and 'variance' strategies, chosen with the functional API.

        The page kernels score by magnitude only; other strategies are resolved here per new page.
        """

        from .mixed import select_key_channels

        cfg = self.config
        probe = LifecycleState(self._life.seen, self._life.k_packed_end, self._life.v_packed_end,
                               list(self._life.pages), list(self._life.sink_pieces))
        fields = plan_append(cfg, probe, chunk)
        selected = []
        if fields.requantize_last_page:
            start = fields.page_token_start - cfg.page_size
            page = self._materialize(0, start, start + cfg.page_size)
            selected.append(select_key_channels(page, cfg.promote_ratio, strategy=cfg.channel_selection)[1])
        for i in range(fields.num_pages):
            start = fields.page_token_start + i * cfg.page_size
            tokens = fields.last_page_tokens if i == fields.num_pages - 1 else cfg.page_size
            page = self._gather_tokens(keys, start, start + tokens)
            selected.append(select_key_channels(page, cfg.promote_ratio, strategy=cfg.channel_selection)[1])
        if not selected:
            return None
        return torch.stack(selected, dim=2)

    def _gather_tokens(self, chunk_keys: torch.Tensor, start: int, stop: int) -> torch.Tensor:
        """Key tokens [start, stop) from the dense ring and/or the incoming chunk."""

        seen = self._life.seen
        parts = []
        if start < seen:
            parts.append(self._materialize(0, start, min(stop, seen)))
        if stop > seen:
            parts.append(chunk_keys[..., max(start, seen) - seen: stop - seen, :])
        return torch.cat(parts, dim=-2) if len(parts) > 1 else parts[0]

    # ------------------------------------------------------------------ materialization
    def _materialize(self, side: int, start: int, stop: int, flavour: int = _lib.DEQUANT_PER_OP) -> torch.Tensor:
        b, h, d = self._shape
        out = torch.empty((b, h, stop - start, d), dtype=self._dtype, device=self._device)
        with device_guard(self._device):
            for lo in range(start, stop, 32768):
                hi = min(stop, lo + 32768)
                piece = out if (lo == start and hi == stop) else torch.empty(
                    (b, h, hi - lo, d), dtype=self._dtype, device=self._device)
                check(LIB.dartkv_cache_materialize(ctypes.byref(self._desc), side, lo, hi, flavour, ptr(piece),
                                                   _lib.DTYPE_CODE[self._dtype], stream_ptr(self._device)))
                if piece is not out:
                    out[:, :, lo - start: hi - start].copy_(piece)
        return out

    def get(self) -> Tuple[torch.Tensor, torch.Tensor]:
        if self._life.seen == 0:
            raise RuntimeError("DartKVCache is empty; call update() before get()")
        return self._materialize(0, 0, self._life.seen), self._materialize(1, 0, self._life.seen)

    @property
    def key_states(self) -> torch.Tensor:
        return self.get()[0]

    @property
    def value_states(self) -> torch.Tensor:
        return self.get()[1]

    def check_finite(self) -> None:
        """Raise if any appended value was NaN/Inf (host synchronization; the reference checks per append)."""

        if self._pools and int(self._pools["nonfinite"].item()):
            raise ValueError("quantize expects all values to be finite")

    # ------------------------------------------------------------------ byte accounting (cache.py:209-227)
    def _element_size(self) -> int:
        return torch.tensor([], dtype=self._dtype).element_size()

    @property
    def storage_bytes(self) -> int:
        if self._shape is None:
            return 0
        b, h, d = self._shape
        cfg, life, desc = self.config, self._life, self._desc
        es = self._element_size()
        mdb = torch.tensor([], dtype=cfg.metadata_dtype).element_size()
        bh = b * h
        sink = min(life.seen, cfg.sink_tokens)
        total = 2 * bh * sink * d * es
        total += bh * (life.seen - life.k_packed_end) * d * es
        total += bh * (life.seen - life.v_packed_end) * d * es
        gk = cfg.resolved_key_group_size
        for _, tokens in life.pages:
            groups = -(-tokens // gk)
            if desc.key_mode == _lib.MIXED_PAGE:
                pb = (gk + 3) // 4
                total += bh * (d * groups * pb + desc.promoted * groups * pb + desc.promoted * 4 + 2 * d * groups * mdb)
            else:
                row = -(-(groups * gk) // (8 // desc.key_bits))
                total += bh * (d * row + 2 * d * groups * mdb)
        rows = max(0, life.v_packed_end - cfg.sink_tokens)
        total += bh * rows * (desc.value_row_bytes + 2 * desc.value_groups * mdb)
        return total

    @property
    def dense_bytes(self) -> int:
        if self._shape is None or self._dtype is None:
            return 0
        batch, heads, head_dim = self._shape
        return 2 * batch * heads * self._life.seen * head_dim * self._element_size()

    @property
    def compression_ratio(self) -> float:
        return self.dense_bytes / self.storage_bytes if self.storage_bytes else 1.0

    # ------------------------------------------------------------------ segments
    def _key_segment_list(self) -> List[Tuple[int, int, int]]:
        return key_segment_list(self._life)

    def _value_segment_list(self) -> List[Tuple[int, int, int]]:
        return value_segment_list(self.config, self._life)

    def _dense_view(self, side: int, start: int, tokens: int) -> torch.Tensor:
        cfg = self.config
        if start + tokens <= min(self._life.seen, cfg.sink_tokens):
            pool = self._pools["k_sink" if side == 0 else "v_sink"]
            return pool[:, :, start:start + tokens]
        return self._materialize(side, start, start + tokens)

    def _key_page_segment(self, slot: int) -> Segment:
        cfg, d = self.config, self._desc
        b, h, hd = self._shape
        start, tokens = self._life.pages[slot]
        page = self._pools["k_pages"][:, :, slot]
        gk = d.key_group
        groups = -(-tokens // gk)
        mdb = torch.tensor([], dtype=cfg.metadata_dtype).element_size()

        def meta(offset: int) -> torch.Tensor:
            return page[..., offset: offset + hd * groups * mdb].view(cfg.metadata_dtype).reshape(b, h, hd, groups)

        if d.key_mode == _lib.MIXED_PAGE:
            pb = (gk + 3) // 4
            k = d.promoted
            low = page[..., : hd * groups * pb].reshape(b, h, hd, groups, pb)
            high = page[..., d.key_off_high: d.key_off_high + k * groups * pb].reshape(b, h, k, groups, pb)
            index = page[..., d.key_off_index: d.key_off_index + 4 * k].view(torch.int32).reshape(b, h, k)
            return MixedQuantizedKey(
                low_values=low, high_values=high, channel_indices=index, scale=meta(d.key_off_scale),
                zero_point=meta(d.key_off_zero), original_shape=(b, h, tokens, hd), padded_tokens=groups * gk,
                group_size=gk, low_bits=2, promote_bits=cfg.promote_bits, output_dtype=self._dtype)
        vpb = 8 // d.key_bits
        padded = groups * gk
        row = -(-padded // vpb)
        values = page[..., : hd * row].reshape(b, h, hd, row)
        return QuantizedTensor(
            values=values, scale=meta(d.key_off_scale), zero_point=meta(d.key_off_zero),
            original_shape=(b, h, tokens, hd), original_dim=tokens, padded_dim=padded, packed_dim=row * vpb,
            group_size=gk, bits=d.key_bits, output_dtype=self._dtype, axis=2)

    def _value_segment(self, start: int, tokens: int) -> QuantizedTensor:
        cfg, d = self.config, self._desc
        b, h, hd = self._shape
        r0 = start - cfg.sink_tokens
        vpb = 8 // d.value_bits
        padded = d.value_groups * d.value_group
        meta = self._pools["v_meta"][:, :, r0:r0 + tokens]
        return QuantizedTensor(
            values=self._pools["v_codes"][:, :, r0:r0 + tokens], scale=meta[:, :, :, 0], zero_point=meta[:, :, :, 1],
            original_shape=(b, h, tokens, hd), original_dim=hd, padded_dim=padded, packed_dim=d.value_row_bytes * vpb,
            group_size=d.value_group, bits=d.value_bits, output_dtype=self._dtype, axis=3)

    def iter_segments(self) -> list[Tuple[Segment, Segment]]:
        """Key/value pages in sequence order at the union of K and V boundaries (cache.py:229-274).

        Whole segments are views of the packed pools; a segment cut by the other side's
        boundary is materialized for that interval only, as in the reference.
        """

        if self._life.seen == 0:
            return []
        ks, vs = self._key_segment_list(), self._value_segment_list()
        pairs: list[Tuple[Segment, Segment]] = []
        ki = vi = 0
        ko = vo = 0
        while ki < len(ks) and vi < len(vs):
            kstart, klen, slot = ks[ki]
            vstart, vlen, packed = vs[vi]
            take = min(klen - ko, vlen - vo)
            if ko == 0 and take == klen:
                kseg: Segment = self._key_page_segment(slot) if slot >= 0 else self._dense_view(0, kstart, klen)
            else:
                kseg = self._materialize(0, kstart + ko, kstart + ko + take)
            if vo == 0 and take == vlen:
                vseg: Segment = self._value_segment(vstart, vlen) if packed else self._dense_view(1, vstart, vlen)
            else:
                vseg = self._materialize(1, vstart + vo, vstart + vo + take)
            pairs.append((kseg, vseg))
            ko += take
            vo += take
            if ko == klen:
                ki, ko = ki + 1, 0
            if vo == vlen:
                vi, vo = vi + 1, 0
        if ki != len(ks) or vi != len(vs):
            raise RuntimeError("DartKVCache key/value logical lengths diverged")
        return pairs

    def segment_table(self) -> List[Tuple[int, int, int, int]]:
        """(sequence_start, token_count, key_mode, value_mode) per segment pair, without touching the device."""

        return segment_table(self.config, self._life)

    def page_metadata(self) -> list[DartPageMetadata]:
        """Describe page order, logical lengths, shapes, and element strides (cache.py:276-300)."""

        metadata: list[DartPageMetadata] = []
        sequence_start = 0
        for index, (key_segment, value_segment) in enumerate(self.iter_segments()):
            key_layout = _segment_layout(key_segment)
            value_layout = _segment_layout(value_segment)
            key_tokens = key_layout.logical_shape[-2]
            if key_tokens != value_layout.logical_shape[-2]:
                raise RuntimeError("DartKVCache key/value page lengths diverged")
            metadata.append(DartPageMetadata(index=index, sequence_start=sequence_start, token_count=key_tokens,
                                             key=key_layout, value=value_layout))
            sequence_start += key_tokens
        if sequence_start != self._life.seen:
            raise RuntimeError(f"page metadata covers {sequence_start} tokens, expected {self._life.seen}")
        return metadata

    def page_table(self, *, device: torch.device | str | None = None, rebuild: bool = False) -> "DartPageTable":
        """Cached page descriptors for the current segments (cache.py:302-323)."""

        from .page_table import DartPageTable

        target = _descriptor_device(device, self._device)
        cached = self._page_table_cache.get(target)
        if cached is not None and not rebuild and cached[0] == self._layout_version:
            return cached[1]
        table = DartPageTable.from_cache(self, device=target)
        self._page_table_cache[target] = (self._layout_version, table)
        return table

    def page_runs(self, *, device: torch.device | str | None = None, page_table: Optional["DartPageTable"] = None,
                  rebuild: bool = False) -> tuple["DartPageRun", ...]:
        """Cached page-major uniform runs for the current segments (cache.py:325-352)."""

        target = _descriptor_device(device, self._device)
        if page_table is None:
            cached = self._page_run_cache.get(target)
            if cached is not None and not rebuild and cached[0] == self._layout_version:
                return cached[1]
            table = self.page_table(device=target, rebuild=rebuild)
        else:
            table = page_table
        runs = table.uniform_quantized_runs(self)
        if device is not None:
            runs = tuple(run if run.device == target else run.to(target) for run in runs)
        if page_table is None:
            self._page_run_cache[target] = (self._layout_version, runs)
        return runs

    def to(self, device: torch.device | str) -> "DartKVCache":
        """Move all pools to another CUDA device and return ``self``."""

        target = _descriptor_device(device, self._device)
        if target.type != "cuda":
            raise RuntimeError("dartkv_b200 caches live on CUDA devices only (there is no CPU fallback)")
        if self._desc is not None and target != self._device:
            self._pools = {name: tensor.to(target) for name, tensor in self._pools.items()}
            self._device = target
            for name in ("k_sink", "v_sink", "k_ring", "v_ring", "k_pages", "v_codes", "v_meta", "page_start",
                         "page_tokens", "state"):
                setattr(self._desc, name, self._pools[name].data_ptr())
            self._workspace = None
        self._layout_version += 1
        self._invalidate_page_descriptors()
        return self

    def reorder_batch(self, batch_indices: torch.Tensor | Sequence[int]) -> "DartKVCache":
        """Select / permute batch rows in place: ``row i <- row batch_indices[i]`` (beam search reorder).

        Every pool is indexed along its batch dimension on the device; packed pages, scales and
        zero points move as bytes, so nothing is dequantized or quantized again (the reference's
        ``DartPageTable.reorder`` describes the same permutation, ``page_table.py:148-165``).
        The number of rows may change; page metadata is shared by all rows and stays as it is.
        """

        if self._desc is None:
            return self
        indices = torch.as_tensor(batch_indices, dtype=torch.long, device=self._device).reshape(-1)
        if indices.numel() == 0:
            raise ValueError("batch_indices must not be empty")
        batch = self._desc.batch
        if int(indices.min()) < 0 or int(indices.max()) >= batch:
            raise IndexError(f"batch_indices must lie in [0, {batch})")
        with device_guard(self._device):
            for name in ("k_sink", "v_sink", "k_ring", "v_ring", "k_pages", "v_codes", "v_meta"):
                self._pools[name] = self._pools[name].index_select(0, indices)
                setattr(self._desc, name, self._pools[name].data_ptr())
        self._desc.batch = int(indices.numel())
        self._shape = (self._desc.batch, self._shape[1], self._shape[2])
        self._workspace = None
        self._layout_version += 1
        self._invalidate_page_descriptors()
        return self

    def clear(self) -> None:
        self._reset()
        self._layout_version += 1

    def _invalidate_page_descriptors(self) -> None:
        self._page_table_cache.clear()
        self._page_run_cache.clear()

    def _validate_inputs(self, key_states: torch.Tensor, value_states: torch.Tensor) -> None:
        if key_states.ndim != 4 or value_states.ndim != 4:
            raise ValueError("key_states and value_states must have shape [B, H, T, D]")
        if key_states.shape != value_states.shape:
            raise ValueError(f"key/value shapes must match, got {key_states.shape} and {value_states.shape}")
        if key_states.dtype != value_states.dtype or key_states.device != value_states.device:
            raise ValueError("key_states and value_states must use the same dtype and device")
        if key_states.shape[-2] == 0 or key_states.shape[-1] == 0:
            raise ValueError("key/value sequence and head dimensions must be non-empty")
        if not torch.is_floating_point(key_states) or not torch.is_floating_point(value_states):
            raise TypeError("key_states and value_states must be floating-point tensors")
        if key_states.dtype not in _lib.DTYPE_CODE:
            raise TypeError("key_states and value_states must be float32, float16 or bfloat16")
        shape = (key_states.shape[0], key_states.shape[1], key_states.shape[3])
        if self._shape is None:
            self._shape = shape
            self._dtype = key_states.dtype
            self._device = key_states.device
        elif shape != self._shape or key_states.dtype != self._dtype or key_states.device != self._device:
            raise ValueError("all updates must keep batch/head/head_dim, dtype, and device unchanged")

    # ------------------------------------------------------------------ attention support
    def decode_workspace(self, query_heads: int) -> Tuple[torch.Tensor, int]:
        """Split-K scratch for the decode kernel and the token capacity it was sized for."""

        d = self._desc
        capacity = self.config.sink_tokens + max(d.max_value_tokens, d.max_key_pages * self.config.page_size) \
            + d.ring_tokens
        key = (query_heads, capacity)
        if self._workspace is None or self._workspace[0] != key:
            nbytes = LIB.dartkv_decode_workspace_bytes(ctypes.byref(d), query_heads, capacity)
            with device_guard(self._device):
                buf = torch.zeros(max(16, nbytes), dtype=torch.uint8, device=self._device)
            self._workspace = (key, buf)
        return self._workspace[1], capacity

    def decode_status(self) -> int:
        """0 unless a decode kernel gave up on a bounded wait for an async copy (synchronizes)."""

        if self._workspace is None:
            return 0
        status = ctypes.c_int(0)
        with device_guard(self._device):
            check(LIB.dartkv_decode_status(ptr(self._workspace[1]), ctypes.byref(status), stream_ptr(self._device)))
        return status.value

    @property
    def descriptor(self) -> CacheDesc:
        if self._desc is None:
            raise ValueError("cache is empty")
        return self._desc


def _segment_layout(segment: Segment) -> DartSegmentLayout:
    if isinstance(segment, torch.Tensor):
        fields = (("values", tuple(segment.shape), tuple(segment.stride())),)
        return DartSegmentLayout("dense", tuple(segment.shape), fields)
    if isinstance(segment, QuantizedTensor):
        fields = tuple((name, tuple(t.shape), tuple(t.stride())) for name, t in (
            ("values", segment.values), ("scale", segment.scale), ("zero_point", segment.zero_point)))
        return DartSegmentLayout("quantized", segment.original_shape, fields)
    fields = tuple((name, tuple(t.shape), tuple(t.stride())) for name, t in (
        ("low_values", segment.low_values), ("high_values", segment.high_values),
        ("channel_indices", segment.channel_indices), ("scale", segment.scale), ("zero_point", segment.zero_point)))
    return DartSegmentLayout("mixed_key", segment.original_shape, fields)


def _descriptor_device(device: torch.device | str | None, fallback: Optional[torch.device]) -> torch.device:
    target = torch.device(device) if device is not None else (fallback or torch.device("cpu"))
    if target.type == "cuda" and target.index is None:
        target = torch.device("cuda", torch.cuda.current_device())
    return target


__all__ = ["DartKVCache", "DartKVCacheConfig", "DartPageMetadata", "DartSegmentLayout"]
