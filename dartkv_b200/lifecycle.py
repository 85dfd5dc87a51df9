"""Host-side page lifecycle: which tokens become sink rows, key pages, packed value rows or ring rows.

This is the integer bookkeeping of the reference cache (``src/dart/cache.py:168-190,403-470``)
restated as a pure function from (configuration, state, chunk length) to an append plan; the
device kernels execute the plan.  It touches no tensor, so it is testable without a GPU.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Tuple


@dataclass
class LifecycleState:
    """What the host remembers about one layer's cache.

    ``k_packed_end`` / ``v_packed_end`` are absolute token indices: tokens in
    ``[min(seen, sink_tokens), packed_end)`` are packed, later tokens sit in the dense ring.
    """

    seen: int = 0
    k_packed_end: int = 0
    v_packed_end: int = 0
    pages: List[Tuple[int, int]] = field(default_factory=list)        # key pages (first token, tokens)
    sink_pieces: List[Tuple[int, int]] = field(default_factory=list)  # one dense piece per append that fed the sink


@dataclass
class AppendPlanFields:
    chunk_start: int
    chunk_tokens: int
    sink_copy: int
    first_page: int
    num_pages: int
    page_token_start: int
    last_page_tokens: int
    value_begin: int
    value_end: int
    ring_begin: int
    seen_after: int
    k_packed_end_after: int
    v_packed_end_after: int
    key_pages_after: int
    requantize_last_page: int


def ring_rows(cfg) -> int:
    """Rows of the dense ring: enough for the largest pending/local suffix either side can hold."""

    return max(cfg.page_size + cfg.local_tokens, cfg.value_local_tokens, cfg.page_size)


def regular_pages(cfg) -> bool:
    """True when key pages are only ever produced full (held, local or Kitty lifecycles)."""

    return bool(cfg.hold_partial_pages or cfg.local_tokens or cfg.value_local_tokens)


def plan_append(cfg, state: LifecycleState, chunk_tokens: int) -> AppendPlanFields:
    """Plan one append of ``chunk_tokens`` tokens and advance ``state`` in place."""

    if chunk_tokens <= 0:
        raise ValueError("key/value sequence and head dimensions must be non-empty")
    page = cfg.page_size
    sink_total = cfg.sink_tokens
    seen = state.seen
    sink_copy = min(max(0, sink_total - seen), chunk_tokens)
    rest = chunk_tokens - sink_copy
    rest_start = seen + sink_copy
    chunk_end = seen + chunk_tokens
    if sink_copy:
        state.sink_pieces.append((seen, sink_copy))
    sink_filled_after = min(chunk_end, sink_total)
    # invariant: packed_end is the end of the packed range, or min(seen, sink_tokens) while nothing is packed
    k_end = state.k_packed_end
    v_end = state.v_packed_end
    pending_k = seen - k_end
    pending_v = seen - v_end
    first_page = len(state.pages)
    num_pages = 0
    last_page_tokens = page
    page_token_start = k_end if pending_k else rest_start
    value_begin = value_end = v_end if pending_v else rest_start
    requantize = 0
    if rest > 0:
        if cfg.value_local_tokens:
            # Kitty lifecycle (cache.py:424-470): keys page by page behind `local_tokens`,
            # values token by token behind the newest `value_local_tokens`
            if seen > 0 and pending_k == 0 and cfg.local_tokens == 1 and rest == 1 and state.pages:
                requantize = 1
            stream = pending_k + rest
            local = 0 if seen == 0 else cfg.local_tokens
            num_pages = max(0, stream - local) // page
            value_end = value_begin + max(0, pending_v + rest - cfg.value_local_tokens)
        elif cfg.hold_partial_pages or cfg.local_tokens:
            stream = pending_k + rest
            num_pages = max(0, stream - cfg.local_tokens) // page
            value_end = value_begin + num_pages * page
        else:
            num_pages = (rest + page - 1) // page
            last_page_tokens = rest - (num_pages - 1) * page
            value_end = value_begin + rest
    for i in range(num_pages):
        tokens = last_page_tokens if i == num_pages - 1 else page
        state.pages.append((page_token_start + i * page, tokens))
    if state.pages:
        k_end_after = state.pages[-1][0] + state.pages[-1][1]
    else:
        k_end_after = sink_filled_after
    if value_end > value_begin:
        v_end_after = value_end
    elif v_end > sink_total:
        v_end_after = v_end
    else:
        v_end_after = sink_filled_after
    plan = AppendPlanFields(
        chunk_start=seen, chunk_tokens=chunk_tokens, sink_copy=sink_copy, first_page=first_page, num_pages=num_pages,
        page_token_start=page_token_start, last_page_tokens=last_page_tokens, value_begin=value_begin,
        value_end=value_end, ring_begin=max(k_end_after, rest_start), seen_after=chunk_end,
        k_packed_end_after=k_end_after, v_packed_end_after=v_end_after, key_pages_after=len(state.pages),
        requantize_last_page=requantize)
    state.seen = chunk_end
    state.k_packed_end = k_end_after
    state.v_packed_end = v_end_after
    return plan


def value_segments(cfg, state: LifecycleState) -> List[Tuple[int, int]]:
    """(first token, tokens) of the packed value segments: page-sized, the last one possibly shorter
    (the coalescing rule of cache.py:514-542 makes them position-determined)."""

    out = []
    start = cfg.sink_tokens
    end = state.v_packed_end
    while start < end:
        n = min(cfg.page_size, end - start)
        out.append((start, n))
        start += n
    return out


def key_segment_list(state: LifecycleState) -> List[Tuple[int, int, int]]:
    """(first token, tokens, slot) in sequence order; slot is -1 for dense pieces (sink pieces, pending tail)."""

    out = [(s, n, -1) for s, n in state.sink_pieces]
    out += [(s, n, i) for i, (s, n) in enumerate(state.pages)]
    if state.seen > state.k_packed_end:
        out.append((state.k_packed_end, state.seen - state.k_packed_end, -1))
    return out


def value_segment_list(cfg, state: LifecycleState) -> List[Tuple[int, int, int]]:
    """(first token, tokens, packed) in sequence order, pending tail included."""

    out = [(s, n, 0) for s, n in state.sink_pieces]
    out += [(s, n, 1) for s, n in value_segments(cfg, state)]
    if state.seen > state.v_packed_end:
        out.append((state.v_packed_end, state.seen - state.v_packed_end, 0))
    return out


def segment_table(cfg, state: LifecycleState) -> List[Tuple[int, int, int, int]]:
    """(sequence_start, token_count, key_mode, value_mode) at the union of the K and V boundaries.

    Modes are numbered like the reference's page table (0 dense, 1 quantized, 2 mixed key); a
    segment cut by the other side's boundary is reported dense because it is materialized
    (cache.py:229-274, 557-560).
    """

    ks, vs = key_segment_list(state), value_segment_list(cfg, state)
    kmode = 2 if cfg.promote_ratio > 0.0 else 1
    rows = []
    ki = vi = ko = vo = 0
    start = 0
    while ki < len(ks) and vi < len(vs):
        _, klen, slot = ks[ki]
        _, vlen, packed = vs[vi]
        take = min(klen - ko, vlen - vo)
        whole_k = ko == 0 and take == klen
        whole_v = vo == 0 and take == vlen
        rows.append((start, take, kmode if (slot >= 0 and whole_k) else 0, 1 if (packed and whole_v) else 0))
        start += take
        ko += take
        vo += take
        if ko == klen:
            ki, ko = ki + 1, 0
        if vo == vlen:
            vi, vo = vi + 1, 0
    return rows
