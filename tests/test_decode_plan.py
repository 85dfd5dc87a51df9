"""The decode work split is host arithmetic: check, without a GPU, that every plan keeps a row's partials inside
the slots the workspace reserves for it, that the blocks' shares tile the units exactly, and that the workspace
bound covers every plan."""

import ctypes
import itertools

import pytest

from dartkv_b200 import _lib
from dartkv_b200._lib import LIB, CacheDesc, DecodePlanInfo, check


def make_desc(batch, heads, *, promoted=32, value_group=64, key_bits=2, value_bits=2, sink=32, dtype=_lib.BF16):
    d = CacheDesc()
    d.batch, d.kv_heads, d.head_dim = batch, heads, 128
    d.dtype = d.md_dtype = dtype
    d.page_size, d.key_group, d.value_group = 128, 128, value_group
    d.key_bits, d.value_bits = key_bits, value_bits
    d.key_mode = _lib.MIXED_PAGE if promoted else _lib.QUANTIZED_PAGE
    d.promoted = promoted
    d.sink_tokens, d.ring_tokens, d.regular_pages = sink, 128, 1
    d.max_key_pages, d.max_value_tokens = 4096, 4096 * 128
    check(LIB.dartkv_cache_geometry(ctypes.byref(d)))
    for i, name in enumerate(("k_sink", "v_sink", "k_ring", "v_ring", "k_pages", "v_codes", "v_meta", "page_start",
                              "page_tokens", "state")):
        setattr(d, name, 0x10000000 + 0x1000000 * i)   # never dereferenced: only their alignment is looked at
    return d


def block_of_unit(x, blocks, units):
    j = x * blocks // units
    if (j + 1) * units // blocks <= x:
        j += 1
    return j


def plan(d, q_dtype, hq, flavour, tokens):
    info = DecodePlanInfo()
    check(LIB.dartkv_decode_plan(ctypes.byref(d), q_dtype, hq, flavour, tokens, ctypes.byref(info)))
    return info


ROWS = [(1, 1), (1, 8), (2, 8), (3, 2), (16, 8), (32, 8), (37, 8), (128, 8), (512, 8)]
TOKENS = [1, 31, 32, 33, 159, 160, 161, 32 + 4 * 128, 32 + 5 * 128 + 77, 8192, 32768, 131072]


@pytest.mark.parametrize("split", [None, "aligned", "unaligned", "unaligned:7", "unaligned:3"])
@pytest.mark.parametrize("flavour", [_lib.DEQUANT_PER_OP, _lib.DEQUANT_FUSED])
def test_tensor_core_plans_stay_inside_their_partial_slots(flavour, split, decode_split):
    decode_split(split)
    for (batch, heads), tokens in itertools.product(ROWS, TOKENS):
        d = make_desc(batch, heads)
        info = plan(d, _lib.BF16, 4 * heads, flavour, tokens)
        assert info.kernel == (1 if flavour == _lib.DEQUANT_PER_OP else 2)
        rows = batch * heads
        pages = max(1, (tokens - 32) // 128)
        assert info.quads == (pages + 3) // 4
        assert info.units == rows * info.quads
        assert 1 <= info.stream_blocks <= info.units
        assert 2 <= info.total_splits <= 17
        # the shares tile the units
        edges = [j * info.units // info.stream_blocks for j in range(info.stream_blocks + 1)]
        assert edges[0] == 0 and edges[-1] == info.units and all(a < b for a, b in zip(edges, edges[1:]))
        # every row's dense slot + stream blocks fit its slots (first, middle and last rows are representative;
        # small cases check every row)
        sample = range(rows) if rows <= 64 else (0, 1, rows // 3, rows // 2, rows - 2, rows - 1)
        for row in sample:
            first = block_of_unit(row * info.quads, info.stream_blocks, info.units)
            last = block_of_unit(row * info.quads + info.quads - 1, info.stream_blocks, info.units)
            assert edges[first] <= row * info.quads < edges[first + 1]
            assert 1 + (last - first + 1) <= info.total_splits
        need = 16 + batch * 4 * heads * info.total_splits * (2 + 128) * 4
        assert LIB.dartkv_decode_workspace_bytes(ctypes.byref(d), 4 * heads, tokens) >= need


def test_other_geometries_take_the_general_tensor_core_kernel():
    for kwargs in (dict(value_bits=4), dict(key_bits=4, promoted=0), dict(value_group=32), dict(value_bits=8, key_bits=8, promoted=0)):
        d = make_desc(2, 2, **kwargs)
        for flavour in (_lib.DEQUANT_PER_OP, _lib.DEQUANT_FP32):
            info = plan(d, _lib.BF16, 8, flavour, 5000)
            assert info.kernel == 3 and info.stream_blocks >= 1 and info.generic_splits == 0
            assert info.quads == (max(1, (5000 - 32) // 128) + 3) // 4 and 2 <= info.total_splits <= 17
        # the unrounded flavour of these geometries has no 16-bit tile to go through: CUDA-core kernel
        info = plan(d, _lib.BF16, 8, _lib.DEQUANT_FUSED, 5000)
        assert info.kernel == 0 and info.stream_blocks == 0 and info.generic_splits >= 1
        assert info.total_splits == info.generic_splits
    d = make_desc(2, 2)
    assert plan(d, _lib.F32, 8, _lib.DEQUANT_PER_OP, 5000).kernel == 0      # query dtype differs from the cache dtype
    assert plan(d, _lib.BF16, 8, _lib.DEQUANT_FP32, 5000).kernel == 3       # the fp32 flavour of the headline geometry
    assert plan(d, _lib.BF16, 16, _lib.DEQUANT_PER_OP, 5000).kernel == 0    # 8 query heads per kv head
    d.md_dtype = _lib.F16                                                    # fp16 metadata beside a bf16 cache
    assert plan(d, _lib.BF16, 8, _lib.DEQUANT_PER_OP, 5000).kernel == 1     # the per-op kernel casts its operands
    assert plan(d, _lib.BF16, 8, _lib.DEQUANT_FP32, 5000).kernel == 3
    assert plan(d, _lib.BF16, 8, _lib.DEQUANT_FUSED, 5000).kernel == 2


def test_plan_argument_errors():
    d = make_desc(1, 2)
    info = DecodePlanInfo()
    assert LIB.dartkv_decode_plan(ctypes.byref(d), _lib.BF16, 3, 0, 100, ctypes.byref(info)) == -1
    assert LIB.dartkv_decode_plan(ctypes.byref(d), _lib.BF16, 8, 9, 100, ctypes.byref(info)) == -1
    assert LIB.dartkv_decode_plan(ctypes.byref(d), _lib.BF16, 8, 0, 0, ctypes.byref(info)) == -1


@pytest.mark.parametrize("kwargs", [dict(value_bits=4), dict(key_bits=4, promoted=0), dict(value_group=32), dict()],
                         ids=["v4", "k4", "vg32", "headline"])
def test_workspace_bound_covers_every_smaller_token_count(kwargs):
    # a workspace sized for a capacity must serve every token count up to it, for every query dtype and flavour
    # (the generic split count is not monotonic in the token count: its chunk is rounded up to whole tiles)
    for batch, heads, hq in ((2, 8, 32), (1, 8, 32), (1, 1, 4), (16, 8, 32)):
        d = make_desc(batch, heads, **kwargs)
        for capacity in (300, 3000, 4256, 8352):
            have = LIB.dartkv_decode_workspace_bytes(ctypes.byref(d), hq, capacity)
            worst = 0
            for tokens in range(1, capacity + 1, 1 if capacity <= 3000 else 7):
                for q_dtype, flavour in ((_lib.BF16, _lib.DEQUANT_PER_OP), (_lib.F32, _lib.DEQUANT_PER_OP),
                                         (_lib.BF16, _lib.DEQUANT_FUSED)):
                    info = plan(d, q_dtype, hq, flavour, tokens)
                    worst = max(worst, 16 + batch * hq * info.total_splits * (2 + 128) * 4)
            assert have >= worst, (kwargs, batch, heads, capacity, have, worst)
