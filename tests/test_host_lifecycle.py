"""Host logic that needs no GPU: the append planner against the oracle's cache lifecycle,
configuration validation, and the C ABI surface."""

import ctypes
import os
import re

import numpy as np
import pytest
import torch

import dartkv_b200 as dart
from dartkv_b200 import _lib
from dartkv_b200.lifecycle import LifecycleState, plan_append, ring_rows, segment_table
from oracle import dartkv_oracle as orc
from tests.golden.cases import CACHE_CASES

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _oracle_cfg(cfg: dart.DartKVCacheConfig) -> orc.CacheConfig:
    tag = {torch.float32: "f32", torch.float16: "f16", torch.bfloat16: "bf16"}[cfg.metadata_dtype]
    return orc.CacheConfig(
        bits=cfg.bits, group_size=cfg.group_size, sink_tokens=cfg.sink_tokens, metadata_dtype=tag,
        key_bits=cfg.key_bits, value_bits=cfg.value_bits, key_group_size=cfg.key_group_size,
        value_group_size=cfg.value_group_size, page_size=cfg.page_size, hold_partial_pages=cfg.hold_partial_pages,
        local_tokens=cfg.local_tokens, value_local_tokens=cfg.value_local_tokens, promote_ratio=cfg.promote_ratio)


def _check_sequence(cfg: dart.DartKVCacheConfig, chunks, head_dim=8):
    rng = np.random.default_rng(0)
    oracle = orc.OracleCache(_oracle_cfg(cfg), "f32")
    state = LifecycleState()
    c_cfg = _lib.LifecycleConfig(cfg.page_size, cfg.sink_tokens, cfg.local_tokens, cfg.value_local_tokens,
                                 int(cfg.hold_partial_pages))
    c_state = _lib.LifecycleStateC()
    c_plan = _lib.AppendPlan()
    for chunk in chunks:
        data = rng.standard_normal((1, 1, chunk, head_dim)).astype(np.float32)
        oracle.append(data, data)
        plan = plan_append(cfg, state, chunk)
        # the library's own planner (what dartkv_cache_append_step runs) gives the same plan and state
        assert _lib.LIB.dartkv_lifecycle_plan(ctypes.byref(c_cfg), ctypes.byref(c_state), chunk, ctypes.byref(c_plan)) == 0
        for name, _ in _lib.AppendPlan._fields_:
            if name != "reserved":
                assert getattr(c_plan, name) == getattr(plan, name), name
        assert (c_state.seen, c_state.k_packed_end, c_state.v_packed_end, c_state.key_pages) == \
            (state.seen, state.k_packed_end, state.v_packed_end, len(state.pages))
        assert plan.seen_after == oracle.seen_tokens
        # key pages: one per quantized oracle key segment, same lengths
        oracle_pages = [orc.segment_tokens(s) for s in oracle.key_segments if not isinstance(s, np.ndarray)]
        assert [n for _, n in state.pages] == oracle_pages
        pend_k = 0 if oracle.pending_key is None else oracle.pending_key.shape[-2]
        pend_v = 0 if oracle.pending_value is None else oracle.pending_value.shape[-2]
        assert state.seen - state.k_packed_end == pend_k
        assert state.seen - state.v_packed_end == pend_v
        assert segment_table(cfg, state) == oracle.segment_table()
        assert pend_k <= ring_rows(cfg) and pend_v <= ring_rows(cfg)
        # everything the plan asks the device to do stays inside the chunk or the ring
        assert plan.ring_begin >= plan.chunk_start + plan.sink_copy
        assert plan.value_begin <= plan.value_end <= plan.seen_after


@pytest.mark.parametrize("name", sorted(CACHE_CASES))
def test_planner_matches_oracle_on_golden_cases(name):
    case = CACHE_CASES[name]
    kwargs = dict(case["config"])
    kwargs["metadata_dtype"] = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[kwargs.pop("md")]
    _check_sequence(dart.DartKVCacheConfig(**kwargs), case["chunks"])


@pytest.mark.parametrize("seed", range(40))
def test_planner_matches_oracle_on_random_lifecycles(seed):
    rng = np.random.default_rng(seed)
    page = int(rng.choice([3, 4, 8]))
    mode = seed % 4
    kwargs = dict(page_size=page, sink_tokens=int(rng.integers(0, 6)), group_size=4, metadata_dtype=torch.float32,
                  promote_ratio=0.25 if seed % 3 == 0 else 0.0)
    if mode == 1:
        kwargs["hold_partial_pages"] = True
    elif mode == 2:
        kwargs["local_tokens"] = int(rng.integers(1, 2 * page))
    elif mode == 3:
        kwargs.update(hold_partial_pages=True, local_tokens=int(rng.choice([0, 1, 1, 2])),
                      value_local_tokens=int(rng.choice([page, 2 * page, 5])))
    chunks = [int(rng.integers(1, 4 * page)) if rng.random() < 0.4 else 1 for _ in range(int(rng.integers(3, 25)))]
    _check_sequence(dart.DartKVCacheConfig(**kwargs), chunks)


def test_config_validation_messages():
    # reference tests/test_cache.py and cache.py:74-99
    with pytest.raises(ValueError, match="bits"):
        dart.DartKVCacheConfig(bits=3)
    with pytest.raises(ValueError, match="group_size"):
        dart.DartKVCacheConfig(group_size=0)
    with pytest.raises(ValueError, match="sink_tokens"):
        dart.DartKVCacheConfig(sink_tokens=-1)
    with pytest.raises(ValueError, match="key_bits"):
        dart.DartKVCacheConfig(key_bits=5)
    with pytest.raises(ValueError, match="value_group_size"):
        dart.DartKVCacheConfig(value_group_size=0)
    with pytest.raises(ValueError, match="page_size"):
        dart.DartKVCacheConfig(page_size=0)
    with pytest.raises(ValueError, match="promote_bits"):
        dart.DartKVCacheConfig(promote_bits=3)
    with pytest.raises(ValueError, match="promote_ratio"):
        dart.DartKVCacheConfig(promote_ratio=1.5)
    with pytest.raises(ValueError, match="channel_selection"):
        dart.DartKVCacheConfig(channel_selection="best")
    with pytest.raises(TypeError, match="metadata_dtype"):
        dart.DartKVCacheConfig(metadata_dtype=torch.int32)
    cfg = dart.DartKVCacheConfig(bits=4, key_bits=2, value_group_size=32)
    assert (cfg.resolved_key_bits, cfg.resolved_value_bits) == (2, 4)
    assert (cfg.resolved_key_group_size, cfg.resolved_value_group_size) == (64, 32)


def test_argument_errors_come_before_any_device_work():
    # reference tests/test_quantization.py:26-34 -- same exception types and keywords, checked on the host
    with pytest.raises(ValueError, match="bits"):
        dart.quantize(torch.ones(2, 3), bits=3)
    with pytest.raises(ValueError, match="group_size"):
        dart.quantize(torch.ones(2, 3), group_size=0)
    with pytest.raises(TypeError, match="floating"):
        dart.quantize(torch.ones(2, 3, dtype=torch.int32))
    with pytest.raises(ValueError, match="B, H, T, D"):
        dart.quantize_key_mixed(torch.ones(2, 3))
    with pytest.raises(ValueError, match="promote_ratio"):
        dart.select_key_channels(torch.ones(1, 1, 2, 4), 2.0)
    cache = dart.DartKVCache()
    keys = torch.zeros(1, 1, 1, 4)
    with pytest.raises(ValueError, match="same dtype and device"):
        cache.append(keys, keys.half())
    with pytest.raises(ValueError, match="shapes must match"):
        cache.append(keys, torch.zeros(1, 1, 2, 4))
    with pytest.raises(RuntimeError, match="empty"):
        dart.DartKVCache().get()
    with pytest.raises(ValueError, match="cache is empty"):
        dart.fused_dart_attention(torch.zeros(1, 1, 2, 4), dart.DartKVCache())


def test_cpu_tensors_are_refused_not_emulated():
    with pytest.raises(RuntimeError, match="CUDA"):
        dart.quantize(torch.ones(2, 4))
    with pytest.raises(RuntimeError, match="CUDA"):
        dart.DartKVCache().append(torch.zeros(1, 1, 1, 4), torch.zeros(1, 1, 1, 4))


def test_empty_cache_descriptors():
    cache = dart.DartKVCache(dart.DartKVCacheConfig(page_size=4))
    table = cache.page_table().validate()
    assert table.page_ids.shape == (0, 0)
    assert cache.shape is None and len(cache) == 0 and cache.storage_bytes == 0 and cache.compression_ratio == 1.0
    assert cache.iter_segments() == [] and cache.page_metadata() == []


def test_shared_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "dartkv_b200.h")).read()
    declared = sorted(set(re.findall(r"\b(dartkv_[a-z_0-9]+)\s*\(", header)))
    assert declared, "no declarations found"
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert sorted(_lib.EXPORTS) == declared
    assert lib.dartkv_version() >= 100


def test_c_abi_rejects_bad_arguments_with_a_message():
    # validation happens before any CUDA call, so this runs without a GPU
    rc = _lib.LIB.dartkv_quantize(0, _lib.F32, 1, 8, 1, 8, 1, 1, 3, 4, _lib.F32, 0, 0, 0, 0, 0, 0)
    assert rc == -1 and "bits" in _lib.last_error()
    rc = _lib.LIB.dartkv_quantize(0, _lib.F32, 1, 8, 1, 8, 1, 1, 2, 0, _lib.F32, 0, 0, 0, 0, 0, 0)
    assert rc == -1 and "group_size" in _lib.last_error()
    rc = _lib.LIB.dartkv_quantize(0, 7, 1, 8, 1, 8, 1, 1, 2, 4, _lib.F32, 0, 0, 0, 0, 0, 0)
    assert rc == -1 and "floating" in _lib.last_error()
    desc = _lib.CacheDesc()
    assert _lib.LIB.dartkv_cache_geometry(ctypes.byref(desc)) == -1
    desc.batch, desc.kv_heads, desc.head_dim = 2, 8, 128
    desc.dtype = desc.md_dtype = _lib.BF16
    desc.page_size, desc.key_group, desc.value_group = 128, 128, 64
    desc.key_bits = desc.value_bits = 2
    desc.key_mode, desc.promoted, desc.sink_tokens, desc.ring_tokens = _lib.MIXED_PAGE, 32, 32, 128
    assert _lib.LIB.dartkv_cache_geometry(ctypes.byref(desc)) == 0
    # headline page: 4096 low + 1024 high + 128 index + 256 scale + 256 zero bytes; 32 + 2*2*2 bytes per value token
    assert (desc.key_page_bytes, desc.key_off_high, desc.key_off_index, desc.key_off_scale, desc.key_off_zero) == \
        (5760, 4096, 5120, 5248, 5504)
    assert (desc.value_row_bytes, desc.value_groups) == (32, 2)
