"""The device-resident cache and the fused decode attention against the reference's golden
vectors (packed bytes, scales, zero points, materialized tensors, attention outputs) and the oracle."""

import copy
import hashlib

import numpy as np
import pytest
import torch

import dartkv_b200 as dart
from dartkv_b200.lifecycle import plan_append
from dartkv_b200.synthetic import make_kvq
from oracle import dartkv_oracle as orc
from tests.golden.cases import CACHE_CASES, TORCH_DTYPES, build_inputs
from tests.helpers import load_golden, to_np

pytestmark = pytest.mark.gpu

CACHES = load_golden("caches.npz")
CUDA_GOLD = load_golden("cuda_reference.npz")


def sha(*arrays):
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def make_config(case):
    kwargs = dict(case["config"])
    kwargs["metadata_dtype"] = TORCH_DTYPES[kwargs.pop("md")]
    return dart.DartKVCacheConfig(**kwargs)


def build_cache(name, inject=True):
    """Replay a golden case on the GPU; ``inject`` feeds the promoted channels the reference run chose."""

    case = CACHE_CASES[name]
    keys, values, query = build_inputs(case)
    cfg = make_config(case)
    cache = dart.DartKVCache(cfg)
    ref_idx = CACHES.get(f"cache/{name}/mixed_indices") if inject else None
    used = 0
    start = 0
    for chunk in case["chunks"]:
        forced = None
        if ref_idx is not None:
            probe = copy.deepcopy(cache._life)
            plan = plan_append(cfg, probe, chunk)
            count = plan.num_pages + plan.requantize_last_page
            if count:
                forced = torch.from_numpy(ref_idx[used:used + count]).permute(1, 2, 0, 3).contiguous()  # [B,H,pages,K]
                used += count
        cache.append(keys[..., start:start + chunk, :].cuda(), values[..., start:start + chunk, :].cuda(),
                     channel_indices=forced)
        start += chunk
    if ref_idx is not None:
        assert used == len(ref_idx)
    return case, cache, keys, values, query


def key_fields(seg):
    if isinstance(seg, torch.Tensor):
        return [to_np(seg)]
    if isinstance(seg, dart.MixedQuantizedKey):
        return [to_np(seg.low_values), to_np(seg.high_values), to_np(seg.channel_indices), to_np(seg.scale),
                to_np(seg.zero_point)]
    return [to_np(seg.values), to_np(seg.scale), to_np(seg.zero_point)]


def cache_owned_segments(cache):
    """The cache-owned K and V segment lists (before the boundary union), like the reference's private lists."""

    sink = set(cache._life.sink_pieces)
    ks = []
    for start, tokens, slot in cache._key_segment_list():
        if slot >= 0:
            ks.append(cache._key_page_segment(slot))
        elif (start, tokens) in sink:
            ks.append(cache._dense_view(0, start, tokens))
    vs = []
    for start, tokens, packed in cache._value_segment_list():
        if packed:
            vs.append(cache._value_segment(start, tokens))
        elif (start, tokens) in sink:
            vs.append(cache._dense_view(1, start, tokens))
    return ks, vs


@pytest.mark.parametrize("name", sorted(CACHE_CASES))
def test_cache_bytes_match_reference(name):
    case, cache, keys, values, query = build_cache(name, inject=True)
    prefix = f"cache/{name}"
    cache.check_finite()
    assert cache.storage_bytes == int(CACHES[f"{prefix}/storage_bytes"])
    assert cache.dense_bytes == int(CACHES[f"{prefix}/dense_bytes"])
    table = cache.page_table().validate()
    got = np.stack([to_np(table.sequence_starts), to_np(table.token_counts), to_np(table.key_modes).astype(np.int32),
                    to_np(table.value_modes).astype(np.int32)], axis=1)
    np.testing.assert_array_equal(got, CACHES[f"{prefix}/table"])
    ks, vs = cache_owned_segments(cache)
    key_rows = CACHES[f"{prefix}/key_segments"]
    value_rows = CACHES[f"{prefix}/value_segments"]
    assert len(ks) == len(key_rows) and len(vs) == len(value_rows)
    for i, seg in enumerate(ks):
        assert sha(*key_fields(seg)) == str(CACHES[f"{prefix}/k{i}/sha"]), f"key segment {i}"
    for i, seg in enumerate(vs):
        assert sha(*key_fields(seg)) == str(CACHES[f"{prefix}/v{i}/sha"]), f"value segment {i}"
    pend = CACHES[f"{prefix}/pending"]
    assert cache.seen_tokens - cache._life.k_packed_end == int(pend[0])
    assert cache.seen_tokens - cache._life.v_packed_end == int(pend[1])
    got_k, got_v = cache.get()
    assert got_k.dtype == keys.dtype and tuple(got_k.shape) == tuple(keys.shape)
    assert sha(to_np(got_k), to_np(got_v)) == str(CACHES[f"{prefix}/get_sha"])


@pytest.mark.parametrize("name", sorted(CACHE_CASES))
def test_cache_own_channel_selection_matches_oracle(name):
    """Without injected channels the kernels select by (score desc, channel asc), exactly like the oracle."""

    case, cache, keys, values, query = build_cache(name, inject=False)
    cfg = dict(case["config"])
    cfg["metadata_dtype"] = cfg.pop("md")
    oracle = orc.OracleCache(orc.CacheConfig(**cfg), case["dt"])
    start = 0
    for chunk in case["chunks"]:
        oracle.append(to_np(keys[..., start:start + chunk, :]), to_np(values[..., start:start + chunk, :]))
        start += chunk
    ks, vs = cache_owned_segments(cache)
    assert len(ks) == len(oracle.key_segments) and len(vs) == len(oracle.value_segments)
    for i, (mine, ref) in enumerate(zip(ks, oracle.key_segments)):
        if isinstance(ref, np.ndarray):
            ref_fields = [ref]
        elif isinstance(ref, orc.MixedKey):
            ref_fields = [ref.low_values, ref.high_values, ref.channel_indices, ref.scale, ref.zero_point]
        else:
            ref_fields = [ref.values, ref.scale, ref.zero_point]
        for a, b in zip(key_fields(mine), ref_fields):
            np.testing.assert_array_equal(a, b, err_msg=f"key segment {i}")
    for i, (mine, ref) in enumerate(zip(vs, oracle.value_segments)):
        ref_fields = [ref] if isinstance(ref, np.ndarray) else [ref.values, ref.scale, ref.zero_point]
        for a, b in zip(key_fields(mine), ref_fields):
            np.testing.assert_array_equal(a, b, err_msg=f"value segment {i}")
    ok, ov = oracle.get()
    gk, gv = cache.get()
    np.testing.assert_array_equal(to_np(gk), ok)
    np.testing.assert_array_equal(to_np(gv), ov)
    out = dart.fused_dart_attention(query.float().cuda(), cache, scale=case.get("scale"), fallback=False)
    ref = orc.streamed_attention(to_np(query), oracle, "f32", scale=case.get("scale"), return_f32=True)
    np.testing.assert_allclose(to_np(out), ref, rtol=0, atol=1e-5)


def ulp_ok(out, ref, dt):
    rel = {"bf16": 2.0 ** -7, "f16": 2.0 ** -10}[dt]
    return np.all(np.abs(out - ref) <= np.abs(ref) * rel + 1e-6)


@pytest.mark.parametrize("name", sorted(CACHE_CASES))
def test_fused_attention_matches_reference_streaming_attention(name):
    case, cache, keys, values, query = build_cache(name, inject=True)
    prefix = f"cache/{name}"
    cache.get = lambda: (_ for _ in ()).throw(AssertionError("fused path materialized the full cache"))
    # fp32 query: the fp32 bar of the path is 1e-5 max-abs
    out32 = dart.fused_dart_attention(query.float().cuda(), cache, scale=case.get("scale"), fallback=False)
    assert out32.dtype == torch.float32 and tuple(out32.shape) == tuple(query.shape)
    np.testing.assert_allclose(to_np(out32), CACHES[f"{prefix}/attn_f32"], rtol=0, atol=1e-5)
    # query in the cache dtype: 2e-3 max-abs where one output ulp is below that, else one ulp
    out = dart.fused_dart_attention(query.cuda(), cache, scale=case.get("scale"), fallback=False)
    ref = CACHES[f"{prefix}/attn"]
    assert out.dtype == query.dtype
    if case["dt"] == "f32":
        np.testing.assert_allclose(to_np(out), ref, rtol=0, atol=1e-5)
    else:
        diff = np.abs(to_np(out) - ref)
        assert np.all((diff <= 2e-3) | (diff <= np.abs(ref) * {"bf16": 2.0 ** -7, "f16": 2.0 ** -10}[case["dt"]]))
        assert ulp_ok(to_np(out), ref, case["dt"])
    # streamed entry point (several query tokens) agrees with the fused one on its first token
    two = torch.cat((query, query.flip(1)), dim=2).cuda()
    streamed = dart.streamed_dart_attention(two, cache, scale=case.get("scale"))
    torch.testing.assert_close(streamed[:, :, :1], out, rtol=0, atol=0)
    # fp32-dequant flavour: what the reference's streamed attention returns for CUDA tensors (recorded on a B200)
    flav = dart.decode_attention(query[:, :, 0].float().cuda(), cache, scale=case.get("scale"), flavour=1)
    np.testing.assert_allclose(to_np(flav), CUDA_GOLD[f"cuda/{name}/streamed_f32"][:, :, 0], rtol=0, atol=1e-5)


def test_config1_report_matches_reference_figures():
    """CPU synthetic single-query decode: max-abs error vs dense attention, packed bytes, compression ratio."""

    for name, storage, ratio in (("config1_mdf32", 277504, 7.557), ("config1_mdf16", 212224, 9.882)):
        case, cache, keys, values, query = build_cache(name)
        out = dart.fused_dart_attention(query.cuda(), cache, fallback=False)
        dense = dart.dense_attention(query.cuda(), keys.cuda(), values.cuda())
        ref_err = np.abs(CACHES[f"cache/{name}/attn"] - CACHES[f"cache/{name}/dense_unquantized"]).max()
        assert abs((out - dense).abs().max().item() - ref_err) < 2e-5
        assert cache.storage_bytes == storage
        assert abs(cache.compression_ratio - ratio) < 2e-3


# ----------------------------------------------------------------------------- interface behaviour
def test_cache_preserves_sink_and_supports_incremental_updates():
    # reference tests/test_cache.py:8-26
    torch.manual_seed(2)
    keys = torch.randn(1, 2, 5, 7, dtype=torch.float32).cuda()
    values = torch.randn_like(keys)
    cache = dart.DartKVCache(dart.DartKVCacheConfig(bits=4, group_size=4, sink_tokens=2, metadata_dtype=torch.float32))
    first_keys, first_values = cache.update(keys[..., :1, :], values[..., :1, :])
    assert cache.get_seq_length() == 1
    torch.testing.assert_close(first_keys, keys[..., :1, :])
    torch.testing.assert_close(first_values, values[..., :1, :])
    restored_keys, restored_values = cache.update(keys[..., 1:, :], values[..., 1:, :])
    assert cache.get_seq_length() == 5
    assert restored_keys.shape == keys.shape and restored_values.shape == values.shape
    torch.testing.assert_close(restored_keys[..., :2, :], keys[..., :2, :])
    torch.testing.assert_close(restored_values[..., :2, :], values[..., :2, :])
    assert cache.storage_bytes < cache.dense_bytes and cache.compression_ratio > 1.0


def test_cache_rejects_incompatible_updates_and_can_clear():
    # reference tests/test_cache.py:29-49
    cache = dart.DartKVCache()
    key = torch.zeros(1, 1, 1, 4).cuda()
    cache.update(key, key)
    with pytest.raises(ValueError, match="batch/head/head_dim"):
        incompatible = torch.zeros(1, 2, 1, 4).cuda()
        cache.update(incompatible, incompatible)
    with pytest.raises(ValueError, match="dtype"):
        cache.update(key.half(), key.half())
    cache.clear()
    assert len(cache) == 0
    with pytest.raises(RuntimeError, match="empty"):
        cache.get()
    keys = torch.zeros(1, 1, 1, 4, dtype=torch.float32).cuda()
    with pytest.raises(ValueError, match="same dtype and device"):
        dart.DartKVCache().update(keys, keys.half())


def test_page_metadata_and_table():
    # reference tests/test_cache.py:76-123
    torch.manual_seed(51)
    keys = torch.randn(2, 2, 11, 12).cuda()
    values = torch.randn_like(keys)
    cache = dart.DartKVCache(dart.DartKVCacheConfig(
        page_size=4, hold_partial_pages=True, sink_tokens=2, key_group_size=4, value_group_size=6,
        promote_ratio=0.25, metadata_dtype=torch.float32))
    cache.update(keys, values)
    pages = cache.page_metadata()
    assert [(p.sequence_start, p.token_count) for p in pages] == [(0, 2), (2, 4), (6, 4), (10, 1)]
    assert pages[0].key.kind == pages[0].value.kind == "dense"
    assert pages[1].key.kind == "mixed_key" and pages[1].value.kind == "quantized"
    assert pages[1].key.fields[0][0] == "low_values"
    assert pages[1].key.fields[0][2][-1] == 1 and pages[1].value.fields[0][2][-1] == 1
    assert pages[-1].token_count == 1
    assert sum(p.token_count for p in pages) == cache.seen_tokens
    table = cache.page_table().validate()
    assert table.page_ids.shape == (2, 4)
    assert table.page_ids.tolist() == [[0, 1, 2, 3], [0, 1, 2, 3]]
    assert table.sequence_ranges().tolist() == [[0, 2], [2, 6], [6, 10], [10, 11]]
    assert table.key_modes.tolist() == [0, 2, 2, 0]
    assert table.value_modes.tolist() == [0, 1, 1, 0]
    assert table.reorder(torch.tensor([1, 1])).page_ids.tolist() == [[0, 1, 2, 3], [0, 1, 2, 3]]
    assert table.to("cpu").device.type == "cpu"


def test_page_descriptors_are_cached_and_invalidated():
    # reference tests/test_cache.py:137-176
    torch.manual_seed(55)
    keys = torch.randn(2, 1, 9, 8).cuda()
    cache = dart.DartKVCache(dart.DartKVCacheConfig(
        page_size=4, hold_partial_pages=True, key_group_size=4, value_group_size=4, metadata_dtype=torch.float32))
    assert cache.layout_version == 0
    empty_table = cache.page_table()
    assert cache.page_table() is empty_table
    cache.update(keys[..., :8, :], keys[..., :8, :])
    assert cache.layout_version == 1
    table, runs = cache.page_table(), cache.page_runs()
    assert cache.page_table() is table and cache.page_runs() is runs
    assert table.page_count == 2
    assert len(runs) == 1 and runs[0].page_count == 2
    cache.update(keys[..., 8:, :], keys[..., 8:, :])
    assert cache.layout_version == 2
    refreshed_table, refreshed_runs = cache.page_table(), cache.page_runs()
    assert refreshed_table is not table and refreshed_runs is not runs
    assert refreshed_table.page_count == 3 and refreshed_runs[0].page_count == 2
    assert cache.page_table(rebuild=True) is not refreshed_table
    reordered = cache.page_table().reorder(torch.tensor([1, 0])).validate()
    assert cache.page_runs(page_table=reordered) is not refreshed_runs
    assert cache.page_runs() is refreshed_runs
    cache.clear()
    assert cache.page_table().page_count == 0


def test_uniform_runs_are_page_major():
    # reference tests/test_cache.py:191-232
    torch.manual_seed(53)
    keys = torch.randn(1, 2, 13, 16).cuda()
    values = torch.randn_like(keys)
    cache = dart.DartKVCache(dart.DartKVCacheConfig(
        page_size=4, hold_partial_pages=True, sink_tokens=1, key_group_size=4, value_group_size=8,
        metadata_dtype=torch.float32))
    cache.update(keys, values)
    table = cache.page_table().validate()
    runs = table.uniform_quantized_runs(cache)
    assert len(runs) == 1
    run = runs[0].validate()
    assert run.first_page_index == 1 and run.page_indices.tolist() == [1, 2, 3]
    assert run.sequence_starts.tolist() == [1, 5, 9] and run.token_counts.tolist() == [4, 4, 4]
    assert run.key_values.shape[:4] == (3, 1, 2, 16) and run.value_values.shape[:4] == (3, 1, 2, 4)
    out = dart.fused_dart_attention(torch.randn(1, 4, 1, 16).cuda(), cache, page_table=table, page_runs=runs,
                                    fallback=False)
    per_page = dart.fused_dart_attention(torch.randn(1, 4, 1, 16).cuda() * 0 + 1, cache, page_table=table,
                                         page_runs=(), fallback=False)
    assert out.shape == per_page.shape == (1, 4, 1, 16)
    mixed = dart.DartKVCache(dart.DartKVCacheConfig(
        page_size=4, hold_partial_pages=True, promote_ratio=0.25, key_group_size=4, value_group_size=4,
        metadata_dtype=torch.float32))
    k = torch.randn(1, 1, 10, 8).cuda()
    mixed.update(k, k)
    t = mixed.page_table().validate()
    assert t.key_modes.tolist() == [2, 2, 0] and t.value_modes.tolist() == [1, 1, 0]
    assert t.uniform_quantized_runs(mixed) == ()


def test_local_tokens_keep_a_dense_suffix():
    # reference tests/test_cache.py:235-262
    torch.manual_seed(57)
    keys = torch.randn(1, 1, 13, 8).cuda()
    cache = dart.DartKVCache(dart.DartKVCacheConfig(
        page_size=4, local_tokens=4, key_group_size=4, value_group_size=4, metadata_dtype=torch.float32))
    cache.update(keys, keys)
    assert [(p.key.kind, p.token_count) for p in cache.page_metadata()] == [
        ("quantized", 4), ("quantized", 4), ("dense", 5)]
    assert cache.page_table().key_modes.tolist() == [1, 1, 0]
    cache.update(keys[..., :3, :], keys[..., :3, :])
    assert [(p.key.kind, p.token_count) for p in cache.page_metadata()] == [
        ("quantized", 4), ("quantized", 4), ("quantized", 4), ("dense", 4)]
    restored, _ = cache.get()
    assert restored.shape[-2] == 16


def test_pools_grow_without_changing_contents():
    torch.manual_seed(9)
    cfg = dart.DartKVCacheConfig(page_size=8, hold_partial_pages=True, sink_tokens=2, key_group_size=8,
                                 value_group_size=8, promote_ratio=0.25, metadata_dtype=torch.float16)
    keys = torch.randn(1, 2, 8 * 40 + 5, 16, dtype=torch.float16).cuda()
    small = dart.DartKVCache(cfg, max_tokens=16)    # forces several reallocations
    big = dart.DartKVCache(cfg, max_tokens=4096)
    for start in range(0, keys.shape[2], 7):
        chunk = keys[:, :, start:start + 7]
        small.append(chunk, chunk)
        big.append(chunk, chunk)
    a, b = small.get(), big.get()
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    q = torch.randn(1, 4, 1, 16, dtype=torch.float16).cuda()
    assert torch.equal(dart.fused_dart_attention(q, small), dart.fused_dart_attention(q, big))


def test_reorder_batch_moves_packed_rows_without_requantizing():
    """Beam reorder on the device pools: bytes of the selected rows are unchanged, attention follows the rows."""
    import dartkv_b200 as dart
    from dartkv_b200.synthetic import make_kvq

    keys, values, query = make_kvq(21, 3, 2, 32 + 3 * 128 + 17, 128, query_heads=8, dtype=torch.bfloat16)
    cfg = dart.DartKVCacheConfig(bits=2, promote_ratio=0.25, page_size=128, key_group_size=128, value_group_size=64,
                                 sink_tokens=32, hold_partial_pages=True, metadata_dtype=torch.bfloat16)
    cache = dart.DartKVCache(cfg)
    cache.append(keys.cuda(), values.cuda())
    before = dart.fused_dart_attention(query.cuda(), cache, fallback=False)
    k_before, v_before = cache.get()
    order = [2, 0, 2, 1]
    cache.reorder_batch(order)
    assert cache.shape[0] == 4
    k_after, v_after = cache.get()
    index = torch.tensor(order, device="cuda")
    assert torch.equal(k_after, k_before.index_select(0, index))
    assert torch.equal(v_after, v_before.index_select(0, index))
    after = dart.fused_dart_attention(query.cuda().index_select(0, index), cache, fallback=False)
    assert torch.equal(after, before.index_select(0, index))
    # appends keep working on the reordered rows
    more_k, more_v, _ = make_kvq(22, 4, 2, 130, 128, query_heads=8, dtype=torch.bfloat16)
    cache.append(more_k.cuda(), more_v.cuda())
    assert cache.seen_tokens == 32 + 3 * 128 + 17 + 130
    with pytest.raises(IndexError):
        cache.reorder_batch([0, 7])


def test_append_reads_projection_layout_without_a_copy():
    """Keys/values that live as [B, T, H, D] (projection output) are appended through a transposed view."""
    import dartkv_b200 as dart

    torch.manual_seed(5)
    b, t, h, d = 2, 32 + 2 * 128 + 40, 4, 128
    k_bthd = torch.randn(b, t, h, d, device="cuda", dtype=torch.bfloat16)
    v_bthd = torch.randn(b, t, h, d, device="cuda", dtype=torch.bfloat16)
    cfg = dart.DartKVCacheConfig(bits=2, promote_ratio=0.25, page_size=128, key_group_size=128, value_group_size=64,
                                 sink_tokens=32, hold_partial_pages=True, metadata_dtype=torch.bfloat16)
    strided, dense = dart.DartKVCache(cfg), dart.DartKVCache(cfg)
    k_view, v_view = k_bthd.transpose(1, 2), v_bthd.transpose(1, 2)
    assert not k_view.is_contiguous()
    strided.append(k_view, v_view)
    dense.append(k_view.contiguous(), v_view.contiguous())
    for (ks, vs), (kd, vd) in zip(strided.iter_segments(), dense.iter_segments()):
        for a, c in ((ks, kd), (vs, vd)):
            if isinstance(a, torch.Tensor):
                assert torch.equal(a, c)
            else:
                assert torch.equal(a.scale, c.scale) and torch.equal(a.zero_point, c.zero_point)
                fields = ("low_values", "high_values", "channel_indices") if hasattr(a, "low_values") else ("values",)
                for name in fields:
                    assert torch.equal(getattr(a, name), getattr(c, name))


def test_hf_cache_reorder_without_requantizing():
    import dartkv_b200 as dart
    from dartkv_b200.integrations import DartHFCache

    torch.manual_seed(6)
    cfg = dart.DartKVCacheConfig(bits=2, promote_ratio=0.25, page_size=128, key_group_size=128, value_group_size=64,
                                 sink_tokens=32, hold_partial_pages=True, metadata_dtype=torch.bfloat16)
    hf = DartHFCache(cfg)
    k = torch.randn(3, 2, 300, 128, device="cuda", dtype=torch.bfloat16)
    v = torch.randn_like(k)
    hf.update(k, v, 0)
    keys_before, values_before = hf._layers[0].get()
    hf.reorder_cache(torch.tensor([1, 1, 0], device="cuda"), requantize=False)
    keys_after, values_after = hf._layers[0].get()
    index = torch.tensor([1, 1, 0], device="cuda")
    assert torch.equal(keys_after, keys_before.index_select(0, index))
    assert torch.equal(values_after, values_before.index_select(0, index))


def test_failed_append_leaves_host_and_device_lifecycle_in_step():
    cfg = dart.DartKVCacheConfig(bits=2, page_size=8, hold_partial_pages=True, key_group_size=8, value_group_size=8,
                                 sink_tokens=2, promote_ratio=0.25, metadata_dtype=torch.float32)
    cache = dart.DartKVCache(cfg)
    keys, values, _ = make_kvq(21, 1, 2, 40, 16, dtype=torch.float32)
    cache.append(keys[:, :, :13].cuda(), values[:, :, :13].cuda())
    before = (cache.seen_tokens, cache._life.k_packed_end, list(cache._life.pages))
    # a forced channel list with the wrong page count is rejected after the step has been planned
    with pytest.raises(ValueError, match="channel_indices must carry"):
        cache.append(keys[:, :, 13:30].cuda(), values[:, :, 13:30].cuda(),
                     channel_indices=torch.zeros(1, 2, 5, 4, dtype=torch.int64))
    assert (cache.seen_tokens, cache._life.k_packed_end, list(cache._life.pages)) == before
    cache.append(keys[:, :, 13:].cuda(), values[:, :, 13:].cuda())
    whole = dart.DartKVCache(cfg)
    whole.append(keys[:, :, :13].cuda(), values[:, :, :13].cuda())
    whole.append(keys[:, :, 13:].cuda(), values[:, :, 13:].cuda())
    for a, b in zip(cache.get(), whole.get()):
        assert torch.equal(a, b)


def test_chunks_longer_than_the_kernel_limit_are_appended_in_pieces():
    # the reference accepts any chunk length (src/dart/cache.py:168-190); 70,000 tokens exceed the 16-bit chunk index
    cfg = dart.DartKVCacheConfig(bits=2, page_size=128, hold_partial_pages=True, key_group_size=128,
                                 value_group_size=64, sink_tokens=32, metadata_dtype=torch.bfloat16)
    gen = torch.Generator(device="cuda").manual_seed(5)
    keys = torch.randn((1, 1, 70000, 128), generator=gen, device="cuda").to(torch.bfloat16)
    values = torch.randn((1, 1, 70000, 128), generator=gen, device="cuda").to(torch.bfloat16)
    one = dart.DartKVCache(cfg)
    one.append(keys, values)
    pieces = dart.DartKVCache(cfg)
    for start in range(0, 70000, 10000):
        pieces.append(keys[:, :, start:start + 10000], values[:, :, start:start + 10000])
    assert one.seen_tokens == pieces.seen_tokens == 70000 and one._life.pages == pieces._life.pages
    for a, b in zip(one.get(), pieces.get()):
        assert torch.equal(a, b)
    assert one.storage_bytes == pieces.storage_bytes
