"""Pin the NumPy oracle to vectors produced by the reference implementation itself."""

import hashlib

import numpy as np
import pytest

from oracle import dartkv_oracle as orc
from tests.golden.cases import CACHE_CASES, build_inputs
from tests.helpers import load_golden, to_np


def sha(*arrays):
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


PRIM = load_golden("primitives.npz")
CACHES = load_golden("caches.npz")

QUANT_KEYS = sorted({k.rsplit("/", 1)[0] for k in PRIM if k.startswith("quant/")})
MIXED_NAMES = sorted({k.split("/")[1] for k in PRIM if k.startswith("mixed/")})


@pytest.mark.parametrize("key", QUANT_KEYS)
def test_quantize_matches_reference_bytes(key):
    _, dt, bits, _ = key.split("/")
    axis, group, padded, packed = (int(v) for v in PRIM[f"{key}/meta"])
    md = str(PRIM[f"{key}/md"])
    q = orc.quantize(PRIM[f"{key}/input"], dt, bits=int(bits[1:]), group_size=group, md=md, axis=axis)
    assert (q.padded_dim, q.packed_dim) == (padded, packed)
    np.testing.assert_array_equal(q.values, PRIM[f"{key}/values"])
    np.testing.assert_array_equal(q.scale, PRIM[f"{key}/scale"])
    np.testing.assert_array_equal(q.zero_point, PRIM[f"{key}/zero"])
    np.testing.assert_array_equal(orc.dequantize(q), PRIM[f"{key}/dequant"])


@pytest.mark.parametrize("name", MIXED_NAMES)
@pytest.mark.parametrize("strategy", ["magnitude", "variance"])
def test_mixed_key_matches_reference_bytes(name, strategy):
    keys = PRIM[f"mixed/{name}/input"]
    dt = str(PRIM[f"mixed/{name}/dt"])
    group = int(PRIM[f"mixed/{name}/group"])
    key = f"mixed/{name}/{strategy}"
    md = str(PRIM[f"{key}/md"])
    ref_idx = PRIM[f"{key}/indices"]
    m = orc.quantize_key_mixed(keys, dt, group_size=group, ratio=0.25, md=md, strategy=strategy, indices=ref_idx)
    np.testing.assert_array_equal(m.low_values, PRIM[f"{key}/low"])
    np.testing.assert_array_equal(m.high_values, PRIM[f"{key}/high"])
    np.testing.assert_array_equal(m.scale, PRIM[f"{key}/scale"])
    np.testing.assert_array_equal(m.zero_point, PRIM[f"{key}/zero"])
    np.testing.assert_array_equal(orc.dequantize_mixed(m), PRIM[f"{key}/dequant"])


@pytest.mark.parametrize("name", MIXED_NAMES)
@pytest.mark.parametrize("strategy", ["magnitude", "variance"])
def test_channel_selection_matches_reference_up_to_ties(name, strategy):
    keys = PRIM[f"mixed/{name}/input"]
    dt = str(PRIM[f"mixed/{name}/dt"])
    ref_score = PRIM[f"mixed/{name}/score_{strategy}"]
    score = orc.channel_scores(keys, dt, strategy)
    if dt == "f32":
        np.testing.assert_allclose(score, ref_score, rtol=2e-6, atol=1e-7)
    else:
        # reduced-precision scores are bit-equal except where the fp32 sum sits on a rounding boundary
        mismatch = np.count_nonzero(score != ref_score)
        assert mismatch <= max(1, score.size // 200), mismatch
        np.testing.assert_allclose(score, ref_score, rtol=1e-2)
    ref_idx = PRIM[f"mixed/{name}/{strategy}/indices"].astype(np.int64)
    _, idx = orc.select_key_channels(keys, dt, 0.25, strategy=strategy)
    count = idx.shape[-1]
    for b in range(idx.shape[0]):
        for h in range(idx.shape[1]):
            s = ref_score[b, h]
            order = np.sort(s)[::-1]
            tie_at_cut = order[count - 1] == order[count]
            if not tie_at_cut and np.array_equal(score[b, h], s):
                assert set(idx[b, h].tolist()) == set(ref_idx[b, h].tolist())
            # whatever the tie-break, both selections take exactly the `count` largest scores
            assert np.array_equal(np.sort(s[ref_idx[b, h]])[::-1], order[:count])


def _run_case(name):
    case = CACHE_CASES[name]
    prefix = f"cache/{name}"
    keys, values, query = (to_np(t) for t in build_inputs(case))
    if case.get("store_inputs", True):
        np.testing.assert_array_equal(keys, CACHES[f"{prefix}/keys"])
        np.testing.assert_array_equal(query, CACHES[f"{prefix}/query"])
    cfg = dict(case["config"])
    cfg["metadata_dtype"] = cfg.pop("md")
    ref_idx = CACHES.get(f"{prefix}/mixed_indices")
    provider = (lambda i: ref_idx[i]) if ref_idx is not None else None
    cache = orc.OracleCache(orc.CacheConfig(**cfg), case["dt"], channel_indices_provider=provider)
    start = 0
    for chunk in case["chunks"]:
        cache.append(keys[..., start:start + chunk, :], values[..., start:start + chunk, :])
        start += chunk
    return case, prefix, cache, query


@pytest.mark.parametrize("name", sorted(CACHE_CASES))
def test_cache_lifecycle_matches_reference(name):
    case, prefix, cache, query = _run_case(name)
    assert cache.storage_bytes == int(CACHES[f"{prefix}/storage_bytes"])
    assert cache.dense_bytes == int(CACHES[f"{prefix}/dense_bytes"])
    table = np.array(cache.segment_table(), dtype=np.int64).reshape(-1, 4)
    np.testing.assert_array_equal(table, CACHES[f"{prefix}/table"])
    key_rows = CACHES[f"{prefix}/key_segments"]
    assert len(cache.key_segments) == len(key_rows)
    for i, seg in enumerate(cache.key_segments):
        assert (orc._mode(seg), orc.segment_tokens(seg)) == tuple(int(v) for v in key_rows[i])
        if isinstance(seg, np.ndarray):
            fields = [seg]
        elif isinstance(seg, orc.MixedKey):
            fields = [seg.low_values, seg.high_values, seg.channel_indices, seg.scale, seg.zero_point]
        else:
            fields = [seg.values, seg.scale, seg.zero_point]
        assert sha(*fields) == str(CACHES[f"{prefix}/k{i}/sha"]), f"key segment {i}"
    value_rows = CACHES[f"{prefix}/value_segments"]
    assert len(cache.value_segments) == len(value_rows)
    for i, seg in enumerate(cache.value_segments):
        assert (orc._mode(seg), orc.segment_tokens(seg)) == tuple(int(v) for v in value_rows[i])
        fields = [seg] if isinstance(seg, np.ndarray) else [seg.values, seg.scale, seg.zero_point]
        assert sha(*fields) == str(CACHES[f"{prefix}/v{i}/sha"]), f"value segment {i}"
    pend = CACHES[f"{prefix}/pending"]
    assert (0 if cache.pending_key is None else cache.pending_key.shape[-2]) == int(pend[0])
    assert (0 if cache.pending_value is None else cache.pending_value.shape[-2]) == int(pend[1])
    got_k, got_v = cache.get()
    assert sha(got_k, got_v) == str(CACHES[f"{prefix}/get_sha"])


@pytest.mark.parametrize("name", sorted(CACHE_CASES))
def test_streamed_attention_matches_reference(name):
    case, prefix, cache, query = _run_case(name)
    out32 = orc.streamed_attention(query, cache, case["dt"], scale=case.get("scale"), return_f32=True)
    # fp32 accumulation order differs between BLAS builds: 1e-5 absolute is the fp32 bar of the path
    np.testing.assert_allclose(out32, CACHES[f"{prefix}/attn_f32"], rtol=0, atol=1e-5)
    out = orc.streamed_attention(query, cache, case["dt"], scale=case.get("scale"))
    ref = CACHES[f"{prefix}/attn"]
    if case["dt"] == "f32":
        np.testing.assert_allclose(out, ref, rtol=0, atol=1e-5)
    else:
        ulp = np.abs(ref) * (2.0 ** -7 if case["dt"] == "bf16" else 2.0 ** -10) + 1e-6
        assert np.all(np.abs(out - ref) <= ulp)


def test_config1_report_values():
    """The figures the reference prints for the CPU synthetic single-query decode."""

    for name, ratio in (("config1_mdf32", 7.557), ("config1_mdf16", 9.882)):
        case, prefix, cache, query = _run_case(name)
        keys, values, _ = (to_np(t) for t in build_inputs(case))
        out = orc.streamed_attention(query, cache, "f32")
        dense = orc.dense_attention(query, keys, values, "f32")
        np.testing.assert_allclose(dense, CACHES[f"{prefix}/dense_unquantized"], atol=1e-5, rtol=0)
        assert abs(np.abs(out - dense).max() - np.abs(CACHES[f"{prefix}/attn"] - dense).max()) < 1e-5
        assert abs(cache.dense_bytes / cache.storage_bytes - ratio) < 2e-3
