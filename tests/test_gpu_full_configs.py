"""Parity at the sizes the benchmark numbers are quoted on: the full decode workloads (batch 32 x context 8192
and batch 128 x context 32768, built with the benchmark's own generator) and the full append workload
(bf16 [16,8,4096,128], 32 sink tokens, then 128 tokens per append) are compared with the oracle on a subset of
batch rows -- the oracle needs seconds per row at these sizes."""

import numpy as np
import pytest
import torch

import dartkv_b200 as dart
from dartkv_b200.synthetic import HEADLINE_GEOMETRY, build_headline_cache, headline_cache_kwargs, make_kvq
from oracle import dartkv_oracle as orc
from tests.helpers import to_np
from tests.test_gpu_cache import cache_owned_segments, key_fields

pytestmark = pytest.mark.gpu


def oracle_rows(keys, values, metadata="bf16"):
    cache = orc.OracleCache(orc.CacheConfig(metadata_dtype=metadata, **headline_cache_kwargs()), "bf16")
    sinks = HEADLINE_GEOMETRY["sinks"]
    k, v = to_np(keys), to_np(values)
    cache.append(k[:, :, :sinks], v[:, :, :sinks])
    cache.append(k[:, :, sinks:], v[:, :, sinks:])
    return cache


def check_against_oracle(out, ref32, ref16):
    """bf16 output of the kernel vs the oracle: within half an output ulp of the oracle's fp32 value, and within
    2e-3 (or one output ulp where an ulp is larger than that) of the oracle's bf16 output."""

    got = to_np(out)
    assert np.all(np.abs(got - ref32) <= np.abs(ref32) * 2.0 ** -8 + 2e-5), float(np.abs(got - ref32).max())
    diff = np.abs(got - ref16)
    assert np.all((diff <= 2e-3) | (diff <= np.abs(ref16) * 2.0 ** -7)), float(diff.max())


def decode_workload(batch, ctx, seed, rows, decode_split):
    device = torch.device("cuda", 0)
    cache, query, keys, values = build_headline_cache(range(batch), ctx, seed, device, keep_rows=rows)
    oracle = oracle_rows(keys, values)
    del keys, values
    q_rows = to_np(query[rows])
    ref32 = orc.streamed_attention(q_rows, oracle, "bf16", return_f32=True)
    ref16 = orc.streamed_attention(q_rows, oracle, "bf16")
    ref_fused = orc.streamed_attention(q_rows, oracle, "bf16", flavour="fused", return_f32=True)
    q3 = query[:, :, 0].contiguous()
    for split in (None, "aligned", "unaligned"):
        decode_split(split)
        out = dart.decode_attention(q3, cache)
        assert cache.decode_status() == 0
        check_against_oracle(out[rows].unsqueeze(2), ref32, ref16)
        fused = dart.decode_attention(q3, cache, flavour=dart.DEQUANT_FUSED)
        err = np.abs(to_np(fused[rows].unsqueeze(2)) - ref_fused).max()
        assert err <= 1e-2 * np.abs(ref_fused).max(), float(err)
    # the packed pages of the checked rows are the oracle's, byte for byte (first, middle and last page)
    ks, vs = cache_owned_segments(cache)
    assert len(ks) == len(oracle.key_segments) and len(vs) == len(oracle.value_segments)
    for i in sorted({1, len(ks) // 2, len(ks) - 1}):
        ref = oracle.key_segments[i]
        ref_fields = [ref.low_values, ref.high_values, ref.channel_indices, ref.scale, ref.zero_point]
        for a, b in zip(key_fields(ks[i]), ref_fields):
            np.testing.assert_array_equal(a[rows], b, err_msg=f"key page {i}")
    for i in sorted({1, len(vs) // 2, len(vs) - 1}):
        ref = oracle.value_segments[i]
        for a, b in zip(key_fields(vs[i]), [ref.values, ref.scale, ref.zero_point]):
            np.testing.assert_array_equal(a[rows], b, err_msg=f"value page {i}")


def test_config3_batch32_context8192_rows_match_oracle(decode_split):
    decode_workload(32, 8192, 2, [0, 31], decode_split)


def test_config5_batch128_context32768_row_matches_oracle(decode_split):
    decode_workload(128, 32768, 4, [77], decode_split)


@pytest.mark.parametrize("bits,ratio", [(2, 0.25), (4, 0.25), (8, 0.25), (2, 0.0), (4, 0.0), (8, 0.0)])
def test_config2_append_bytes_match_oracle(bits, ratio):
    """bf16 [16,8,4096,128] with outlier key channels: 32 sink tokens, 31 pages from 128-token appends and 96 pending
    tokens; every packed byte, scale and zero point of two of the sixteen rows equals the oracle's."""

    keys, values, _ = make_kvq(1, 16, 8, 4096, 128, dtype=torch.bfloat16)
    kwargs = dict(headline_cache_kwargs(), bits=bits, promote_ratio=ratio)
    cache = dart.DartKVCache(dart.DartKVCacheConfig(metadata_dtype=torch.bfloat16, **kwargs), max_tokens=4096 + 256)
    rows = [3, 12]
    oracle = orc.OracleCache(orc.CacheConfig(metadata_dtype="bf16", **kwargs), "bf16")
    k_dev, v_dev = keys.cuda(), values.cuda()
    k_np, v_np = to_np(keys[rows]), to_np(values[rows])
    pos = 0
    for chunk in [32] + [128] * 31 + [96]:
        cache.append(k_dev[:, :, pos:pos + chunk], v_dev[:, :, pos:pos + chunk])
        oracle.append(k_np[:, :, pos:pos + chunk], v_np[:, :, pos:pos + chunk])
        pos += chunk
    assert pos == 4096
    cache.check_finite()
    assert cache.seen_tokens - cache._life.k_packed_end == 96
    ks, vs = cache_owned_segments(cache)
    assert len(ks) == len(oracle.key_segments) == 32 and len(vs) == len(oracle.value_segments) == 32
    for i, (mine, ref) in enumerate(zip(ks, oracle.key_segments)):
        if isinstance(ref, np.ndarray):
            ref_fields = [ref]
        elif isinstance(ref, orc.MixedKey):
            ref_fields = [ref.low_values, ref.high_values, ref.channel_indices, ref.scale, ref.zero_point]
        else:
            ref_fields = [ref.values, ref.scale, ref.zero_point]
        for a, b in zip(key_fields(mine), ref_fields):
            np.testing.assert_array_equal(a[rows], b, err_msg=f"key segment {i}")
    for i, (mine, ref) in enumerate(zip(vs, oracle.value_segments)):
        ref_fields = [ref] if isinstance(ref, np.ndarray) else [ref.values, ref.scale, ref.zero_point]
        for a, b in zip(key_fields(mine), ref_fields):
            np.testing.assert_array_equal(a[rows], b, err_msg=f"value segment {i}")
    # the dense pending tail is returned unchanged
    got_k, got_v = cache.get()
    assert torch.equal(got_k[:, :, -96:].cpu(), keys[:, :, -96:]) and torch.equal(got_v[:, :, -96:].cpu(), values[:, :, -96:])
