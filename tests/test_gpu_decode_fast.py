"""The tensor-core decode kernel (head_dim 128, 128-token pages) against the oracle on seeded inputs,
across the geometry it accepts, plus size-independent properties at the benchmark's full context."""

import numpy as np
import pytest
import torch

import dartkv_b200 as dart
from dartkv_b200.synthetic import make_kvq
from oracle import dartkv_oracle as orc
from tests.helpers import DT_TAG, to_np

pytestmark = pytest.mark.gpu


def run_case(dtype, *, batch=2, heads=2, hq=8, tokens=32 + 5 * 128 + 77, chunks=None, seed=0, outliers=True, metadata=None,
             **cfg):
    tag = DT_TAG[dtype]
    metadata = metadata or dtype
    keys, values, query = make_kvq(seed, batch, heads, tokens, 128, query_heads=hq, dtype=dtype,
                                   outlier_fraction=0.05 if outliers else 0.0)
    base = dict(bits=2, page_size=128, key_group_size=128, value_group_size=64, sink_tokens=32, hold_partial_pages=True)
    base.update(cfg)
    cache = dart.DartKVCache(dart.DartKVCacheConfig(metadata_dtype=metadata, **base))
    oracle = orc.OracleCache(orc.CacheConfig(metadata_dtype=DT_TAG[metadata], **base), tag)
    start = 0
    for chunk in chunks or [tokens]:
        cache.append(keys[:, :, start:start + chunk].cuda(), values[:, :, start:start + chunk].cuda())
        oracle.append(to_np(keys[:, :, start:start + chunk]), to_np(values[:, :, start:start + chunk]))
        start += chunk
    assert start == tokens
    out = dart.fused_dart_attention(query.cuda(), cache, fallback=False)
    assert cache.decode_status() == 0
    ref32 = orc.streamed_attention(to_np(query), oracle, tag, return_f32=True)
    ref = orc.streamed_attention(to_np(query), oracle, tag)
    got = to_np(out)
    # the kernel rounds its fp32 result once to the 16-bit output: within half an ulp of the fp32 oracle value
    ulp = np.abs(ref32) * (2.0 ** -8 if tag == "bf16" else 2.0 ** -11)
    assert np.all(np.abs(got - ref32) <= ulp + 2e-5), float(np.abs(got - ref32).max())
    diff = np.abs(got - ref)
    assert np.all((diff <= 2e-3) | (diff <= np.abs(ref) * (2.0 ** -7 if tag == "bf16" else 2.0 ** -10)))
    # same cache through the generic kernel (fp32 query), which is checked against the golden vectors elsewhere
    generic = dart.fused_dart_attention(query.float().cuda(), cache, fallback=False)
    np.testing.assert_allclose(to_np(generic), ref32, rtol=0, atol=1e-5)
    return cache, oracle, query


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_headline_geometry(dtype):
    run_case(dtype, promote_ratio=0.25, chunks=[32, 128, 128, 128, 128, 128, 77])


@pytest.mark.parametrize("dtype,metadata", [(torch.bfloat16, torch.float16), (torch.float16, torch.bfloat16)])
def test_metadata_dtype_differs_from_the_cache_dtype(dtype, metadata):
    # the reference's default: fp16 scales and zero points, also beside a bf16 model (src/dart/cache.py:57); the
    # dequantized value is rounded in the metadata dtype and then cast to the cache dtype (quantization.py:103-106)
    run_case(dtype, metadata=metadata, seed=20, promote_ratio=0.25, chunks=[32, 128, 128, 128, 128, 128, 77])
    run_case(dtype, metadata=metadata, seed=21, chunks=[300, 449])                       # uniform 2-bit keys
    run_case(dtype, metadata=metadata, seed=22, promote_ratio=0.1)                       # 12 promoted channels
    run_case(dtype, metadata=metadata, seed=23, promote_ratio=0.25, value_group_size=128, sink_tokens=0,
             tokens=4 * 128 + 3)
    run_case(dtype, metadata=metadata, seed=24, batch=1, heads=2, hq=8, tokens=32 + 3 * 128 + 40 + 30, promote_ratio=0.25,
             local_tokens=1, value_local_tokens=128, chunks=[32 + 3 * 128 + 40] + [1] * 30)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_uniform_two_bit_keys(dtype):
    run_case(dtype, seed=1, chunks=[300, 449])


@pytest.mark.parametrize("hq", [2, 4, 8])
def test_query_group_sizes(hq):
    run_case(torch.bfloat16, seed=2, heads=2, hq=hq, promote_ratio=0.25)


def test_promoted_count_not_a_multiple_of_eight():
    # 0.1 * 128 -> 12 promoted channels: the second contraction step mixes promoted and plain channels
    run_case(torch.bfloat16, seed=3, promote_ratio=0.1)
    run_case(torch.float16, seed=4, promote_ratio=0.02)   # 2 promoted channels


def test_value_group_128_and_no_sink():
    run_case(torch.bfloat16, seed=5, promote_ratio=0.25, value_group_size=128, sink_tokens=0, tokens=4 * 128 + 3)


def test_many_pages_use_both_pipeline_stages_and_several_splits():
    run_case(torch.bfloat16, seed=6, batch=1, heads=1, hq=4, tokens=32 + 41 * 128 + 5, promote_ratio=0.25)


def test_kitty_lifecycle_leaves_keys_and_values_packed_to_different_points():
    # value_local_tokens keeps the newest values dense while their keys are already packed
    run_case(torch.float16, seed=7, batch=1, heads=2, hq=8, tokens=32 + 3 * 128 + 40 + 30, promote_ratio=0.25,
             local_tokens=1, value_local_tokens=128, chunks=[32 + 3 * 128 + 40] + [1] * 30)


def test_no_packed_page_yet():
    run_case(torch.bfloat16, seed=8, tokens=100, promote_ratio=0.25)
    run_case(torch.bfloat16, seed=9, tokens=20, promote_ratio=0.25)


def test_peaked_softmax_and_large_values():
    # scaled queries make one token dominate: the hi/lo split of the probabilities must carry it
    keys, values, query = make_kvq(10, 1, 1, 32 + 2 * 128, 128, query_heads=4, dtype=torch.bfloat16)
    cfg = dict(bits=2, page_size=128, key_group_size=128, value_group_size=64, sink_tokens=32,
               hold_partial_pages=True, promote_ratio=0.25)
    cache = dart.DartKVCache(dart.DartKVCacheConfig(metadata_dtype=torch.bfloat16, **cfg))
    oracle = orc.OracleCache(orc.CacheConfig(metadata_dtype="bf16", **cfg), "bf16")
    cache.append(keys.cuda(), (values * 50).cuda())
    oracle.append(to_np(keys), to_np(values * 50))
    q = (query * 4).to(torch.bfloat16)
    out = dart.fused_dart_attention(q.cuda(), cache, scale=0.3, fallback=False)
    ref32 = orc.streamed_attention(to_np(q), oracle, "bf16", scale=0.3, return_f32=True)
    assert np.all(np.abs(to_np(out) - ref32) <= np.abs(ref32) * 2.0 ** -8 + 1e-3)


def test_full_context_properties():
    """Benchmark-size context (32768 tokens): properties that need no oracle run.

    * attention over identical value rows returns that row (softmax weights sum to one);
    * the tensor-core path and the generic path agree on the same packed cache.
    """

    batch, heads, hq, tokens = 1, 2, 8, 32768
    keys, _, query = make_kvq(11, batch, heads, tokens, 128, query_heads=hq, dtype=torch.bfloat16)
    row = torch.linspace(-2, 2, 128).to(torch.bfloat16)
    values = row.view(1, 1, 1, 128).expand(batch, heads, tokens, 128).contiguous()
    # no sink and a whole number of pages: every token's value row is packed, hence identical after dequantization
    cfg = dart.DartKVCacheConfig(bits=2, page_size=128, key_group_size=128, value_group_size=64, sink_tokens=0,
                                 hold_partial_pages=True, promote_ratio=0.25, metadata_dtype=torch.bfloat16)
    cache = dart.DartKVCache(cfg)
    cache.append(keys.cuda(), values.cuda())
    out = dart.fused_dart_attention(query.cuda(), cache, fallback=False)
    assert cache.decode_status() == 0
    _, restored = cache.get()
    expect = restored[:, :, 40].float()          # every packed value row dequantizes to the same vector
    assert torch.equal(restored[:, :, 40], restored[:, :, 20000])
    got = out[:, :, 0].float().view(batch, heads, hq // heads, 128)
    assert torch.all((got - expect.unsqueeze(2)).abs() <= expect.abs().unsqueeze(2) * 2.0 ** -7 + 1e-3)
    generic = dart.fused_dart_attention(query.float().cuda(), cache, fallback=False)
    assert torch.all((out.float() - generic).abs() <= generic.abs() * 2.0 ** -8 + 2e-5)


@pytest.mark.parametrize("split", ["aligned", "unaligned", "unaligned:7", "unaligned:5"])
def test_both_split_families_and_blocks_that_span_rows(split, decode_split):
    # 6 (batch, kv head) rows x 3 four-page units: with 7 or 5 blocks every block's share crosses a row boundary
    decode_split(split)
    run_case(torch.bfloat16, seed=9, batch=3, heads=2, hq=8, tokens=32 + 11 * 128 + 9, promote_ratio=0.25)


@pytest.mark.parametrize("tokens", [1, 5, 31, 32, 33, 100, 159, 160, 161, 32 + 128 + 15, 32 + 2 * 128])
def test_short_caches_with_few_or_no_packed_pages(tokens):
    # no page at all, sink only, sink + a partial tail tile, exactly one page, a page plus a short tail
    run_case(torch.bfloat16, seed=30 + tokens, batch=2, heads=2, hq=8, tokens=tokens, promote_ratio=0.25)


@pytest.mark.parametrize("tokens", [7, 40, 32 + 128 + 15])
def test_short_caches_token_by_token(tokens):
    run_case(torch.float16, seed=50 + tokens, batch=1, heads=2, hq=4, tokens=tokens, promote_ratio=0.25,
             chunks=[1] * tokens)


@pytest.mark.parametrize("hq,tokens", [(2, 4), (4, 3), (8, 5)])
def test_several_query_tokens_share_launches(hq, tokens):
    # reference attention.py:70-72 attends every query token to the whole cache (no mask between them): the tokens
    # of a head travel as extra heads of its KV head, up to four per launch on the tensor-core kernel
    keys, values, query = make_kvq(40 + hq, 2, 2, 32 + 3 * 128 + 20, 128, query_heads=hq, dtype=torch.bfloat16)
    gen = torch.Generator().manual_seed(tokens)
    multi = torch.randn(2, hq, tokens, 128, generator=gen).to(torch.bfloat16)
    cfg = dict(bits=2, page_size=128, key_group_size=128, value_group_size=64, sink_tokens=32, hold_partial_pages=True,
               promote_ratio=0.25)
    cache = dart.DartKVCache(dart.DartKVCacheConfig(metadata_dtype=torch.bfloat16, **cfg))
    oracle = orc.OracleCache(orc.CacheConfig(metadata_dtype="bf16", **cfg), "bf16")
    cache.append(keys.cuda(), values.cuda())
    oracle.append(to_np(keys), to_np(values))
    from dartkv_b200 import _lib as lib_mod
    before = lib_mod.LIB.dartkv_launch_count()
    out = dart.streamed_dart_attention(multi.cuda(), cache)
    launches = lib_mod.LIB.dartkv_launch_count() - before
    per_launch = max(1, 4 // (hq // 2))
    assert launches == 2 * -(-tokens // per_launch)          # decode + merge kernel per group of tokens
    ref32 = orc.streamed_attention(to_np(multi), oracle, "bf16", return_f32=True)
    assert tuple(out.shape) == (2, hq, tokens, 128)
    assert np.all(np.abs(to_np(out) - ref32) <= np.abs(ref32) * 2.0 ** -8 + 2e-5)
    # fp32 queries take the generic kernel, up to sixteen (head, token) pairs per KV head and launch
    out32 = dart.streamed_dart_attention(multi.float().cuda(), cache)
    np.testing.assert_allclose(to_np(out32), ref32, rtol=0, atol=1e-5)
    single = dart.fused_dart_attention(multi[:, :, 1:2].cuda(), cache, fallback=False)
    assert torch.equal(single, out[:, :, 1:2])


@pytest.mark.parametrize("hq", [12, 16])
def test_more_than_four_query_heads_per_kv_head_run_in_groups_of_four(hq):
    # 6 and 8 query heads per KV head: two tensor-core passes instead of the CUDA-core kernel
    from dartkv_b200 import _lib as lib_mod

    cache, oracle, query = None, None, None
    keys, values, query = make_kvq(50 + hq, 2, 2, 32 + 4 * 128 + 11, 128, query_heads=hq, dtype=torch.bfloat16)
    cfg = dict(bits=2, page_size=128, key_group_size=128, value_group_size=64, sink_tokens=32, hold_partial_pages=True,
               promote_ratio=0.25)
    cache = dart.DartKVCache(dart.DartKVCacheConfig(metadata_dtype=torch.bfloat16, **cfg))
    oracle = orc.OracleCache(orc.CacheConfig(metadata_dtype="bf16", **cfg), "bf16")
    cache.append(keys.cuda(), values.cuda())
    oracle.append(to_np(keys), to_np(values))
    before = lib_mod.LIB.dartkv_launch_count()
    out = dart.fused_dart_attention(query.cuda(), cache, fallback=False)
    assert lib_mod.LIB.dartkv_launch_count() - before == 2 * 2      # two passes of (decode + merge)
    ref32 = orc.streamed_attention(to_np(query), oracle, "bf16", return_f32=True)
    assert np.all(np.abs(to_np(out) - ref32) <= np.abs(ref32) * 2.0 ** -8 + 2e-5)
    assert cache.decode_status() == 0
