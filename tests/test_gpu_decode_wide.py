"""The general tensor-core decode kernel (every code width, group size and the fp32 flavour on 128-token pages)
against the oracle's streamed attention on seeded inputs."""

import ctypes

import numpy as np
import pytest
import torch

import dartkv_b200 as dart
from dartkv_b200 import _lib
from dartkv_b200.synthetic import make_kvq
from oracle import dartkv_oracle as orc
from tests.helpers import DT_TAG, to_np

pytestmark = pytest.mark.gpu

ORACLE_FLAVOUR = {_lib.DEQUANT_PER_OP: "cpu", _lib.DEQUANT_FP32: "fp32"}


def plan_kernel(cache, dtype, hq, flavour):
    info = _lib.DecodePlanInfo()
    rc = _lib.LIB.dartkv_decode_plan(ctypes.byref(cache.descriptor), _lib.DTYPE_CODE[dtype], hq, flavour,
                                     cache.seen_tokens, ctypes.byref(info))
    assert rc == 0
    return info.kernel


def run_case(dtype, *, batch=2, heads=2, hq=8, tokens=32 + 5 * 128 + 77, chunks=None, seed=0, flavour=_lib.DEQUANT_PER_OP,
             row_start=None, expect_kernel=3, metadata=None, **cfg):
    tag = DT_TAG[dtype]
    metadata = metadata or dtype
    keys, values, query = make_kvq(seed, batch, heads, tokens, 128, query_heads=hq, dtype=dtype, outlier_fraction=0.05)
    base = dict(bits=2, page_size=128, key_group_size=128, value_group_size=64, sink_tokens=32, hold_partial_pages=True)
    base.update(cfg)
    cache = dart.DartKVCache(dart.DartKVCacheConfig(metadata_dtype=metadata, **base))
    oracle = orc.OracleCache(orc.CacheConfig(metadata_dtype=DT_TAG[metadata], **base), tag)
    start = 0
    for chunk in chunks or [tokens]:
        cache.append(keys[:, :, start:start + chunk].cuda(), values[:, :, start:start + chunk].cuda())
        oracle.append(to_np(keys[:, :, start:start + chunk]), to_np(values[:, :, start:start + chunk]))
        start += chunk
    assert plan_kernel(cache, dtype, hq, flavour) == expect_kernel
    starts = None if row_start is None else torch.tensor(row_start, dtype=torch.int32).cuda()
    out = dart.fused_dart_attention(query.cuda(), cache, fallback=False, flavour=flavour, row_start=starts)
    assert cache.decode_status() == 0
    ref32 = orc.streamed_attention(to_np(query), oracle, tag, return_f32=True, flavour=ORACLE_FLAVOUR[flavour],
                                   row_start=None if row_start is None else np.asarray(row_start))
    got = to_np(out)
    # the kernel rounds its fp32 result once to the 16-bit output: within half an ulp of the fp32 oracle value
    ulp = np.abs(ref32) * (2.0 ** -8 if tag == "bf16" else 2.0 ** -11)
    assert np.all(np.abs(got - ref32) <= ulp + 2e-5), float(np.abs(got - ref32).max())
    return cache, oracle, query


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("bits", [4, 8])
def test_uniform_keys_and_values_of_every_width(dtype, bits):
    run_case(dtype, bits=bits, seed=bits)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("bits", [4, 8])
def test_promoted_key_channels_with_wider_values(dtype, bits):
    # promote_ratio > 0 always means 2+2-bit keys; the values follow `bits`
    run_case(dtype, bits=bits, promote_ratio=0.25, seed=10 + bits)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("value_group", [16, 32])
def test_small_value_groups(dtype, value_group):
    run_case(dtype, promote_ratio=0.25, value_group_size=value_group, seed=20 + value_group)
    run_case(dtype, value_group_size=value_group, seed=21 + value_group)       # uniform 2-bit keys


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("key_group", [32, 64])
def test_several_key_groups_per_page(dtype, key_group):
    run_case(dtype, bits=4, key_group_size=key_group, seed=30 + key_group)
    run_case(dtype, bits=2, promote_ratio=0.1, key_group_size=key_group, seed=31 + key_group)   # 12 promoted channels


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("cfg", [dict(promote_ratio=0.25), dict(), dict(bits=4), dict(bits=8, promote_ratio=0.25)])
def test_fp32_flavour_runs_on_tensor_cores(dtype, cfg):
    run_case(dtype, flavour=_lib.DEQUANT_FP32, seed=40, **cfg)


def test_large_scales_do_not_overflow_the_packed_arithmetic():
    # fp16 scales above 64: magic * scale would overflow in the fused-multiply form at bit position 0
    keys, values, query = make_kvq(50, 1, 2, 32 + 3 * 128, 128, query_heads=8, dtype=torch.float16)
    cfg = dict(bits=8, page_size=128, key_group_size=128, value_group_size=64, sink_tokens=32, hold_partial_pages=True)
    cache = dart.DartKVCache(dart.DartKVCacheConfig(metadata_dtype=torch.float16, **cfg))
    oracle = orc.OracleCache(orc.CacheConfig(metadata_dtype="f16", **cfg), "f16")
    big_v = (values * 6000).to(torch.float16)      # value range / 255 ~ 190 per code step
    cache.append(keys.cuda(), big_v.cuda())
    oracle.append(to_np(keys), to_np(big_v))
    out = dart.fused_dart_attention(query.cuda(), cache, fallback=False)
    ref32 = orc.streamed_attention(to_np(query), oracle, "f16", return_f32=True)
    assert np.isfinite(to_np(out)).all()
    assert np.all(np.abs(to_np(out) - ref32) <= np.abs(ref32) * 2.0 ** -11 + 2e-2)


def test_lifecycle_and_token_by_token_appends():
    run_case(torch.float16, bits=4, seed=60, batch=1, tokens=32 + 3 * 128 + 40 + 30, local_tokens=1,
             value_local_tokens=128, chunks=[32 + 3 * 128 + 40] + [1] * 30)
    run_case(torch.bfloat16, bits=8, promote_ratio=0.25, seed=61, batch=1, tokens=32 + 2 * 128 + 50,
             chunks=[7, 25, 128, 100, 28, 50])
    # tokens packed on one side only, with several key groups per page and small value groups
    run_case(torch.float16, bits=4, key_group_size=32, value_group_size=32, seed=62, batch=1,
             tokens=32 + 3 * 128 + 40 + 30, local_tokens=1, value_local_tokens=128, chunks=[32 + 3 * 128 + 40] + [1] * 30)
    run_case(torch.bfloat16, bits=2, promote_ratio=0.25, key_group_size=64, value_group_size=16, seed=63, batch=1,
             tokens=32 + 2 * 128 + 100 + 20, local_tokens=1, value_local_tokens=128, chunks=[32 + 2 * 128 + 100] + [1] * 20,
             flavour=_lib.DEQUANT_FP32)


@pytest.mark.parametrize("split", ["aligned", "unaligned:5"])
def test_both_split_families(split, decode_split):
    decode_split(split)
    run_case(torch.bfloat16, bits=4, seed=70, batch=3, heads=2, hq=8, tokens=32 + 11 * 128 + 9)


def test_left_padding():
    starts = [0, 33, 32 + 128 + 7, 32 + 3 * 128 + 121, 32 + 5 * 128 + 3, 32 + 5 * 128 + 76]
    run_case(torch.bfloat16, bits=4, seed=80, batch=len(starts), row_start=starts)
    run_case(torch.float16, bits=2, promote_ratio=0.25, flavour=_lib.DEQUANT_FP32, seed=81, batch=len(starts), row_start=starts)


@pytest.mark.parametrize("hq", [2, 4, 8])
def test_query_group_sizes(hq):
    run_case(torch.bfloat16, bits=4, seed=90 + hq, hq=hq)


@pytest.mark.parametrize("dtype,metadata", [(torch.bfloat16, torch.float16), (torch.float16, torch.bfloat16)])
@pytest.mark.parametrize("cfg", [dict(promote_ratio=0.25), dict(bits=4), dict(bits=8, promote_ratio=0.25), dict(bits=8)])
def test_metadata_dtype_differs_from_the_cache_dtype(dtype, metadata, cfg):
    # the reference's scripts keep fp16 metadata beside bf16 models (its default metadata dtype): the dequantized
    # value is rounded in the metadata dtype and then cast to the cache dtype
    # 2-bit pages keep their own per-op kernel (it casts its operands); their fp32 flavour comes here
    two_bit = cfg.get("bits", 2) == 2
    run_case(dtype, metadata=metadata, seed=100, chunks=[32 + 2 * 128 + 40, 3 * 128 + 37], expect_kernel=1 if two_bit else 3,
             **cfg)
    run_case(dtype, metadata=metadata, seed=101, flavour=_lib.DEQUANT_FP32, **cfg)


def test_corners_of_the_supported_geometry():
    # smallest groups with the widest codes (largest staged chunks: one block per SM), every channel promoted,
    # one value group per token, a single query head per KV head
    run_case(torch.bfloat16, bits=8, key_group_size=16, value_group_size=16, seed=110)
    run_case(torch.float16, bits=4, key_group_size=16, value_group_size=128, seed=111)
    run_case(torch.bfloat16, bits=4, promote_ratio=1.0, seed=112)
    run_case(torch.float16, bits=8, promote_ratio=0.5, key_group_size=32, seed=113)
    run_case(torch.bfloat16, bits=4, heads=4, hq=4, seed=114)


def test_headline_geometry_keeps_its_own_kernels():
    run_case(torch.bfloat16, promote_ratio=0.25, seed=99, expect_kernel=1)
