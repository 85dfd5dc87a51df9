"""Decode attention with the arithmetic of the reference's Triton kernels (``DEQUANT_FUSED``:
``code * scale + zero`` kept in fp32, src/dart/fused_attention.py:149-262) against the oracle's
restatement of that arithmetic, and against the pinned per-op oracle at the tolerance the reference's
own test of its Triton kernel uses (tests/test_fused_attention.py:53, rtol 3e-2 / atol 3e-3).

The Triton kernels cannot run where the golden vectors were made (no GPU), so this flavour has no
golden vectors: parity unpinned, checked against the restatement only.
"""

import numpy as np
import pytest
import torch

import dartkv_b200 as dart
from dartkv_b200.synthetic import make_kvq
from oracle import dartkv_oracle as orc
from tests.helpers import DT_TAG, to_np

pytestmark = pytest.mark.gpu


def run_case(dtype, *, batch=2, heads=2, hq=8, tokens=32 + 5 * 128 + 77, chunks=None, seed=0, outliers=True,
             data_scale=1.0, generic_bound=1e-4, metadata=None, **cfg):
    tag = DT_TAG[dtype]
    metadata = metadata or dtype
    keys, values, query = make_kvq(seed, batch, heads, tokens, 128, query_heads=hq, dtype=dtype,
                                   outlier_fraction=0.05 if outliers else 0.0)
    if data_scale != 1.0:
        keys = (keys.float() * data_scale).to(dtype)
        values = (values.float() * data_scale).to(dtype)
    base = dict(bits=2, page_size=128, key_group_size=128, value_group_size=64, sink_tokens=32, hold_partial_pages=True)
    base.update(cfg)
    cache = dart.DartKVCache(dart.DartKVCacheConfig(metadata_dtype=metadata, **base))
    oracle = orc.OracleCache(orc.CacheConfig(metadata_dtype=DT_TAG[metadata], **base), tag)
    start = 0
    for chunk in chunks or [tokens]:
        cache.append(keys[:, :, start:start + chunk].cuda(), values[:, :, start:start + chunk].cuda())
        oracle.append(to_np(keys[:, :, start:start + chunk]), to_np(values[:, :, start:start + chunk]))
        start += chunk
    # scaled keys get a compensating softmax scale: the logits (and the conditioning of the softmax) stay put
    factor = 1.0 / (np.sqrt(128.0) * data_scale)
    out = dart.fused_dart_attention(query.cuda(), cache, fallback=False, flavour=dart.DEQUANT_FUSED, scale=factor)
    assert cache.decode_status() == 0
    got = to_np(out).astype(np.float64)
    ref = orc.streamed_attention(to_np(query), oracle, tag, factor, flavour="fused", return_f32=True).astype(np.float64)
    mag = np.abs(ref).max()
    # tensor-core kernel: the result is rounded once to the 16-bit output (2^-9 / 2^-12 relative) and the value
    # weights p * scale enter the MMA as fp16 (2^-12 relative to the |scale * code| terms, which exceed the
    # result where zero-points cancel them); measured maxima are 5.0e-3 (bf16) and 2.6e-3 (fp16) of `mag`
    bound = (7e-3 if tag == "bf16" else 4e-3) * mag
    assert np.abs(got - ref).max() <= bound, (float(np.abs(got - ref).max()), float(mag))
    # generic kernel (fp32 query, fp32 output): fp32 arithmetic end to end
    generic = to_np(dart.fused_dart_attention(query.float().cuda(), cache, fallback=False, flavour=dart.DEQUANT_FUSED,
                                              scale=factor))
    assert np.abs(generic - ref).max() <= generic_bound * mag + 1e-6
    return got, oracle, query, tag


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_headline_geometry(dtype):
    run_case(dtype, promote_ratio=0.25, chunks=[32, 128, 128, 128, 128, 128, 77])


@pytest.mark.parametrize("dtype,metadata", [(torch.bfloat16, torch.float16), (torch.float16, torch.bfloat16)])
def test_metadata_dtype_differs_from_the_cache_dtype(dtype, metadata):
    # fp16 scales and zero points beside a bf16 cache is the reference's default (src/dart/cache.py:57)
    import ctypes

    from dartkv_b200 import _lib

    run_case(dtype, metadata=metadata, seed=30, promote_ratio=0.25, chunks=[32, 128, 128, 128, 128, 128, 77])
    got, oracle, query, tag = run_case(dtype, metadata=metadata, seed=31, chunks=[300, 449])
    cache = dart.DartKVCache(dart.DartKVCacheConfig(metadata_dtype=metadata, bits=2, page_size=128, key_group_size=128,
                                                    value_group_size=64, sink_tokens=32, hold_partial_pages=True))
    keys, values, _ = make_kvq(31, 2, 2, 300, 128, query_heads=8, dtype=dtype)
    cache.append(keys.cuda(), values.cuda())
    info = _lib.DecodePlanInfo()
    assert _lib.LIB.dartkv_decode_plan(ctypes.byref(cache.descriptor), _lib.DTYPE_CODE[dtype], 8, _lib.DEQUANT_FUSED, 300,
                                       ctypes.byref(info)) == 0
    assert info.kernel == 2      # the tensor-core kernel of this flavour, not the CUDA-core one


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_matches_the_per_op_oracle_at_the_reference_tolerance_for_its_triton_kernel(dtype):
    got, oracle, query, tag = run_case(dtype, promote_ratio=0.25, outliers=False, seed=11)
    per_op = orc.streamed_attention(to_np(query), oracle, tag, return_f32=True)
    np.testing.assert_allclose(got, per_op, rtol=3e-2, atol=3e-3)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_uniform_two_bit_keys(dtype):
    run_case(dtype, seed=1, chunks=[300, 449])


@pytest.mark.parametrize("hq", [2, 4, 8])
def test_query_group_sizes(hq):
    run_case(torch.bfloat16, seed=2, heads=2, hq=hq, promote_ratio=0.25)


def test_promoted_count_not_a_multiple_of_eight():
    run_case(torch.bfloat16, seed=3, promote_ratio=0.1)    # 12 promoted channels: the last high-plane step is half empty
    run_case(torch.float16, seed=4, promote_ratio=0.02)    # 2 promoted channels


def test_value_group_128_and_no_sink():
    run_case(torch.bfloat16, seed=5, promote_ratio=0.25, value_group_size=128, sink_tokens=0, tokens=4 * 128 + 3)


def test_many_pages_use_both_pipeline_stages_and_several_splits():
    run_case(torch.bfloat16, seed=6, batch=1, heads=1, hq=4, tokens=32 + 41 * 128 + 5, promote_ratio=0.25)


@pytest.mark.parametrize("data_scale", [1e-3, 1e2, 1e6])
def test_power_of_two_normalisation_keeps_fp16_weights_in_range(data_scale):
    # key / value scales far below and far above 1: the weights q*s and p*s would leave the fp16 range unnormalised
    run_case(torch.bfloat16, seed=8, promote_ratio=0.25, data_scale=data_scale)


def test_kitty_lifecycle_leaves_keys_and_values_packed_to_different_points():
    # where key and value segments end at different tokens the reference cuts them by dequantizing the packed side
    # with per-op rounding (cache.py iter_segments), and the oracle follows; the kernels apply the unrounded
    # arithmetic to every packed token, hence the wider bound for the fp32 comparison
    run_case(torch.float16, seed=7, batch=1, heads=2, hq=8, tokens=32 + 3 * 128 + 40 + 30, promote_ratio=0.25,
             local_tokens=1, value_local_tokens=128, chunks=[32 + 3 * 128 + 40] + [1] * 30, generic_bound=1e-3)


def test_unknown_flavour_is_rejected():
    keys, values, query = make_kvq(0, 1, 1, 200, 128, query_heads=4, dtype=torch.bfloat16)
    cache = dart.DartKVCache(dart.DartKVCacheConfig(bits=2, page_size=128, hold_partial_pages=True, metadata_dtype=torch.bfloat16))
    cache.append(keys.cuda(), values.cuda())
    with pytest.raises(ValueError, match="unknown dequant flavour"):
        dart.fused_dart_attention(query.cuda(), cache, fallback=False, flavour=7)


@pytest.mark.parametrize("split", ["aligned", "unaligned:7"])
def test_both_split_families(split, decode_split):
    decode_split(split)
    run_case(torch.bfloat16, seed=9, batch=3, heads=2, hq=8, tokens=32 + 11 * 128 + 9, promote_ratio=0.25)


@pytest.mark.parametrize("tokens", [1, 31, 33, 160, 161, 32 + 2 * 128])
def test_short_caches_with_few_or_no_packed_pages(tokens):
    run_case(torch.bfloat16, seed=30 + tokens, batch=2, heads=2, hq=8, tokens=tokens, promote_ratio=0.25)
