"""Left-padded batches: ``row_start`` masks the tokens before every row's first live one on all decode kernels.

The reference's fused call has no mask (its adapter serves uniform-length batches); the expected values come from
the oracle's streamed attention with the same tokens set to -inf, which is what a dense masked softmax computes.
"""

import numpy as np
import pytest
import torch

import dartkv_b200 as dart
from dartkv_b200 import _lib
from dartkv_b200.synthetic import make_kvq
from oracle import dartkv_oracle as orc
from tests.helpers import DT_TAG, to_np

pytestmark = pytest.mark.gpu

BASE = dict(bits=2, page_size=128, key_group_size=128, value_group_size=64, sink_tokens=32, hold_partial_pages=True,
            promote_ratio=0.25)
TOKENS = 32 + 6 * 128 + 45


def build(dtype, starts, *, tokens=TOKENS, seed=0, heads=2, hq=8, **cfg):
    tag = DT_TAG[dtype]
    batch = len(starts)
    keys, values, query = make_kvq(seed, batch, heads, tokens, 128, query_heads=hq, dtype=dtype)
    base = dict(BASE)
    base.update(cfg)
    cache = dart.DartKVCache(dart.DartKVCacheConfig(metadata_dtype=dtype, **base))
    oracle = orc.OracleCache(orc.CacheConfig(metadata_dtype=tag, **base), tag)
    cache.append(keys.cuda(), values.cuda())
    oracle.append(to_np(keys), to_np(values))
    return cache, oracle, query, tag


def check(cache, oracle, query, tag, starts, flavour=_lib.DEQUANT_PER_OP, oracle_flavour="cpu", bound=2e-5):
    row_start = torch.tensor(starts, dtype=torch.int32)
    out = dart.fused_dart_attention(query.cuda(), cache, fallback=False, flavour=flavour, row_start=row_start.cuda())
    assert cache.decode_status() == 0
    ref32 = orc.streamed_attention(to_np(query), oracle, tag, return_f32=True, row_start=np.asarray(starts),
                                   flavour=oracle_flavour)
    got = to_np(out)
    assert np.isfinite(got).all()
    ulp = np.abs(ref32) * (2.0 ** -8 if tag == "bf16" else 2.0 ** -11)
    assert np.all(np.abs(got - ref32) <= ulp + bound), float(np.abs(got - ref32).max())
    return out


# first live token: none masked, inside the sink, on a page edge, at every residue of a page's 16-token groups,
# inside the last page, inside the dense tail
STARTS = [0, 1, 31, 32, 33, 32 + 7, 32 + 8, 32 + 15, 32 + 16, 32 + 64, 32 + 127, 32 + 128, 32 + 128 + 77,
          32 + 3 * 128 + 4, 32 + 5 * 128 + 100, 32 + 6 * 128, 32 + 6 * 128 + 20, TOKENS - 1]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_per_op_kernel_masks_the_padding(dtype):
    cache, oracle, query, tag = build(dtype, STARTS, seed=1)
    check(cache, oracle, query, tag, STARTS)


def test_rows_with_different_padding_do_not_disturb_each_other():
    starts = [0, 500, 0, 97]
    cache, oracle, query, tag = build(torch.bfloat16, starts, seed=2)
    out = check(cache, oracle, query, tag, starts)
    plain = dart.fused_dart_attention(query.cuda(), cache, fallback=False)
    assert torch.equal(out[0], plain[0]) and torch.equal(out[2], plain[2])
    assert not torch.equal(out[1], plain[1])


def test_fused_flavour_kernel_masks_the_padding():
    cache, oracle, query, tag = build(torch.float16, STARTS, seed=3)
    check(cache, oracle, query, tag, STARTS, flavour=_lib.DEQUANT_FUSED, oracle_flavour="fused", bound=2e-3)


def test_generic_kernel_masks_the_padding():
    # fp32 queries take the CUDA-core kernel
    cache, oracle, query, tag = build(torch.bfloat16, STARTS, seed=4)
    row_start = torch.tensor(STARTS, dtype=torch.int32).cuda()
    out = dart.fused_dart_attention(query.float().cuda(), cache, fallback=False, row_start=row_start)
    ref32 = orc.streamed_attention(to_np(query), oracle, tag, return_f32=True, row_start=np.asarray(STARTS))
    np.testing.assert_allclose(to_np(out), ref32, rtol=0, atol=1e-5)


@pytest.mark.parametrize("split", ["aligned", "unaligned:5"])
def test_padding_with_both_split_families(split, decode_split):
    decode_split(split)
    starts = [32 + 9 * 128 + 3, 0, 32 + 2 * 128 + 127, 700]
    cache, oracle, query, tag = build(torch.bfloat16, starts, tokens=32 + 11 * 128 + 9, seed=5)
    check(cache, oracle, query, tag, starts)


def test_a_masked_prefix_equals_a_shorter_cache_when_pages_line_up():
    # masking whole pages must give exactly what a cache without those tokens' weights gives: compare with the
    # oracle only (the packed statistics of later pages do not depend on earlier tokens)
    starts = [32 + 4 * 128] * 2
    cache, oracle, query, tag = build(torch.float16, starts, seed=6, sink_tokens=32)
    check(cache, oracle, query, tag, starts)


def test_row_start_is_validated():
    cache, oracle, query, tag = build(torch.bfloat16, [0, 0], seed=7)
    with pytest.raises(ValueError):
        dart.fused_dart_attention(query.cuda(), cache, row_start=torch.zeros(3, dtype=torch.int32).cuda())
