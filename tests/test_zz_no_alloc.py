"""Decode attention through the entry point that brings its own scratch memory.

Some hosts of this library may not allocate device memory where they call it (a serving loop with
a frozen memory pool, a callback inside another runtime, a latency-critical path), so they cannot
provide the split-K workspace.  ``dartkv_decode_attention_builtin_scratch`` keeps that workspace
in a fixed array inside the library.  This file is collected last on purpose: a run that stops at
the first failure has then already exercised everything else.
"""

import ctypes
import math

import numpy as np
import pytest
import torch

import dartkv_b200 as dart
from dartkv_b200 import _lib
from dartkv_b200.synthetic import make_kvq

pytestmark = pytest.mark.gpu


def _builtin(cache, query, scale):
    """Call the C entry point directly: caller-owned query/output tensors, no workspace argument."""

    q = query.contiguous()
    out = torch.empty_like(q)
    device = q.device
    with torch.cuda.device(device):
        rc = _lib.LIB.dartkv_decode_attention_builtin_scratch(
            ctypes.byref(cache.descriptor), q.data_ptr(), _lib.DTYPE_CODE[q.dtype], q.shape[1], float(scale),
            _lib.DEQUANT_PER_OP, cache.seen_tokens, out.data_ptr(), torch.cuda.current_stream(device).cuda_stream)
    return rc, out


@pytest.mark.parametrize("dtype,geometry", [
    (torch.bfloat16, dict(page_size=128, key_group_size=128, value_group_size=64, sink_tokens=32, promote_ratio=0.25)),
    (torch.float32, dict(page_size=8, key_group_size=8, value_group_size=16, sink_tokens=3, promote_ratio=0.25)),
])
def test_builtin_scratch_matches_workspace_variant_twice_in_a_row(dtype, geometry):
    head_dim = 128 if dtype == torch.bfloat16 else 32
    tokens = 32 + 6 * 128 + 50 if dtype == torch.bfloat16 else 61
    keys, values, query = make_kvq(77, 2, 2, tokens, head_dim, query_heads=8, dtype=dtype)
    md = dtype if dtype != torch.float32 else torch.float32
    cache = dart.DartKVCache(dart.DartKVCacheConfig(bits=2, hold_partial_pages=True, metadata_dtype=md, **geometry))
    cache.append(keys.cuda(), values.cuda())
    scale = 1.0 / math.sqrt(head_dim)
    q1 = query[:, :, 0].cuda()
    q2 = (query[:, :, 0] * 0.5 + 0.25).to(dtype).cuda()
    # the array is shared and keeps old contents: the second call must not see anything of the first
    for q in (q1, q2):
        expected = dart.decode_attention(q, cache, scale=scale)
        rc, got = _builtin(cache, q, scale)
        assert rc == 0, _lib.last_error()
        torch.cuda.synchronize()
        np.testing.assert_allclose(got.float().cpu().numpy(), expected.float().cpu().numpy(), rtol=0, atol=1e-5)
        assert torch.equal(got, expected)


def test_builtin_scratch_rejects_calls_that_do_not_fit():
    keys, values, query = make_kvq(78, 1, 1, 40, 32, query_heads=2, dtype=torch.float32)
    cache = dart.DartKVCache(dart.DartKVCacheConfig(bits=2, group_size=8, page_size=8, metadata_dtype=torch.float32))
    cache.append(keys.cuda(), values.cuda())
    q = query[:, :, 0].cuda().contiguous()
    out = torch.empty_like(q)
    limit = _lib.LIB.dartkv_builtin_scratch_bytes()
    assert limit == 32 << 20
    # a token count that would need far more split partials than the array holds; rejected before any launch
    desc = _lib.CacheDesc.from_buffer_copy(cache.descriptor)
    desc.batch = 4096
    rc = _lib.LIB.dartkv_decode_attention_builtin_scratch(
        ctypes.byref(desc), q.data_ptr(), _lib.F32, 64 * desc.kv_heads, 1.0, _lib.DEQUANT_PER_OP, 1 << 20,
        out.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == -3
    message = _lib.last_error()
    assert "built-in scratch" in message and str(limit) in message
