"""The two dequantization flavours that only exist in the reference's CUDA code paths, against outputs of those
paths recorded on a B200 (``tests/golden/make_golden_cuda.py`` ran the unmodified reference there):

* ``DEQUANT_FP32``  -- its Triton dequantize kernels (``src/dart/triton_ops.py:310-324``: one fp32 multiply-add
  rounded once) and ``streamed_dart_attention`` on CUDA tensors, which calls them (``src/dart/attention.py:74-75``);
* ``DEQUANT_FUSED`` -- its Triton attention kernels (``fused_dart_attention`` with the fallback off,
  ``src/dart/fused_attention.py:654-771``), which never round the dequantized value.

Every cache is rebuilt from the case's seed with the promoted channels the reference chose, so the packed bytes are
the ones the reference read."""

import copy
import hashlib

import numpy as np
import pytest
import torch

import dartkv_b200 as dart
from dartkv_b200.lifecycle import plan_append
from tests.golden.cases import CACHE_CASES, CUDA_EXTRA_CASES, TORCH_DTYPES, build_inputs
from tests.helpers import load_golden, to_np
from tests.test_gpu_cache import cache_owned_segments

pytestmark = pytest.mark.gpu

GOLD = load_golden("cuda_reference.npz")
CASES = dict(CACHE_CASES)
CASES.update(CUDA_EXTRA_CASES)
HALF_ULP = {"bf16": 2.0 ** -8, "f16": 2.0 ** -11}


def sha(array):
    return hashlib.sha256(np.ascontiguousarray(array).tobytes()).hexdigest()


def build(name):
    case = CASES[name]
    keys, values, query = build_inputs(case)
    kwargs = dict(case["config"])
    kwargs["metadata_dtype"] = TORCH_DTYPES[kwargs.pop("md")]
    cfg = dart.DartKVCacheConfig(**kwargs)
    cache = dart.DartKVCache(cfg)
    recorded = GOLD.get(f"cuda/{name}/mixed_indices")   # [B,H,pages,K] in the order the reference quantized them
    used = start = 0
    for chunk in case["chunks"]:
        forced = None
        if recorded is not None:
            plan = plan_append(cfg, copy.deepcopy(cache._life), chunk)
            count = plan.num_pages + plan.requantize_last_page
            if count:
                forced = torch.from_numpy(np.ascontiguousarray(recorded[:, :, used:used + count]))
                used += count
        cache.append(keys[..., start:start + chunk, :].cuda(), values[..., start:start + chunk, :].cuda(),
                     channel_indices=forced)
        start += chunk
    if recorded is not None:
        assert used == recorded.shape[2]
    return case, cache, query


@pytest.mark.parametrize("name", sorted(CASES))
def test_page_dequantization_equals_the_triton_dequantize_kernels(name):
    case, cache, _ = build(name)
    ks, vs = cache_owned_segments(cache)
    want = dict(item.split(":") for item in GOLD[f"cuda/{name}/dequant_sha"].tolist())
    seen = 0
    for side, segments in (("k", ks), ("v", vs)):
        for i, seg in enumerate(segments):
            if isinstance(seg, torch.Tensor):
                continue
            restored = to_np(dart.triton_dequantize(seg))
            assert sha(restored) == want[f"{side}{i}"], f"{side} segment {i}"
            stored = GOLD.get(f"cuda/{name}/dequant_{side}{i}")
            if stored is not None:
                np.testing.assert_array_equal(restored, stored)
            seen += 1
    assert seen == len(want)


def check_16bit(out, ref16, ref32, tag, slack):
    """A 16-bit output against the reference's: one output ulp (or 2e-3) of its 16-bit result, and half an output
    ulp plus `slack` of its fp32 result."""

    diff = np.abs(out - ref16)
    assert np.all((diff <= 2e-3) | (diff <= np.abs(ref16) * 2 * HALF_ULP[tag] * 1.01)), float(diff.max())
    excess = np.abs(out - ref32) - np.abs(ref32) * HALF_ULP[tag]
    assert float(excess.max()) <= slack, float(excess.max())


@pytest.mark.parametrize("name", sorted(CASES))
def test_fp32_flavour_equals_the_reference_streamed_attention_on_cuda(name):
    case, cache, query = build(name)
    q3 = query[:, :, 0].cuda()
    scale = case.get("scale")
    ref32 = GOLD[f"cuda/{name}/streamed_f32"][:, :, 0]
    out32 = dart.decode_attention(q3.float(), cache, scale=scale, flavour=dart.DEQUANT_FP32)
    np.testing.assert_allclose(to_np(out32), ref32, rtol=0, atol=1e-5)
    if case["dt"] != "f32":
        out = dart.decode_attention(q3, cache, scale=scale, flavour=dart.DEQUANT_FP32)
        check_16bit(to_np(out), GOLD[f"cuda/{name}/streamed"][:, :, 0], ref32, case["dt"], slack=2e-5)
    assert cache.decode_status() == 0


@pytest.mark.parametrize("name", sorted(CASES))
def test_fused_flavour_equals_the_reference_triton_attention(name):
    case, cache, query = build(name)
    q3 = query[:, :, 0].cuda()
    scale = case.get("scale")
    ref32 = GOLD[f"cuda/{name}/fused_f32"][:, :, 0]
    # fp32 query: the generic kernel, fp32 arithmetic like the Triton kernels
    out32 = dart.decode_attention(q3.float(), cache, scale=scale, flavour=dart.DEQUANT_FUSED)
    np.testing.assert_allclose(to_np(out32), ref32, rtol=0, atol=1e-5)
    if case["dt"] != "f32":
        # 16-bit query: on the headline page geometry this is the tensor-core kernel, whose q*scale and p*scale
        # weights are fp16 (the high plane of promoted channels gets a second fp16 term).  Bar: 2e-3 on top of half
        # an output ulp of the Triton kernel's fp32 result; measured 5.8e-4 with promoted keys that have outlier
        # channels (|out| up to 2.5), 1.6e-3 with uniform 2-bit keys on the same data, 1e-4 on Gaussian keys
        out = dart.decode_attention(q3, cache, scale=scale, flavour=dart.DEQUANT_FUSED)
        ref16 = GOLD[f"cuda/{name}/fused"][:, :, 0]
        excess = np.abs(to_np(out) - ref32) - np.abs(ref32) * HALF_ULP[case["dt"]]
        assert float(excess.max()) <= 2e-3, float(excess.max())
        diff = np.abs(to_np(out) - ref16)
        assert np.all(diff <= 2e-3 + np.abs(ref16) * 2 * HALF_ULP[case["dt"]]), float(diff.max())
    assert cache.decode_status() == 0
