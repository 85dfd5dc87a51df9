"""Cache lifecycle cases shared by the fixture generator and the parity tests.

Each case names a cache configuration (the keyword arguments of the reference's
``DartKVCacheConfig``, with ``md`` standing for ``metadata_dtype``), the data
dtype, the tensor shape and the sequence of append chunk lengths.  Small cases
store their inputs in the fixture; large ones are regenerated from the seed.
"""

from __future__ import annotations

import torch

from dartkv_b200.synthetic import make_kvq

TORCH_DTYPES = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}

_HEADLINE = dict(bits=2, promote_ratio=0.25, page_size=128, key_group_size=128, value_group_size=64,
                 sink_tokens=32, hold_partial_pages=True)

CACHE_CASES = {
    # reference tests/test_attention.py:6-30 (sink + mixed pages + partial last page, default flush mode)
    "attn_mixed_f32": dict(
        config=dict(page_size=5, key_group_size=5, value_group_size=4, promote_ratio=0.25, sink_tokens=1, md="f32"),
        dt="f32", shape=(1, 2, 19, 8), hq=4, chunks=[19], seed=7),
    # reference tests/test_attention.py:33-49 (pending page)
    "pending_f32": dict(
        config=dict(page_size=4, hold_partial_pages=True, key_group_size=4, value_group_size=4, md="f32"),
        dt="f32", shape=(1, 1, 7, 8), hq=1, chunks=[7], seed=8),
    # reference tests/test_fused_attention.py:30-53 (sink + mixed + pending + GQA, fp16)
    "fused_f16": dict(
        config=dict(page_size=8, sink_tokens=3, hold_partial_pages=True, key_group_size=8, value_group_size=8,
                    promote_ratio=0.25, md="f16"),
        dt="f16", shape=(1, 2, 21, 16), hq=4, chunks=[21], seed=72),
    # reference tests/test_cache.py:8-26 (4-bit, head_dim not divisible by the group, incremental)
    "incremental_4bit": dict(
        config=dict(bits=4, group_size=4, sink_tokens=2, md="f32"),
        dt="f32", shape=(1, 2, 5, 7), hq=2, chunks=[1, 4], seed=2),
    # default flush mode with single-token appends: partial key pages, coalesced value pages
    "partial_pages_bf16": dict(
        config=dict(bits=2, group_size=8, page_size=4, sink_tokens=1, md="bf16"),
        dt="bf16", shape=(2, 2, 12, 16), hq=4, chunks=[6, 1, 1, 3, 1], seed=11),
    # held pages with a dense local suffix (cache.py:408-419)
    "local_suffix_f16": dict(
        config=dict(bits=4, group_size=8, page_size=4, local_tokens=3, md="f16"),
        dt="f16", shape=(1, 2, 14, 16), hq=2, chunks=[9, 1, 1, 1, 1, 1], seed=12),
    # Kitty lifecycle, prefill ends on a page boundary: re-quantization on the first decode (cache.py:427-439)
    "kitty_boundary_f16": dict(
        config=dict(bits=2, page_size=8, local_tokens=1, value_local_tokens=8, hold_partial_pages=True,
                    sink_tokens=2, promote_ratio=0.25, key_group_size=8, value_group_size=8, md="f16"),
        dt="f16", shape=(1, 2, 30, 16), hq=4, chunks=[18] + [1] * 12, seed=13),
    # Kitty lifecycle, the token pattern of reference tests/test_reproduction.py:158-199
    "kitty_stream_bf16": dict(
        config=dict(bits=2, page_size=8, local_tokens=1, value_local_tokens=8, hold_partial_pages=True,
                    sink_tokens=0, promote_ratio=0.25, key_group_size=8, value_group_size=16, md="bf16"),
        dt="bf16", shape=(2, 2, 23, 16), hq=2, chunks=[13] + [1] * 10, seed=14),
    # uniform keys at 4 and 8 bits with the headline page geometry
    "uniform_4bit_bf16": dict(
        config=dict(bits=4, page_size=128, key_group_size=128, value_group_size=64, sink_tokens=32,
                    hold_partial_pages=True, md="bf16"),
        dt="bf16", shape=(1, 2, 200, 128), hq=8, chunks=[32, 128, 40], seed=15, outliers=True, store_inputs=False),
    "uniform_8bit_f16": dict(
        config=dict(bits=8, page_size=128, key_group_size=128, value_group_size=128, sink_tokens=32,
                    hold_partial_pages=True, md="f16"),
        dt="f16", shape=(1, 2, 200, 128), hq=4, chunks=[160, 40], seed=16, outliers=True, store_inputs=False),
    # CPU synthetic single-query decode: fp32, 2-bit, group 32, 2 sinks (with fp32 and default fp16 metadata)
    "config1_mdf32": dict(
        config=dict(bits=2, group_size=32, sink_tokens=2, md="f32"),
        dt="f32", shape=(1, 8, 256, 128), hq=8, chunks=[256], seed=0, outliers=False, store_inputs=False),
    "config1_mdf16": dict(
        config=dict(bits=2, group_size=32, sink_tokens=2, md="f16"),
        dt="f32", shape=(1, 8, 256, 128), hq=8, chunks=[256], seed=0, outliers=False, store_inputs=False),
    # headline geometry (2-bit + 0.25 promotion, page 128, groups 128/64, 32 sinks), shortened context
    "headline_bf16": dict(
        config=dict(_HEADLINE, md="bf16"),
        dt="bf16", shape=(2, 2, 32 + 3 * 128 + 96, 128), hq=8, chunks=[32, 128, 128, 128, 96], seed=2,
        outliers=True, store_inputs=False),
    "headline_bf16_mdf16": dict(
        config=dict(_HEADLINE, md="f16"),
        dt="bf16", shape=(1, 2, 32 + 2 * 128 + 17, 128), hq=8, chunks=[300, 5], seed=3,
        outliers=True, store_inputs=False),
    "headline_f16": dict(
        config=dict(_HEADLINE, md="f16"),
        dt="f16", shape=(1, 2, 32 + 2 * 128 + 96, 128), hq=8, chunks=[32 + 256 + 96], seed=4,
        outliers=True, store_inputs=False),
    # value bits 4 with promoted 2+2-bit keys (promotion overrides key_bits, cache.py:488-495)
    "promoted_v4_bf16": dict(
        config=dict(_HEADLINE, value_bits=4, md="bf16"),
        dt="bf16", shape=(1, 2, 32 + 128 + 9, 128), hq=4, chunks=[169], seed=5, outliers=True, store_inputs=False),
}

# Larger headline-geometry cases read only through the reference's CUDA code paths (make_golden_cuda.py): outputs
# of its Triton dequantize kernels and of its Triton attention kernels.
CUDA_EXTRA_CASES = {
    # config 3 geometry with a shorter context: 32 sinks + 16 pages + 96 pending tokens, outlier key channels
    "config3_short_bf16": dict(
        config=dict(_HEADLINE, md="bf16"),
        dt="bf16", shape=(2, 8, 32 + 16 * 128 + 96, 128), hq=32, chunks=[32, 16 * 128 + 96], seed=2,
        outliers=True, store_inputs=False),
    "config3_short_f16": dict(
        config=dict(_HEADLINE, md="f16"),
        dt="f16", shape=(1, 8, 32 + 8 * 128 + 96, 128), hq=32, chunks=[32, 8 * 128 + 96], seed=22,
        outliers=True, store_inputs=False),
    # the same without outlier channels (plain Gaussian keys)
    "gaussian_bf16": dict(
        config=dict(_HEADLINE, md="bf16"),
        dt="bf16", shape=(1, 4, 32 + 8 * 128 + 40, 128), hq=16, chunks=[32 + 8 * 128 + 40], seed=23,
        outliers=False, store_inputs=False),
    # uniform 2-bit keys (no promotion), value group 128
    "uniform_2bit_bf16": dict(
        config=dict(bits=2, page_size=128, key_group_size=128, value_group_size=128, sink_tokens=32,
                    hold_partial_pages=True, md="bf16"),
        dt="bf16", shape=(1, 4, 32 + 6 * 128 + 17, 128), hq=8, chunks=[32 + 6 * 128 + 17], seed=24,
        outliers=True, store_inputs=False),
}


def build_inputs(case: dict):
    """K, V ``[B,H,T,D]`` and query ``[B,Hq,1,D]`` for a case, on the CPU, in the case dtype."""

    b, h, t, d = case["shape"]
    dt = TORCH_DTYPES[case["dt"]]
    frac = 0.05 if case.get("outliers", False) else 0.0
    return make_kvq(case["seed"], b, h, t, d, query_heads=case["hq"], dtype=dt, outlier_fraction=frac)
