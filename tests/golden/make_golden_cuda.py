"""Record what the reference's own CUDA code paths compute, for the two dequantization flavours that only
exist there: its Triton dequantize kernels (one fp32 multiply-add rounded once, used by
``streamed_dart_attention`` on CUDA tensors) and its Triton attention kernels (``fused_dart_attention`` with the
fallback off, which never round the dequantized value).

Run on a machine with a CUDA device and an install of the unmodified reference package under ``oracle/_ref``
(``oracle/make_ref.sh`` makes one):

    python tests/golden/make_golden_cuda.py [output.npz]

Every cache is quantized by the reference on the CPU (so its packed bytes are the ones the CPU fixtures pin), then
moved to the GPU with the reference's own ``DartKVCache.to`` and read by its CUDA paths.  Inputs are regenerated
from the seeds in ``tests/golden/cases.py``; only outputs are stored.  The default output is
``tests/golden/cuda_reference.npz``, which the GPU parity tests read.
"""

from __future__ import annotations

import hashlib
import json
import os
import sys
import traceback

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle", "_ref"))

from tests.golden.cases import CACHE_CASES, CUDA_EXTRA_CASES, TORCH_DTYPES, build_inputs  # noqa: E402


def npy(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.float().numpy().copy()
    return t.numpy().copy()


def sha(*arrays: np.ndarray) -> str:
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def main() -> None:
    import dart  # the reference package, unmodified
    from dart.triton_ops import TRITON_AVAILABLE, triton_dequantize

    assert torch.cuda.is_available(), "needs a CUDA device"
    assert TRITON_AVAILABLE, "the reference did not find Triton"
    out_path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "cuda_reference.npz")
    out: dict = {}
    notes: dict = {"device": torch.cuda.get_device_name(0), "torch": torch.__version__}
    cases = dict(CACHE_CASES)
    cases.update(CUDA_EXTRA_CASES)
    for name, case in cases.items():
        keys, values, query = build_inputs(case)
        cfg_kwargs = dict(case["config"])
        cfg_kwargs["metadata_dtype"] = TORCH_DTYPES[cfg_kwargs.pop("md")]
        cache = dart.DartKVCache(dart.DartKVCacheConfig(**cfg_kwargs))
        # the promoted channels of every mixed key page, in the order the cache quantizes them: the parity tests
        # feed them to the append kernels so that the packed bytes are the ones read here
        import dart.cache as dart_cache
        calls = []
        original = dart_cache.quantize_key_mixed

        def recording(*args, **kwargs):
            result = original(*args, **kwargs)
            calls.append(result.channel_indices.numpy().copy())
            return result

        dart_cache.quantize_key_mixed = recording
        start = 0
        for chunk in case["chunks"]:
            cache.append(keys[..., start:start + chunk, :], values[..., start:start + chunk, :])
            start += chunk
        dart_cache.quantize_key_mixed = original
        scale = case.get("scale")
        prefix = f"cuda/{name}"
        if calls:
            out[f"{prefix}/mixed_indices"] = np.concatenate([c.reshape(c.shape[0], c.shape[1], -1, c.shape[-1])
                                                             for c in calls], axis=2)   # [B,H,pages,K]
        cpu_f32 = dart.streamed_dart_attention(query.float(), cache, scale=scale)
        out[f"{prefix}/cpu_streamed_f32"] = npy(cpu_f32)
        cache.to("cuda")
        q = query.cuda()
        results = {}
        for label, fn in (
            ("streamed", lambda: dart.streamed_dart_attention(q, cache, scale=scale)),
            ("streamed_f32", lambda: dart.streamed_dart_attention(q.float(), cache, scale=scale)),
            ("fused", lambda: dart.fused_dart_attention(q, cache, scale=scale, fallback=False)),
            ("fused_f32", lambda: dart.fused_dart_attention(q.float(), cache, scale=scale, fallback=False)),
        ):
            try:
                results[label] = npy(fn())
                out[f"{prefix}/{label}"] = results[label]
            except Exception as exc:  # recorded, not fatal: a path the reference does not support for this case
                notes[f"{name}/{label}"] = f"{type(exc).__name__}: {exc}"
                traceback.print_exc()
        # page dequantization by the Triton kernels: hashes always, arrays for small pages
        seg_shas = []
        for side, segments in (("k", cache._key_segments), ("v", cache._value_segments)):
            for i, seg in enumerate(segments):
                if isinstance(seg, torch.Tensor):
                    continue
                try:
                    restored = npy(triton_dequantize(seg))
                except Exception as exc:
                    notes[f"{name}/dequant_{side}{i}"] = f"{type(exc).__name__}: {exc}"
                    continue
                seg_shas.append(f"{side}{i}:{sha(restored)}")
                if restored.size <= 40000:
                    out[f"{prefix}/dequant_{side}{i}"] = restored
        out[f"{prefix}/dequant_sha"] = np.array(seg_shas)
        if "streamed_f32" in results:
            notes[f"{name}/cuda_vs_cpu_streamed_f32_max_abs"] = float(np.abs(results["streamed_f32"] - npy(cpu_f32)).max())
        if "fused_f32" in results and "streamed_f32" in results:
            notes[f"{name}/fused_vs_streamed_f32_max_abs"] = float(np.abs(results["fused_f32"] - results["streamed_f32"]).max())

    # how the reference's quantizer behaves on CUDA tensors compared with CPU tensors (scalar division quirk,
    # top-k ties): counts of differing bytes, for the record
    try:
        case = CACHE_CASES["headline_bf16"]
        keys, values, _ = build_inputs(case)
        page_k, page_v = keys[:, :, 32:160], values[:, :, 32:160]
        for bits in (2, 4, 8):
            a = dart.quantize(page_v, bits=bits, group_size=64)
            b = dart.quantize(page_v.cuda(), bits=bits, group_size=64)
            notes[f"quantize_cuda_vs_cpu/b{bits}"] = {
                "values_differ": int((a.values != b.values.cpu()).sum()), "of": int(a.values.numel()),
                "scale_differ": int((a.scale.float() != b.scale.cpu().float()).sum()),
                "zero_differ": int((a.zero_point.float() != b.zero_point.cpu().float()).sum())}
        a = dart.quantize_key_mixed(page_k, group_size=128, promote_ratio=0.25)
        b = dart.quantize_key_mixed(page_k.cuda(), group_size=128, promote_ratio=0.25)
        notes["quantize_key_mixed_cuda_vs_cpu"] = {
            "indices_equal": bool((a.channel_indices == b.channel_indices.cpu()).all()),
            "index_sets_equal": bool((a.channel_indices.sort(-1).values == b.channel_indices.cpu().sort(-1).values).all()),
            "low_differ": int((a.low_values != b.low_values.cpu()).sum()),
            "scale_differ": int((a.scale.float() != b.scale.cpu().float()).sum())}
    except Exception as exc:
        notes["quantize_cuda_vs_cpu"] = f"{type(exc).__name__}: {exc}"
        traceback.print_exc()

    out["notes"] = np.array(json.dumps(notes, indent=1, sort_keys=True))
    np.savez_compressed(out_path, **out)
    print(json.dumps(notes, indent=1, sort_keys=True))
    print(out_path, os.path.getsize(out_path), "bytes")


if __name__ == "__main__":
    main()
