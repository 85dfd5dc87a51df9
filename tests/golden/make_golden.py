"""Generate the golden fixtures in this directory by running the reference implementation.

Run from the repository root on a machine that has the reference checkout:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's own ``dart`` package (CPU, unmodified), feeds it
seeded inputs and stores inputs (when small), packed fields, scales, zero
points, promoted channel indices, materialized caches and page-streamed
attention outputs as ``.npz`` files.  Nothing else in the repository needs the
reference checkout: the tests only read the ``.npz`` files written here.
"""

from __future__ import annotations

import hashlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from dartkv_b200.synthetic import make_kvq  # noqa: E402
from tests.golden.cases import CACHE_CASES, TORCH_DTYPES, build_inputs  # noqa: E402


def npy(t: torch.Tensor) -> np.ndarray:
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.float().numpy().copy()
    return t.numpy().copy()


def sha(*arrays: np.ndarray) -> str:
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def primitives(dart, out: dict) -> None:
    # uniform quantizer -------------------------------------------------------
    for dt_name, dt in TORCH_DTYPES.items():
        for bits in (2, 4, 8):
            gen = torch.Generator().manual_seed(100 + bits)
            cases = {
                "odd": (torch.randn(2, 3, 7, generator=gen), dict(group_size=4, metadata_dtype=torch.float32), -1),
                "row": (torch.randn(2, 2, 16, 64, generator=gen) * 3.0, dict(group_size=32), -1),
                "tok": (torch.randn(2, 3, 9, 5, generator=gen), dict(group_size=4), -2),
                "big": (torch.randn(1, 1, 48, 128, generator=gen), dict(group_size=64, metadata_dtype=torch.float16), -1),
                "key": (torch.randn(1, 1, 128, 48, generator=gen) * 4.0, dict(group_size=128), -2),
            }
            for name, (data, kwargs, axis) in cases.items():
                data = data.to(dt)
                q = dart.quantize(data, bits=bits, axis=axis, **kwargs)
                key = f"quant/{dt_name}/b{bits}/{name}"
                out[f"{key}/input"] = npy(data)
                out[f"{key}/values"] = q.values.numpy().copy()
                out[f"{key}/scale"] = npy(q.scale)
                out[f"{key}/zero"] = npy(q.zero_point)
                out[f"{key}/dequant"] = npy(q.dequantize())
                out[f"{key}/meta"] = np.array([axis, kwargs["group_size"], q.padded_dim, q.packed_dim], dtype=np.int64)
                md = {torch.float32: "f32", torch.float16: "f16", torch.bfloat16: "bf16"}[q.scale.dtype]
                out[f"{key}/md"] = np.array(md)

    # mixed keys ---------------------------------------------------------------
    mixed_cases = {
        "tiny_f32": ("f32", (1, 2, 17, 16), 8, None, False),
        "page_bf16": ("bf16", (1, 2, 128, 128), 128, None, True),
        "page_f16": ("f16", (1, 2, 128, 128), 128, None, True),
        "page_bf16_mdf16": ("bf16", (1, 1, 128, 128), 128, torch.float16, True),
        "ragged_bf16": ("bf16", (1, 2, 37, 32), 16, None, False),
        "ragged_f16_g5": ("f16", (2, 1, 11, 12), 5, torch.float32, False),
    }
    for name, (dt_name, shape, group, md, outliers) in mixed_cases.items():
        dt = TORCH_DTYPES[dt_name]
        b, h, t, d = shape
        keys, _, _ = make_kvq(200 + len(name), b, h, t, d, dtype=dt, outlier_fraction=0.05 if outliers else 0.0)
        for strategy in ("magnitude", "variance"):
            m = dart.quantize_key_mixed(keys, group_size=group, promote_ratio=0.25, metadata_dtype=md, strategy=strategy)
            key = f"mixed/{name}/{strategy}"
            if strategy == "magnitude":
                out[f"mixed/{name}/input"] = npy(keys)
                out[f"mixed/{name}/score_magnitude"] = npy(keys.abs().mean(dim=-2))
                centered = keys - keys.mean(dim=-2, keepdim=True)
                out[f"mixed/{name}/score_variance"] = npy(centered.square().mean(dim=-2))
                out[f"mixed/{name}/group"] = np.array(group)
                out[f"mixed/{name}/dt"] = np.array(dt_name)
            out[f"{key}/low"] = m.low_values.numpy().copy()
            out[f"{key}/high"] = m.high_values.numpy().copy()
            out[f"{key}/indices"] = m.channel_indices.numpy().copy()
            out[f"{key}/scale"] = npy(m.scale)
            out[f"{key}/zero"] = npy(m.zero_point)
            out[f"{key}/dequant"] = npy(m.dequantize())
            mdn = {torch.float32: "f32", torch.float16: "f16", torch.bfloat16: "bf16"}[m.scale.dtype]
            out[f"{key}/md"] = np.array(mdn)


def cache_cases(dart, out: dict) -> None:
    for name, case in CACHE_CASES.items():
        keys, values, query = build_inputs(case)
        cfg_kwargs = dict(case["config"])
        cfg_kwargs["metadata_dtype"] = TORCH_DTYPES[cfg_kwargs.pop("md")]
        cache = dart.DartKVCache(dart.DartKVCacheConfig(**cfg_kwargs))
        # record the promoted channels of every mixed key page in the order the cache quantizes them
        # (the re-quantized boundary page of the Kitty lifecycle appears twice)
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
        assert start == keys.shape[-2]
        dart_cache.quantize_key_mixed = original
        prefix = f"cache/{name}"
        if case.get("store_inputs", True):
            out[f"{prefix}/keys"] = npy(keys)
            out[f"{prefix}/values"] = npy(values)
            out[f"{prefix}/query"] = npy(query)
        got_k, got_v = cache.get()
        small = got_k.numel() <= 70000
        if small:
            out[f"{prefix}/get_k"] = npy(got_k)
            out[f"{prefix}/get_v"] = npy(got_v)
        out[f"{prefix}/get_sha"] = np.array(sha(npy(got_k), npy(got_v)))
        out[f"{prefix}/storage_bytes"] = np.array(cache.storage_bytes)
        out[f"{prefix}/dense_bytes"] = np.array(cache.dense_bytes)
        table = cache.page_table()
        out[f"{prefix}/table"] = np.stack([
            table.sequence_starts.numpy(), table.token_counts.numpy(),
            table.key_modes.numpy().astype(np.int32), table.value_modes.numpy().astype(np.int32)], axis=1)
        # packed fields of the cache-owned segment lists (before the boundary union)
        idx_list = []
        key_rows = []
        for i, seg in enumerate(cache._key_segments):
            if isinstance(seg, torch.Tensor):
                key_rows.append((0, seg.shape[-2]))
                field_arrays = [npy(seg)]
            elif isinstance(seg, dart.MixedQuantizedKey):
                key_rows.append((2, seg.original_shape[-2]))
                idx_list.append(seg.channel_indices.numpy().copy())
                field_arrays = [seg.low_values.numpy(), seg.high_values.numpy(), seg.channel_indices.numpy(),
                                npy(seg.scale), npy(seg.zero_point)]
                if small:
                    out[f"{prefix}/k{i}/low"] = field_arrays[0].copy()
                    out[f"{prefix}/k{i}/high"] = field_arrays[1].copy()
                    out[f"{prefix}/k{i}/scale"] = field_arrays[3]
                    out[f"{prefix}/k{i}/zero"] = field_arrays[4]
            else:
                key_rows.append((1, seg.original_shape[-2]))
                field_arrays = [seg.values.numpy(), npy(seg.scale), npy(seg.zero_point)]
                if small:
                    out[f"{prefix}/k{i}/values"] = field_arrays[0].copy()
                    out[f"{prefix}/k{i}/scale"] = field_arrays[1]
                    out[f"{prefix}/k{i}/zero"] = field_arrays[2]
            out[f"{prefix}/k{i}/sha"] = np.array(sha(*field_arrays))
        value_rows = []
        for i, seg in enumerate(cache._value_segments):
            if isinstance(seg, torch.Tensor):
                value_rows.append((0, seg.shape[-2]))
                field_arrays = [npy(seg)]
            else:
                value_rows.append((1, seg.original_shape[-2]))
                field_arrays = [seg.values.numpy(), npy(seg.scale), npy(seg.zero_point)]
                if small:
                    out[f"{prefix}/v{i}/values"] = field_arrays[0].copy()
                    out[f"{prefix}/v{i}/scale"] = field_arrays[1]
                    out[f"{prefix}/v{i}/zero"] = field_arrays[2]
            out[f"{prefix}/v{i}/sha"] = np.array(sha(*field_arrays))
        out[f"{prefix}/key_segments"] = np.array(key_rows, dtype=np.int64).reshape(-1, 2)
        out[f"{prefix}/value_segments"] = np.array(value_rows, dtype=np.int64).reshape(-1, 2)
        pend_k = 0 if cache._pending_key is None else cache._pending_key.shape[-2]
        pend_v = 0 if cache._pending_value is None else cache._pending_value.shape[-2]
        out[f"{prefix}/pending"] = np.array([pend_k, pend_v], dtype=np.int64)
        if calls:
            out[f"{prefix}/mixed_indices"] = np.stack(calls, axis=0)
        scale = case.get("scale")
        out[f"{prefix}/attn"] = npy(dart.streamed_dart_attention(query, cache, scale=scale))
        out[f"{prefix}/attn_f32"] = npy(dart.streamed_dart_attention(query.float(), cache, scale=scale))
        rep = query.shape[1] // keys.shape[1]
        dense = dart.dense_attention(query, keys.repeat_interleave(rep, dim=1), values.repeat_interleave(rep, dim=1),
                                     scale=scale)
        out[f"{prefix}/dense_unquantized"] = npy(dense)


TINY_QWEN3 = dict(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                  num_key_value_heads=2, head_dim=8, max_position_embeddings=128)
TINY_QWEN3_CACHE = dict(key_bits=2, value_bits=2, key_group_size=8, value_group_size=8, sink_tokens=2, page_size=8,
                        local_tokens=1, value_local_tokens=8, hold_partial_pages=True, promote_bits=4,
                        promote_ratio=0.25)


def tiny_qwen3(seed: int = 0):
    """The two-layer Qwen3 of the reference's tests/test_reproduction.py:353-395, weights drawn on the CPU."""

    from transformers import Qwen3Config, Qwen3ForCausalLM

    torch.manual_seed(seed)
    config = Qwen3Config(**TINY_QWEN3)
    config._attn_implementation = "eager"
    return Qwen3ForCausalLM(config).eval()


def qwen3_hook_case(dart, out: dict) -> None:
    """Greedy tokens of the reference's dart-engine decode hook: 13-token prompt + 20 new tokens, batch 2, fp32."""

    from oracle.ref_compat import patch_reference_integrations

    patch_reference_integrations(dart)
    from dart.integrations import DartHFCache, attach_dart_fused_attention

    model = attach_dart_fused_attention(tiny_qwen3())
    gen = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, TINY_QWEN3["vocab_size"], (2, 13), generator=gen)
    cache = DartHFCache(dart.DartKVCacheConfig(metadata_dtype=torch.float32, **TINY_QWEN3_CACHE))
    tokens = prompt
    margins = []
    step_logits = []
    with torch.inference_mode():
        logits = model(prompt, past_key_values=cache, use_cache=True).logits[:, -1]
        for _ in range(20):
            top2 = logits.topk(2, dim=-1).values
            margins.append((top2[:, 0] - top2[:, 1]).numpy().copy())
            step_logits.append(logits.numpy().copy())
            nxt = logits.argmax(-1, keepdim=True)
            tokens = torch.cat((tokens, nxt), dim=1)
            logits = model(nxt, past_key_values=cache, use_cache=True).logits[:, -1]
    assert tokens.shape == (2, 33) and cache.get_seq_length() == 33
    out["prompt"] = prompt.numpy()
    out["tokens"] = tokens.numpy()
    out["margins"] = np.stack(margins)          # [step, batch] gap between the two largest logits
    out["logits"] = np.stack(step_logits)       # [step, batch, vocab]
    out["weight_checksum"] = np.array(float(sum(p.detach().double().abs().sum() for p in model.parameters())))
    print("tiny Qwen3 hook: smallest top-2 logit margin", float(np.min(out["margins"])))


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path to a checkout of the reference project>")
    reference = sys.argv[1]
    sys.path.insert(0, os.path.join(reference, "src"))
    import dart  # the reference package, unmodified

    torch.set_num_threads(8)
    prim: dict = {}
    primitives(dart, prim)
    np.savez_compressed(os.path.join(HERE, "primitives.npz"), **prim)
    caches: dict = {}
    cache_cases(dart, caches)
    np.savez_compressed(os.path.join(HERE, "caches.npz"), **caches)
    hook: dict = {}
    qwen3_hook_case(dart, hook)
    np.savez_compressed(os.path.join(HERE, "qwen3_hook.npz"), **hook)
    for fn in ("primitives.npz", "caches.npz", "qwen3_hook.npz"):
        print(fn, os.path.getsize(os.path.join(HERE, fn)), "bytes")


if __name__ == "__main__":
    main()
