"""DartHFCache and the Qwen3 decode hook on a tiny random-weight Qwen3 (reference
tests/test_cache.py:265-308 and tests/test_reproduction.py:353-395)."""

import pytest
import torch

import dartkv_b200 as dart
from dartkv_b200.integrations import DartHFCache, attach_dart_fused_attention

pytestmark = pytest.mark.gpu


def tiny_model(head_dim=8, dtype=torch.float32):
    from transformers import Qwen3Config, Qwen3ForCausalLM

    torch.manual_seed(0)
    config = Qwen3Config(vocab_size=97, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=2, head_dim=head_dim, max_position_embeddings=128)
    config._attn_implementation = "eager"
    return Qwen3ForCausalLM(config).to(dtype).cuda().eval()


def test_hf_cache_postquant_return_and_reorder():
    torch.manual_seed(60)
    cfg = dart.DartKVCacheConfig(page_size=4, hold_partial_pages=True, key_group_size=4, value_group_size=4,
                                 metadata_dtype=torch.float32)
    cache = DartHFCache(cfg)
    keys = torch.randn(2, 2, 6, 8).cuda()
    values = torch.randn_like(keys)
    k0, v0 = cache.update(keys[..., :5, :], values[..., :5, :], 0)
    # prefill returns the raw tensors (attention sees the step's K/V before they are packed)
    assert torch.equal(k0, keys[..., :5, :]) and cache.last_update_was_prefill(0)
    assert cache.get_seq_length() == 5
    k1, v1 = cache.update(keys[..., 5:, :], values[..., 5:, :], 0)
    assert not cache.last_update_was_prefill(0)
    assert k1.shape[-2] == 6 and torch.equal(k1[..., 5:, :], keys[..., 5:, :])
    prior, _ = cache.layer_for_attention(0).get()
    assert torch.equal(k1[..., :5, :], prior[..., :5, :])       # history comes back dequantized
    k2, _ = cache.update(keys[..., :1, :], values[..., :1, :], 0, {"dart_fused_attention": True})
    assert k2.shape[-2] == 1                                     # fused update: only the new token
    assert cache.storage_bytes < cache.dense_bytes and cache.compression_ratio > 1.0
    assert cache.page_table(0).seen_tokens == 7 and cache.get_max_cache_shape() is None
    before = cache.layer_for_attention(0).get()[0]
    cache.reorder_cache(torch.tensor([1, 0]).cuda())
    after = cache.layer_for_attention(0).get()[0]
    assert after.shape == before.shape
    with pytest.raises(RuntimeError, match="not been initialized"):
        cache.layer_for_attention(3)


@pytest.mark.parametrize("head_dim,dtype", [(8, torch.float32), (128, torch.bfloat16)])
def test_tiny_qwen3_dart_engine_generation(head_dim, dtype):
    model = attach_dart_fused_attention(tiny_model(head_dim, dtype))
    page = 4 if head_dim == 8 else 128
    cfg = dart.DartKVCacheConfig(
        bits=2, page_size=page, hold_partial_pages=True, local_tokens=1, value_local_tokens=page,
        key_group_size=page, value_group_size=min(64, head_dim), sink_tokens=2, promote_ratio=0.25,
        metadata_dtype=torch.float32 if dtype == torch.float32 else dtype)
    prompt_len, new_tokens = (13, 20) if head_dim == 8 else (150, 140)
    torch.manual_seed(1)
    prompt = torch.randint(0, 97, (2, prompt_len)).cuda()
    cache = DartHFCache(cfg)
    with torch.no_grad():
        out = model.generate(prompt, max_new_tokens=new_tokens, min_new_tokens=new_tokens, do_sample=False,
                             past_key_values=cache, use_cache=True, disable_compile=True, pad_token_id=0)
    assert out.shape == (2, prompt_len + new_tokens)
    assert cache.get_seq_length() == prompt_len + new_tokens - 1
    for layer in range(2):
        assert cache.layer_for_attention(layer).decode_status() == 0
        cache.layer_for_attention(layer).check_finite()


def test_fused_hook_matches_materializing_path_logits():
    """One decode step: the fused hook equals dense attention over the materialized (dequantized) cache."""

    model = tiny_model(8, torch.float32)
    cfg = dart.DartKVCacheConfig(bits=4, page_size=4, hold_partial_pages=True, key_group_size=4, value_group_size=8,
                                 sink_tokens=1, promote_ratio=0.25, metadata_dtype=torch.float32)
    torch.manual_seed(2)
    prompt = torch.randint(0, 97, (2, 11)).cuda()
    nxt = torch.randint(0, 97, (2, 1)).cuda()
    with torch.no_grad():
        plain = DartHFCache(cfg)
        model(prompt, past_key_values=plain, use_cache=True)
        expected = model(nxt, past_key_values=plain, use_cache=True).logits
        attach_dart_fused_attention(model)
        fused = DartHFCache(cfg)
        model(prompt, past_key_values=fused, use_cache=True)
        got = model(nxt, past_key_values=fused, use_cache=True).logits
    torch.testing.assert_close(got, expected, rtol=2e-3, atol=2e-3)


def test_decode_hook_greedy_tokens_equal_the_reference_hook():
    """The reference's tiny Qwen3 run (tests/test_reproduction.py:353-395: 13-token prompt + 20 greedy tokens,
    Kitty lifecycle, fp32) through its own dart-engine hook on the CPU gives these token ids and logits; the
    same weights through this package's hook and kernels must give the same tokens."""

    import numpy as np

    from tests.golden.make_golden import TINY_QWEN3, TINY_QWEN3_CACHE, tiny_qwen3
    from tests.helpers import load_golden

    gold = load_golden("qwen3_hook.npz")
    model = tiny_qwen3()
    checksum = float(sum(p.detach().double().abs().sum() for p in model.parameters()))
    assert abs(checksum - float(gold["weight_checksum"])) < 1e-6 * checksum, "the seeded weights differ from the recorded run"
    model = attach_dart_fused_attention(model.cuda())
    cache = DartHFCache(dart.DartKVCacheConfig(metadata_dtype=torch.float32, **TINY_QWEN3_CACHE))
    prompt = torch.from_numpy(gold["prompt"]).cuda()
    tokens = prompt
    with torch.no_grad():
        logits = model(prompt, past_key_values=cache, use_cache=True).logits[:, -1]
        for step in range(20):
            np.testing.assert_allclose(logits.cpu().numpy(), gold["logits"][step], rtol=0, atol=2e-4)
            nxt = logits.argmax(-1, keepdim=True)
            tokens = torch.cat((tokens, nxt), dim=1)
            logits = model(nxt, past_key_values=cache, use_cache=True).logits[:, -1]
    assert tokens.shape == (2, 13 + 20) and TINY_QWEN3["vocab_size"] == 128
    np.testing.assert_array_equal(tokens.cpu().numpy(), gold["tokens"])
    assert cache.get_seq_length() == 33


def _padded_step(model, cache_cfg, prompt, mask, nxt):
    positions = (mask.cumsum(-1) - 1).clamp(min=0)
    cache = DartHFCache(cache_cfg)
    model(prompt, attention_mask=mask, position_ids=positions, past_key_values=cache, use_cache=True)
    step_mask = torch.cat((mask, torch.ones_like(mask[:, :1])), dim=1)
    step_pos = positions[:, -1:] + 1
    return model(nxt, attention_mask=step_mask, position_ids=step_pos, past_key_values=cache, use_cache=True).logits


@pytest.mark.parametrize("hole", [False, True])
def test_fused_hook_honours_the_attention_mask(hole, monkeypatch):
    """Left-padded batch: the hook turns the mask into per-row first live tokens for the packed kernels.  A mask
    with a hole is not a left padding and goes through the dense path.  Both equal the materializing path."""

    from dartkv_b200.integrations import qwen3 as adapter

    fused_calls = []
    kernel_entry = adapter.fused_dart_attention

    def counted(*args, **kwargs):
        fused_calls.append(kwargs.get("row_start"))
        return kernel_entry(*args, **kwargs)

    monkeypatch.setattr(adapter, "fused_dart_attention", counted)
    model = tiny_model(8, torch.float32)
    cfg = dart.DartKVCacheConfig(bits=4, page_size=4, hold_partial_pages=True, key_group_size=4, value_group_size=8,
                                 sink_tokens=1, promote_ratio=0.25, metadata_dtype=torch.float32)
    torch.manual_seed(3)
    prompt = torch.randint(0, 97, (3, 11)).cuda()
    nxt = torch.randint(0, 97, (3, 1)).cuda()
    mask = torch.ones(3, 11, dtype=torch.long).cuda()
    mask[0, :5] = 0
    mask[2, :1] = 0
    if hole:
        mask[1, 4] = 0
    with torch.no_grad():
        expected = _padded_step(model, cfg, prompt, mask, nxt)
        unmasked = _padded_step(model, cfg, prompt, torch.ones_like(mask), nxt)
        attach_dart_fused_attention(model)
        got = _padded_step(model, cfg, prompt, mask, nxt)
    torch.testing.assert_close(got, expected, rtol=2e-3, atol=2e-3)
    assert (expected[0] - unmasked[0]).abs().max() > 1e-2          # the mask matters for the padded row
    if hole:
        assert fused_calls == []                                    # both layers took the dense path
    else:
        assert [starts.tolist() for starts in fused_calls] == [[5, 0, 1]] * 2      # one packed call per layer


def test_graph_decode_replays_the_layer_step_and_agrees_with_the_eager_hook():
    """``DartHFCache(graph_decode=True)``: after the first two steps every layer replays one CUDA graph (append planned
    on the device + decode attention); the logits follow the eager hook (the work split of the attention differs,
    so sums are reordered) and the packed caches are byte-equal."""

    from transformers import Qwen3Config, Qwen3ForCausalLM

    from dartkv_b200.integrations.huggingface import _LayerDecodeGraph

    torch.manual_seed(0)
    config = Qwen3Config(vocab_size=97, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=2, head_dim=128, max_position_embeddings=1024)
    config._attn_implementation = "eager"
    model = attach_dart_fused_attention(Qwen3ForCausalLM(config).to(torch.bfloat16).cuda().eval())
    cfg = dart.DartKVCacheConfig(bits=2, promote_ratio=0.25, page_size=128, key_group_size=128, value_group_size=64,
                                 sink_tokens=32, hold_partial_pages=True, local_tokens=1, value_local_tokens=128,
                                 metadata_dtype=torch.float16)
    prompt = torch.randint(0, 97, (2, 32 + 128 + 40)).cuda()
    steps = 150
    eager, graphed = DartHFCache(cfg), DartHFCache(cfg, max_tokens=prompt.shape[1] + steps + 8, graph_decode=True)
    with torch.no_grad():
        logits_e = model(prompt, past_key_values=eager, use_cache=True).logits[:, -1]
        logits_g = model(prompt, past_key_values=graphed, use_cache=True).logits[:, -1]
        assert torch.equal(logits_e, logits_g)
        for step in range(steps):
            nxt = logits_e.argmax(-1, keepdim=True)
            logits_e = model(nxt, past_key_values=eager, use_cache=True).logits[:, -1]
            logits_g = model(nxt, past_key_values=graphed, use_cache=True).logits[:, -1]
            torch.testing.assert_close(logits_g.float(), logits_e.float(), rtol=2e-2, atol=2e-2)
    assert all(isinstance(graphed._decode_graphs[i], _LayerDecodeGraph) for i in range(2))
    assert graphed.get_seq_length() == eager.get_seq_length() == prompt.shape[1] + steps
    for index in range(2):
        a, b = eager.layer_for_attention(index), graphed.layer_for_attention(index)
        assert a.segment_table() == b.segment_table()
        keys_a, values_a = a.get()
        keys_b, values_b = b.get()
        # layer 0 sees identical inputs: identical bytes; deeper layers inherit the reordered sums of the layers before
        if index == 0:
            assert torch.equal(keys_a, keys_b) and torch.equal(values_a, values_b)
        assert b.decode_status() == 0


def test_graph_decode_needs_max_tokens_and_falls_back_where_the_geometry_does_not_fit():
    with pytest.raises(ValueError, match="max_tokens"):
        DartHFCache(dart.DartKVCacheConfig(), graph_decode=True)
    model = attach_dart_fused_attention(tiny_model(8, torch.float32))      # head_dim 8: generic kernels, eager steps
    cfg = dart.DartKVCacheConfig(bits=4, page_size=4, hold_partial_pages=True, key_group_size=4, value_group_size=8,
                                 sink_tokens=1, promote_ratio=0.25, metadata_dtype=torch.float32)
    torch.manual_seed(4)
    prompt = torch.randint(0, 97, (2, 9)).cuda()
    plain, graphed = DartHFCache(cfg), DartHFCache(cfg, max_tokens=64, graph_decode=True)
    with torch.no_grad():
        a = model(prompt, past_key_values=plain, use_cache=True).logits[:, -1]
        b = model(prompt, past_key_values=graphed, use_cache=True).logits[:, -1]
        for _ in range(6):
            nxt = a.argmax(-1, keepdim=True)
            a = model(nxt, past_key_values=plain, use_cache=True).logits[:, -1]
            b = model(nxt, past_key_values=graphed, use_cache=True).logits[:, -1]
            assert torch.equal(a, b)
    assert graphed._decode_graphs == {0: False, 1: False}


def test_graph_decode_with_a_left_padded_batch():
    from transformers import Qwen3Config, Qwen3ForCausalLM

    from dartkv_b200.integrations.huggingface import _LayerDecodeGraph

    torch.manual_seed(1)
    config = Qwen3Config(vocab_size=97, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=2, head_dim=128, max_position_embeddings=1024)
    config._attn_implementation = "eager"
    model = attach_dart_fused_attention(Qwen3ForCausalLM(config).to(torch.bfloat16).cuda().eval())
    cfg = dart.DartKVCacheConfig(bits=2, promote_ratio=0.25, page_size=128, key_group_size=128, value_group_size=64,
                                 sink_tokens=32, hold_partial_pages=True, metadata_dtype=torch.bfloat16)
    length, steps = 32 + 128 + 20, 12
    prompt = torch.randint(0, 97, (2, length)).cuda()
    mask = torch.ones(2, length, dtype=torch.long).cuda()
    mask[0, :37] = 0
    positions = (mask.cumsum(-1) - 1).clamp(min=0)
    eager, graphed = DartHFCache(cfg), DartHFCache(cfg, max_tokens=length + steps + 8, graph_decode=True)
    with torch.no_grad():
        outs = []
        for cache in (eager, graphed):
            logits = model(prompt, attention_mask=mask, position_ids=positions, past_key_values=cache,
                           use_cache=True).logits[:, -1]
            step_mask, step_pos, trace = mask, positions[:, -1:], []
            for _ in range(steps):
                nxt = logits.argmax(-1, keepdim=True) if cache is eager else outs[0][len(trace)][0]
                step_mask = torch.cat((step_mask, torch.ones_like(step_mask[:, :1])), dim=1)
                step_pos = step_pos + 1
                logits = model(nxt, attention_mask=step_mask, position_ids=step_pos, past_key_values=cache,
                               use_cache=True).logits[:, -1]
                trace.append((nxt, logits))
            outs.append(trace)
    for (tok_e, log_e), (tok_g, log_g) in zip(*outs):
        assert torch.equal(tok_e, tok_g)
        torch.testing.assert_close(log_g.float(), log_e.float(), rtol=2e-2, atol=2e-2)
    assert all(isinstance(graphed._decode_graphs[i], _LayerDecodeGraph) for i in range(2))
    assert graphed._decode_graphs[0].row_start.tolist() == [37, 0]


@pytest.mark.parametrize("padded", [False, True])
def test_whole_generation_step_as_one_cuda_graph(padded):
    """DartGraphedDecoder: the model's forward for one new token is captured once (device-planned appends, attention
    sized for the capacity) and replayed; tokens and logits follow the eager hook."""

    from transformers import Qwen3Config, Qwen3ForCausalLM

    from dartkv_b200.integrations import DartGraphedDecoder

    torch.manual_seed(2)
    config = Qwen3Config(vocab_size=97, hidden_size=64, intermediate_size=128, num_hidden_layers=3,
                         num_attention_heads=4, num_key_value_heads=2, head_dim=128, max_position_embeddings=1024)
    config._attn_implementation = "sdpa"
    model = attach_dart_fused_attention(Qwen3ForCausalLM(config).to(torch.bfloat16).cuda().eval())
    cfg = dart.DartKVCacheConfig(bits=2, promote_ratio=0.25, page_size=128, key_group_size=128, value_group_size=64,
                                 sink_tokens=32, hold_partial_pages=True, local_tokens=1, value_local_tokens=128,
                                 metadata_dtype=torch.float16)
    length, steps = 32 + 128, 140       # the prompt ends on a page boundary: the first step re-quantizes that page
    prompt = torch.randint(0, 97, (2, length)).cuda()
    mask = torch.ones(2, length, dtype=torch.long).cuda()
    if padded:
        mask[1, :21] = 0
    positions = (mask.cumsum(-1) - 1).clamp(min=0)
    eager, graphed = DartHFCache(cfg), DartHFCache(cfg, max_tokens=length + steps + 8)
    with torch.no_grad():
        logits_e = model(prompt, attention_mask=mask, position_ids=positions, past_key_values=eager,
                         use_cache=True).logits[:, -1]
        logits_g = model(prompt, attention_mask=mask, position_ids=positions, past_key_values=graphed,
                         use_cache=True).logits[:, -1]
        assert torch.equal(logits_e, logits_g)
        decoder = DartGraphedDecoder(model, graphed, position_ids=positions[:, -1:] + 1,
                                     row_start=torch.tensor([0, 21]) if padded else None)
        step_mask, step_pos = mask, positions[:, -1:]
        for step in range(steps):
            nxt = logits_e.argmax(-1, keepdim=True)
            step_mask = torch.cat((step_mask, torch.ones_like(step_mask[:, :1])), dim=1)
            step_pos = step_pos + 1
            logits_e = model(nxt, attention_mask=step_mask, position_ids=step_pos, past_key_values=eager,
                             use_cache=True).logits[:, -1]
            logits_g = decoder.step(nxt)
            torch.testing.assert_close(logits_g.float(), logits_e.float(), rtol=3e-2, atol=3e-2)
    assert decoder.graph is not None
    assert graphed.get_seq_length() == eager.get_seq_length() == length + steps
    first_e, first_g = eager.layer_for_attention(0), graphed.layer_for_attention(0)
    assert first_e.segment_table() == first_g.segment_table()
    keys_e, values_e = first_e.get()
    keys_g, values_g = first_g.get()
    assert torch.equal(keys_e, keys_g) and torch.equal(values_e, values_g)     # layer 0 sees identical inputs
    assert all(graphed.layer_for_attention(i).decode_status() == 0 for i in range(3))
