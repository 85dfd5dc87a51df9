"""Appends planned on the device (no host plan in the launches): same bytes as the host-planned path, and a whole
decode step (append + attention) captured once in a CUDA graph and replayed token after token."""

import pytest
import torch

import dartkv_b200 as dart
from dartkv_b200.synthetic import make_kvq

pytestmark = pytest.mark.gpu

CFG = dict(bits=2, promote_ratio=0.25, page_size=128, key_group_size=128, value_group_size=64, sink_tokens=32,
           hold_partial_pages=True)


def new_cache(dtype=torch.bfloat16, max_tokens=None, **overrides):
    cfg = dict(CFG)
    cfg.update(overrides)
    return dart.DartKVCache(dart.DartKVCacheConfig(metadata_dtype=dtype, **cfg), max_tokens=max_tokens)


def pools_equal(a, b):
    state = a._pools["state"][:5].tolist()
    assert state == b._pools["state"][:5].tolist()
    seen, pages, k_end, v_end, sink_filled = state
    sink = a.config.sink_tokens
    # the pools come from torch.empty: only what the appends wrote is comparable
    assert torch.equal(a._pools["k_sink"][:, :, :sink_filled], b._pools["k_sink"][:, :, :sink_filled])
    assert torch.equal(a._pools["v_sink"][:, :, :sink_filled], b._pools["v_sink"][:, :, :sink_filled])
    assert torch.equal(a._pools["k_pages"][:, :, :pages], b._pools["k_pages"][:, :, :pages])
    rows = max(0, v_end - sink)
    assert torch.equal(a._pools["v_codes"][:, :, :rows], b._pools["v_codes"][:, :, :rows])
    assert torch.equal(a._pools["v_meta"][:, :, :rows], b._pools["v_meta"][:, :, :rows])
    assert torch.equal(a._pools["page_start"][:pages], b._pools["page_start"][:pages])
    assert torch.equal(a._pools["page_tokens"][:pages], b._pools["page_tokens"][:pages])
    # ring rows that hold live (not yet packed) tokens, through the materialized cache
    keys_a, values_a = a.get()
    keys_b, values_b = b.get()
    assert torch.equal(keys_a, keys_b) and torch.equal(values_a, values_b)


@pytest.mark.parametrize("chunk", [1, 7, 128, 300])
@pytest.mark.parametrize("overrides", [dict(), dict(promote_ratio=0.0, bits=4), dict(value_group_size=128, sink_tokens=0),
                                       dict(local_tokens=1, value_local_tokens=128), dict(local_tokens=5),
                                       dict(hold_partial_pages=False, value_local_tokens=64)])
def test_same_bytes_as_the_host_planned_append(chunk, overrides):
    tokens = 40 + 3 * 128 + 2 * chunk + 70
    keys, values, query = make_kvq(3, 2, 2, tokens, 128, query_heads=8, dtype=torch.bfloat16)
    keys, values = keys.cuda(), values.cuda()
    host, device = new_cache(**overrides), new_cache(**overrides)
    host.append(keys[:, :, :40], values[:, :, :40])
    device.append(keys[:, :, :40], values[:, :, :40])
    start = 40
    while start < tokens:
        step = min(chunk, tokens - start)
        k, v = keys[:, :, start:start + step], values[:, :, start:start + step]
        host.append(k, v)
        device.append_device_planned(k, v)
        start += step
    assert host.seen_tokens == device.seen_tokens == tokens
    pools_equal(host, device)
    assert host.segment_table() == device.segment_table()
    out_host = dart.fused_dart_attention(query.cuda(), host, fallback=False)
    out_device = dart.fused_dart_attention(query.cuda(), device, fallback=False)
    assert torch.equal(out_host, out_device)
    device.check_finite()


def test_a_decode_step_replays_from_one_cuda_graph():
    batch, heads, hq, prompt, new_tokens = 2, 2, 8, 32 + 128 + 57, 330
    capacity = prompt + new_tokens + 128
    keys, values, _ = make_kvq(5, batch, heads, prompt + new_tokens, 128, query_heads=hq, dtype=torch.bfloat16)
    gen = torch.Generator().manual_seed(6)
    queries = torch.randn(new_tokens, batch, hq, 1, 128, generator=gen).to(torch.bfloat16).cuda()
    keys, values = keys.cuda(), values.cuda()
    eager, graphed = new_cache(max_tokens=capacity), new_cache(max_tokens=capacity)
    eager.append(keys[:, :, :prompt], values[:, :, :prompt])
    graphed.append(keys[:, :, :prompt], values[:, :, :prompt])
    k_in = torch.empty(batch, heads, 1, 128, dtype=torch.bfloat16, device="cuda")
    v_in = torch.empty_like(k_in)
    q_in = torch.empty(batch, hq, 1, 128, dtype=torch.bfloat16, device="cuda")
    out = torch.empty(batch, hq, 128, dtype=torch.bfloat16, device="cuda")
    pointers = {name: pool.data_ptr() for name, pool in graphed._pools.items()}

    def step():
        graphed.append_device_planned(k_in, v_in)
        dart.fused_dart_attention(q_in, graphed, fallback=False, token_capacity=capacity, out=out)

    # one eager step first (workspace allocation, kernel attributes), then the capture of the next step
    for t in range(2):
        k_in.copy_(keys[:, :, prompt + t:prompt + t + 1])
        v_in.copy_(values[:, :, prompt + t:prompt + t + 1])
        q_in.copy_(queries[t])
        if t == 0:
            step()
        else:
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
            # the capture only recorded the step (the host bookkeeping already counted it): run it
            graph.replay()
        eager.append(keys[:, :, prompt + t:prompt + t + 1], values[:, :, prompt + t:prompt + t + 1])
        expected = dart.fused_dart_attention(queries[t], eager, fallback=False)
        assert torch.equal(out.unsqueeze(2), expected), t
    for t in range(2, new_tokens):
        k_in.copy_(keys[:, :, prompt + t:prompt + t + 1])
        v_in.copy_(values[:, :, prompt + t:prompt + t + 1])
        q_in.copy_(queries[t])
        graphed.advance_device_planned(1)
        graph.replay()
        eager.append(keys[:, :, prompt + t:prompt + t + 1], values[:, :, prompt + t:prompt + t + 1])
        expected = dart.fused_dart_attention(queries[t], eager, fallback=False)
        assert torch.equal(out.unsqueeze(2), expected), t
    torch.cuda.synchronize()
    assert {name: pool.data_ptr() for name, pool in graphed._pools.items()} == pointers   # nothing was reallocated
    assert graphed.seen_tokens == eager.seen_tokens == prompt + new_tokens
    pools_equal(eager, graphed)
    assert graphed.decode_status() == 0


def test_what_device_planned_appends_refuse():
    keys, values, _ = make_kvq(7, 1, 2, 64, 128, query_heads=8, dtype=torch.bfloat16)
    keys, values = keys.cuda(), values.cuda()
    with pytest.raises(ValueError, match="first chunk"):
        new_cache().append_device_planned(keys, values)
    flushing = new_cache(hold_partial_pages=False)
    flushing.append(keys[:, :, :40], values[:, :, :40])
    with pytest.raises(ValueError, match="only pack full pages"):
        flushing.append_device_planned(keys[:, :, 40:41], values[:, :, 40:41])
    assert flushing.seen_tokens == 40      # a refused step leaves the bookkeeping where it was
    # Kitty lifecycle, prompt ending on a page boundary: the next one-token step re-quantizes that page
    big_k, big_v, _ = make_kvq(8, 1, 2, 32 + 128 + 1, 128, query_heads=8, dtype=torch.bfloat16)
    kitty = new_cache(local_tokens=1, value_local_tokens=128)
    kitty.append(big_k[:, :, :160].cuda(), big_v[:, :, :160].cuda())
    with pytest.raises(ValueError, match="re-quantizes"):
        kitty.append_device_planned(big_k[:, :, 160:].cuda(), big_v[:, :, 160:].cuda())
    assert kitty.seen_tokens == 160
    kitty.append(big_k[:, :, 160:].cuda(), big_v[:, :, 160:].cuda())
    kitty.append_device_planned(big_k[:, :, 160:].cuda(), big_v[:, :, 160:].cuda())   # later steps are fine
    assert kitty.seen_tokens == 162
