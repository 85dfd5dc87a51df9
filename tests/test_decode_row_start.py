"""How the Qwen3 adapter reads a decode step's attention mask (host logic, no GPU)."""

import types

import torch

from dartkv_b200.integrations.qwen3 import decode_row_start


def holder():
    return types.SimpleNamespace()


def test_no_mask_and_all_live_masks_mean_nothing_is_masked():
    assert decode_row_start(holder(), None, 7) is None
    assert decode_row_start(holder(), torch.ones(2, 7, dtype=torch.long), 7) is None
    assert decode_row_start(holder(), torch.zeros(2, 1, 1, 7), 7) is None
    assert decode_row_start(holder(), torch.ones(2, 1, 1, 7, dtype=torch.bool), 7) is None


def test_left_padding_gives_the_first_live_token_of_every_row():
    mask = torch.ones(3, 9, dtype=torch.long)
    mask[0, :4] = 0
    mask[2, :8] = 0
    assert decode_row_start(holder(), mask, 9).tolist() == [4, 0, 8]
    additive = torch.zeros(3, 1, 1, 9)
    additive[0, :, :, :4] = torch.finfo(torch.float32).min
    additive[2, :, :, :8] = float("-inf")
    got = decode_row_start(holder(), additive, 9)
    assert got.dtype == torch.int32 and got.tolist() == [4, 0, 8]
    boolean = additive == 0
    assert decode_row_start(holder(), boolean, 9).tolist() == [4, 0, 8]
    # a mask wider than the cache (preallocated): only the first kv_len columns count
    wide = torch.cat((mask, torch.zeros(3, 3, dtype=torch.long)), dim=1)
    assert decode_row_start(holder(), wide, 9).tolist() == [4, 0, 8]


def test_other_masks_are_left_to_the_dense_path():
    hole = torch.ones(2, 9, dtype=torch.long)
    hole[1, 3] = 0
    assert decode_row_start(holder(), hole, 9) is False
    right = torch.ones(2, 9, dtype=torch.long)
    right[0, 6:] = 0
    assert decode_row_start(holder(), right, 9) is False
    dead = torch.ones(2, 9, dtype=torch.long)
    dead[1] = 0
    assert decode_row_start(holder(), dead, 9) is False
    assert decode_row_start(holder(), torch.ones(2, 5, dtype=torch.long), 9) is False      # narrower than the cache
    assert decode_row_start(holder(), torch.ones(2, 3, 9), 9) is False                     # not a mask shape we know


def test_the_answer_is_kept_for_the_layers_of_one_step():
    cache = holder()
    mask = torch.ones(2, 9, dtype=torch.long)
    mask[0, :2] = 0
    first = decode_row_start(cache, mask, 9)
    assert decode_row_start(cache, mask, 9) is first
    mask[0, :3] = 0                              # modified in place: not the same step any more
    assert decode_row_start(cache, mask, 9).tolist() == [3, 0]


def test_graphed_decoder_refuses_caches_it_cannot_replay():
    import pytest

    import dartkv_b200 as dart
    from dartkv_b200.integrations import DartGraphedDecoder, DartHFCache

    with pytest.raises(ValueError, match="max_tokens"):
        DartGraphedDecoder(None, DartHFCache(dart.DartKVCacheConfig()))            # pools could move under the graph
    with pytest.raises(ValueError, match="max_tokens"):
        DartGraphedDecoder(None, object())
    with pytest.raises(ValueError, match="prompt"):
        DartGraphedDecoder(None, DartHFCache(dart.DartKVCacheConfig(), max_tokens=64))   # nothing cached yet
    with pytest.raises(ValueError, match="max_tokens"):
        DartHFCache(dart.DartKVCacheConfig(), graph_decode=True)
