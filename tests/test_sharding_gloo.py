"""The N>1 path on CPU: gloo ranks each own a rectangle of batch rows x KV heads, run the (oracle) decode
attention on their shard and gather the outputs; the result must equal the unsharded run.  Covered: an even
batch split, a ragged batch split, and a split over KV heads when there are more ranks than batch rows."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dartkv_b200.sharding import gather_outputs, shard_plan, shard_rows
from dartkv_b200.synthetic import make_kvq
from oracle import dartkv_oracle as orc

CFG = dict(bits=2, page_size=8, key_group_size=8, value_group_size=8, sink_tokens=2, hold_partial_pages=True,
           promote_ratio=0.25, metadata_dtype="f32")


def _attention(keys, values, query):
    cache = orc.OracleCache(orc.CacheConfig(**CFG), "f32")
    cache.append(keys, values)
    return orc.streamed_attention(query, cache, "f32")


def _worker(rank, world, port, result_path, batch):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    kv_heads, hq = 2, 4
    keys, values, query = (t.numpy() for t in make_kvq(5, batch, kv_heads, 29, 16, query_heads=hq, dtype=torch.float32))
    shard = shard_plan(batch, kv_heads, world, rank)
    rows = slice(shard.row_begin, shard.row_end)
    q_lo, q_hi = shard.query_heads(hq, kv_heads)
    local = torch.from_numpy(_attention(keys[rows, shard.head_begin:shard.head_end],
                                        values[rows, shard.head_begin:shard.head_end], query[rows, q_lo:q_hi]))
    full = gather_outputs(local, shard=shard, batch=batch, kv_heads=kv_heads)
    if rank == 0:
        np.save(result_path, full.numpy())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("batch,world", [(4, 2), (3, 2), (1, 2)], ids=["even", "ragged", "kv_heads"])
def test_sharded_attention_matches_single_rank(tmp_path, batch, world):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    result = str(tmp_path / "gathered.npy")
    mp.spawn(_worker, args=(world, port, result, batch), nprocs=world, join=True)
    keys, values, query = (t.numpy() for t in make_kvq(5, batch, 2, 29, 16, query_heads=4, dtype=torch.float32))
    np.testing.assert_array_equal(np.load(result), _attention(keys, values, query))


def test_shard_rows_validation():
    assert shard_rows(128, 8, 3) == (48, 64)
    assert [shard_rows(4, 2, r) for r in range(2)] == [(0, 2), (2, 4)]
    assert [shard_rows(10, 4, r) for r in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]   # ragged: first groups larger
    with pytest.raises(ValueError, match="fewer rows"):
        shard_rows(2, 4, 0)
    with pytest.raises(ValueError, match="rank"):
        shard_rows(8, 2, 2)
    t = torch.ones(2, 3)
    assert gather_outputs(t) is t   # no process group: identity


def test_shard_plan_covers_every_unit_exactly_once():
    for batch, heads, world in [(128, 8, 8), (4, 8, 8), (1, 8, 8), (3, 8, 4), (5, 8, 2), (2, 8, 8), (7, 4, 4)]:
        seen = np.zeros((batch, heads), dtype=np.int32)
        padded = set()
        for rank in range(world):
            s = shard_plan(batch, heads, world, rank)
            assert s.rows >= 1 and s.heads >= 1 and s.batch_groups * s.head_groups == world
            seen[s.row_begin:s.row_end, s.head_begin:s.head_end] += 1
            padded.add(s.rows_padded)
            assert s.rows <= s.rows_padded
        assert (seen == 1).all(), (batch, heads, world)
        assert len(padded) == 1
    # KV heads are split only when the batch cannot feed every rank
    assert shard_plan(8, 8, 8, 0).head_groups == 1
    assert shard_plan(4, 8, 8, 0).head_groups == 2
    with pytest.raises(ValueError, match="cannot shard"):
        shard_plan(1, 2, 8, 0)
