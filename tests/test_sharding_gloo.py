"""The N>1 path on CPU: two gloo ranks each own half of the batch rows, run the (oracle) decode
attention on their shard and gather the outputs; the result must equal the unsharded run."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dartkv_b200.sharding import gather_outputs, shard_rows
from dartkv_b200.synthetic import make_kvq
from oracle import dartkv_oracle as orc

CFG = dict(bits=2, page_size=8, key_group_size=8, value_group_size=8, sink_tokens=2, hold_partial_pages=True,
           promote_ratio=0.25, metadata_dtype="f32")


def _attention(keys, values, query):
    cache = orc.OracleCache(orc.CacheConfig(**CFG), "f32")
    cache.append(keys, values)
    return orc.streamed_attention(query, cache, "f32")


def _worker(rank, world, port, result_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    keys, values, query = (t.numpy() for t in make_kvq(5, 4, 2, 29, 16, query_heads=4, dtype=torch.float32))
    lo, hi = shard_rows(4, world, rank)
    local = torch.from_numpy(_attention(keys[lo:hi], values[lo:hi], query[lo:hi]))
    full = gather_outputs(local)
    if rank == 0:
        np.save(result_path, full.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_batch_sharding_matches_single_rank(tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    result = str(tmp_path / "gathered.npy")
    mp.spawn(_worker, args=(2, port, result), nprocs=2, join=True)
    keys, values, query = (t.numpy() for t in make_kvq(5, 4, 2, 29, 16, query_heads=4, dtype=torch.float32))
    np.testing.assert_array_equal(np.load(result), _attention(keys, values, query))


def test_shard_rows_validation():
    assert shard_rows(128, 8, 3) == (48, 64)
    assert [shard_rows(4, 2, r) for r in range(2)] == [(0, 2), (2, 4)]
    with pytest.raises(ValueError, match="evenly"):
        shard_rows(10, 4, 0)
    with pytest.raises(ValueError, match="rank"):
        shard_rows(8, 2, 2)
    t = torch.ones(2, 3)
    assert gather_outputs(t) is t   # no process group: identity
