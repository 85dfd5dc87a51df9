"""Two ranks on two GPUs of one node: the decode kernels deliver their output rows straight into every rank's
gathered tensor (peer stores + arrival flags); the result must equal an NCCL all-gather of the same outputs and the
unsharded decode.  Skipped on machines with fewer than two GPUs."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, batch, ctx, result_path):
    import datetime

    import dartkv_b200 as dart
    from dartkv_b200.sharding import PeerGather, gather_outputs, shard_plan
    from dartkv_b200.synthetic import HEADLINE_GEOMETRY as G, build_headline_cache

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    device = torch.device("cuda", rank)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device,
                            timeout=datetime.timedelta(seconds=120))
    shard = shard_plan(batch, G["kv_heads"], world, rank)
    cache, query = build_headline_cache(range(shard.row_begin, shard.row_end), ctx, 11, device,
                                        heads=(shard.head_begin, shard.head_end))
    q3 = query[:, :, 0].contiguous()
    peer = PeerGather(shard, batch, G["query_heads"], G["kv_heads"], G["head_dim"], torch.bfloat16, device)
    ok = True
    for step in range(6):
        q = (q3.float() * (1.0 + 0.25 * step)).to(torch.bfloat16)   # a different result every step
        full = dart.decode_attention(q, cache, peer_gather=peer).clone()
        local = dart.decode_attention(q, cache)
        want = gather_outputs(local, shard=shard, batch=batch, kv_heads=G["kv_heads"])
        ok = ok and bool(torch.equal(full, want))
    status = cache.decode_status()
    flags = torch.tensor([int(ok), int(status == 0)], dtype=torch.int32, device=device)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    if rank == 0:
        # the same rows decoded by one rank alone (a different split of the work: one output ulp is allowed)
        whole, wq = build_headline_cache(range(batch), ctx, 11, device)
        q = (wq[:, :, 0].float() * (1.0 + 0.25 * 5)).to(torch.bfloat16)
        single = dart.decode_attention(q, whole).float()
        diff = (full.float() - single).abs()
        close = bool(((diff <= 2e-3) | (diff <= single.abs() * 2.0 ** -7)).all())
        torch.save({"equal_nccl": bool(flags[0].item()), "status_ok": bool(flags[1].item()), "close": close}, result_path)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("batch", [4, 3, 1], ids=["even", "ragged", "kv_heads"])
def test_peer_store_gather_equals_nccl_gather_and_unsharded_decode(tmp_path, batch):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    result = str(tmp_path / "result.pt")
    mp.spawn(_worker, args=(2, port, batch, 32 + 9 * 128 + 50, result), nprocs=2, join=True)
    got = torch.load(result)
    assert got == {"equal_nccl": True, "status_ok": True, "close": True}, got
