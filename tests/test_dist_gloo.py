"""CPU, two processes over gloo: the data-parallel host logic (batch sharding and the single-bucket
gradient all-reduce) that bench.py uses between GPUs."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    from mappedconvolutions_b200.dist import allreduce_gradients, shard_batch
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # every rank computes "gradients" of its own batch shard; the reduced result must equal
        # the gradient of the whole batch
        g = torch.Generator().manual_seed(0)
        per_sample_w = torch.randn(8, 4, 3, 5, generator=g)
        per_sample_b = torch.randn(8, 4, generator=g)
        lo, hi = shard_batch(8, rank, world)
        gw = per_sample_w[lo:hi].sum(0).to(torch.bfloat16)
        gb = per_sample_b[lo:hi].sum(0)
        bucket = allreduce_gradients([gw, None, gb])
        assert bucket.dtype == torch.float32 and bucket.numel() == gw.numel() + gb.numel()
        ok_w = torch.allclose(gw.float(), per_sample_w.sum(0), atol=0.1)
        ok_b = torch.allclose(gb, per_sample_b.sum(0), atol=1e-5)
        out.put((rank, bool(ok_w and ok_b), (lo, hi)))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_bucket_allreduce_world_size_2():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29500 + os.getpid() % 500
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(out.get(timeout=100) for _ in procs)
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    assert [r[1] for r in res] == [True, True]
    assert [r[2] for r in res] == [(0, 4), (4, 8)]


def test_shard_batch_is_a_partition():
    from mappedconvolutions_b200.dist import shard_batch
    for batch in (1, 7, 8, 64):
        for world in (1, 2, 3, 8):
            parts = [shard_batch(batch, r, world) for r in range(world)]
            assert parts[0][0] == 0 and parts[-1][1] == batch
            assert all(parts[i][1] == parts[i + 1][0] for i in range(world - 1))
            sizes = [b - a for a, b in parts]
            assert max(sizes) - min(sizes) <= 1
