"""Host-side partitioner, incl. a world_size-2 gloo run that gathers shards back (the only
collective the multi-GPU path uses, and only for validation)."""

import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from generative_recommenders_b200 import sharding, workloads as W
from oracle import hstu_oracle as O


def test_partition_is_balanced_and_complete():
    w = W.config4(256)
    for ws in (1, 2, 4, 8):
        bins = sharding.partition_by_tokens(w.lengths.tolist(), ws)
        assert sorted(i for b in bins for i in b) == list(range(256))
        loads = [int(w.lengths[b].sum()) for b in bins]
        assert max(loads) - min(loads) <= int(w.lengths.max())
    fb = sharding.partition_by_tokens(w.lengths.tolist(), 4, cost_quadratic=1e-3)
    assert sorted(i for b in fb for i in b) == list(range(256))


def test_shard_unshard_roundtrip():
    g = torch.Generator().manual_seed(0)
    lengths = torch.randint(0, 9, (11,), generator=g)
    offs = W._offsets(lengths)
    x = torch.randn(int(offs[-1]), 3, generator=g)
    bins = sharding.partition_by_tokens(lengths.tolist(), 3)
    parts = [sharding.shard_jagged(x, offs, b)[0] for b in bins]
    assert torch.equal(sharding.unshard_jagged(parts, offs, bins), x)


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(7)
    lengths = torch.randint(1, 40, (9,), generator=g)
    offs = W._offsets(lengths)
    L = int(offs[-1])
    qkv = [torch.randn(L, 2, 8, generator=g) for _ in range(3)]
    bins = sharding.partition_by_tokens(lengths.tolist(), world)
    mine = [sharding.shard_jagged(t, offs, bins[rank]) for t in qkv]
    # each rank computes its own sequences with the oracle standing in for the kernels
    out = O.hstu_mha(40, 0.3, mine[0][0], mine[1][0], mine[2][0], mine[0][1])
    gathered = [None] * world
    dist.all_gather_object(gathered, out)
    full = sharding.unshard_jagged(gathered, offs, bins)
    ref = O.hstu_mha(40, 0.3, qkv[0], qkv[1], qkv[2], offs)
    q.put((rank, float((full - ref).abs().max())))
    dist.destroy_process_group()


def test_two_rank_gloo_gather_matches_single_rank():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    assert all(err < 1e-6 for _, err in res), res
