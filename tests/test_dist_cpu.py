"""The multi-rank host logic on two gloo ranks (CPU): request sharding, in-place weight broadcast, ragged rollout
gather."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from ultraviolet_b200 import dist as uvdist
    try:
        assert uvdist.world() == (rank, world)
        # weight arena: rank 0's values land in place on every rank
        arena = torch.full((1000,), float(rank + 1), dtype=torch.bfloat16)
        side = torch.arange(10, dtype=torch.float32) * (rank + 1)
        ptr = arena.data_ptr()
        uvdist.broadcast_flat([arena, side], 0)
        assert arena.data_ptr() == ptr and bool((arena == 1).all()) and bool((side == torch.arange(10)).all())
        # ragged rollouts: rank r has r + 2 rows of width 5 + r
        n, L = rank + 2, 5 + rank
        toks = torch.arange(n * L).view(n, L) + 1000 * rank
        lens = torch.arange(1, n + 1)
        res, _ = uvdist.gather_rollouts(toks, lens, dst=0)
        if rank == 0:
            assert len(res) == world
            for r, (t, l) in enumerate(res):
                nr, Lr = r + 2, 5 + r
                assert t.shape[0] == nr and torch.equal(t[:, :Lr], torch.arange(nr * Lr).view(nr, Lr) + 1000 * r)
                assert torch.equal(l, torch.arange(1, nr + 1))
        else:
            assert res is None
        # packed rollouts (tokens + log-probs + lengths + versions + ids), ragged per rank
        lens = torch.tensor([3, 1 + rank], dtype=torch.int32)
        nt = int(lens.sum())
        toks = (torch.arange(nt) + 100 * rank).to(torch.int32)
        lps = -(torch.arange(nt).float() + rank)
        vers = torch.tensor([rank, rank + 5], dtype=torch.int32)
        ids = torch.tensor([10 * rank, 10 * rank + 1], dtype=torch.int32)
        res, _ = uvdist.gather_packed(toks, lps, lens, vers, ids, dst=0)
        if rank == 0:
            assert len(res) == world
            for r, (t, l, n_, v, i) in enumerate(res):
                k = 3 + 1 + r
                assert t.dtype == torch.int32 and l.dtype == torch.float32
                assert torch.equal(t, (torch.arange(k) + 100 * r).to(torch.int32))
                assert torch.equal(l, -(torch.arange(k).float() + r))
                assert n_.tolist() == [3, 1 + r] and v.tolist() == [r, r + 5] and i.tolist() == [10 * r, 10 * r + 1]
        else:
            assert res is None
        q.put((rank, uvdist.shard_requests(11, rank, world)))
    finally:
        dist.destroy_process_group()


def test_two_rank_broadcast_gather_and_sharding():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in ps:
        p.start()
    shards = dict(q.get(timeout=120) for _ in range(world))
    for p in ps:
        p.join(timeout=120)
        assert p.exitcode == 0
    # the ranks together cover the request stream exactly once (tests/test_rl_sampler.py:68-76 in the reference)
    assert sorted(shards[0] + shards[1]) == list(range(11)) and shards[0] == [0, 2, 4, 6, 8, 10]
