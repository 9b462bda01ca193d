"""Multi-GPU plumbing of the rollout path: one full replica per GPU, the request stream sharded across ranks, and
the only two collectives the path has (ultraviolet scripts/rl_grpo.py:1305-1307 and :1458-1464 in the reference):

* ``broadcast_weights``: the fused weight arena of rank 0 lands IN PLACE in every rank's arena (one flat bf16
  buffer + the small fp32 side arena), so captured graphs keep their pointers and no re-fuse step follows;
* ``gather_rollouts``: finished rollouts (ragged token rows) to rank 0: lengths first, then one padded gather.

``shard_requests`` is the partition rule of UniformSampler(shard=(r, W)) (scripts/rl_sampler.py:16-38): rank r takes
positions r, r+W, ... of the shared request stream.  Works on any backend (NCCL on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

import time

import torch
import torch.distributed as dist


def world() -> tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


def shard_requests(n: int, rank: int, world_size: int) -> list[int]:
    """Indices of the shared request stream owned by `rank`: rank, rank + W, rank + 2W, ..."""
    return list(range(rank, n, world_size))


def warmup(device) -> None:
    """Create the communicator and its channels before anything is timed (the first collective of a process pays
    for NCCL initialisation)."""
    rank, W = world()
    if W == 1:
        return
    t = torch.ones(1024, device=device)
    dist.all_reduce(t)
    dist.broadcast(t, 0)
    out = [torch.empty_like(t) for _ in range(W)] if rank == 0 else None
    dist.gather(t, out, dst=0)
    lst = [torch.empty_like(t) for _ in range(W)]
    dist.all_gather(lst, t)
    # a rollout-sized gather too: the first large message sets up the transport's big-buffer protocol (tens of
    # milliseconds once), which would otherwise be charged to the first real rollout gather
    big = torch.zeros(1 << 21, dtype=torch.int32, device=device)
    out = [torch.empty_like(big) for _ in range(W)] if rank == 0 else None
    dist.gather(big, out, dst=0)
    _sync(t)


def _sync(t: torch.Tensor) -> None:
    if t.is_cuda:
        torch.cuda.synchronize(t.device)


def broadcast_flat(tensors, src: int = 0) -> float:
    """Broadcast each flat tensor in place from `src`; returns seconds (host clock around a device sync)."""
    for t in tensors:
        _sync(t)
    t0 = time.perf_counter()
    for t in tensors:
        dist.broadcast(t, src)
    for t in tensors:
        _sync(t)
    return time.perf_counter() - t0


def broadcast_weights(engine, src: int = 0) -> float:
    """Per-RL-step policy-weight broadcast: rank `src`'s arena into every rank's arena, in place."""
    dt = broadcast_flat([engine.arena, engine.arena32], src)
    engine.version += 1
    return dt


def gather_rollouts(tokens: torch.Tensor, lengths: torch.Tensor | None = None, dst: int = 0):
    """tokens (n, L) int64 rows of this rank (row i valid up to lengths[i], default L).  Returns
    (list over ranks of (n_r, L_max) tensors + lengths on `dst`, else None; seconds)."""
    rank, W = world()
    n, L = tokens.shape
    if lengths is None:
        lengths = torch.full((n,), L, dtype=torch.int64, device=tokens.device)
    _sync(tokens)
    t0 = time.perf_counter()
    shape = torch.tensor([n, L], dtype=torch.int64, device=tokens.device)
    shapes = [torch.zeros_like(shape) for _ in range(W)]
    dist.all_gather(shapes, shape)
    n_max = int(max(s[0].item() for s in shapes))
    l_max = int(max(s[1].item() for s in shapes))
    pad = torch.zeros(n_max, l_max + 1, dtype=torch.int64, device=tokens.device)
    pad[:n, :L] = tokens
    pad[:n, l_max] = lengths
    out = [torch.empty_like(pad) for _ in range(W)] if rank == dst else None
    dist.gather(pad, out, dst=dst)
    _sync(tokens)
    dt = time.perf_counter() - t0
    if rank != dst:
        return None, dt
    res = []
    for r, s in enumerate(shapes):
        k = int(s[0].item())
        res.append((out[r][:k, :l_max], out[r][:k, l_max]))
    return res, dt


def gather_packed(tokens: torch.Tensor, logp: torch.Tensor, lengths: torch.Tensor, versions: torch.Tensor,
                  ids: torch.Tensor, dst: int = 0):
    """Finished rollouts of this rank, as GpuScheduler.harvest_packed() hands them over, to rank `dst`: flat int32
    tokens and fp32 behaviour log-probs (sum(lengths),), and per rollout its length, the weight version it started
    under and its request id (int32) -- the record the reference gathers with all_gather_object (scripts/rl_grpo.py:
    1458-1464), as three sized buffers instead of pickled Python objects.  Counts travel first (one all_gather of
    two integers), then each buffer is gathered padded to the largest rank's size.  Returns (list over ranks of
    (tokens, logp, lengths, versions, ids) on `dst`, else None; seconds)."""
    rank, W = world()
    dev = tokens.device
    _sync(tokens)
    t0 = time.perf_counter()
    if W == 1:
        return [(tokens, logp, lengths, versions, ids)], 0.0
    size = torch.tensor([tokens.numel(), lengths.numel()], dtype=torch.int64, device=dev)
    sizes = [torch.zeros_like(size) for _ in range(W)]
    dist.all_gather(sizes, size)
    sizes_h = torch.stack(sizes).cpu()
    t_max, n_max = int(sizes_h[:, 0].max()), int(sizes_h[:, 1].max())

    def padded(x, n, dtype):
        out = torch.zeros(n, dtype=dtype, device=dev)
        out[:x.numel()] = x.to(dtype)
        return out
    tok_p, lp_p = padded(tokens, t_max, torch.int32), padded(logp, t_max, torch.float32)
    meta_p = torch.stack([padded(lengths, n_max, torch.int32), padded(versions, n_max, torch.int32),
                          padded(ids, n_max, torch.int32)])
    outs = []
    for buf in (tok_p, lp_p, meta_p):
        dest = [torch.empty_like(buf) for _ in range(W)] if rank == dst else None
        dist.gather(buf, dest, dst=dst)
        outs.append(dest)
    _sync(tokens)
    dt = time.perf_counter() - t0
    if rank != dst:
        return None, dt
    res = []
    for r in range(W):
        nt, nr = int(sizes_h[r, 0]), int(sizes_h[r, 1])
        res.append((outs[0][r][:nt], outs[1][r][:nt], outs[2][r][0, :nr], outs[2][r][1, :nr], outs[2][r][2, :nr]))
    return res, dt
