"""Streaming rollout generator with the API of scripts/rl_stream.py (StreamGen, sync_weights_inplace), running on
the GPU-resident scheduler: slots are retired and refilled on the device after every decode step instead of by a host
loop every ``check_every`` steps.

Differences a caller can observe, all within the reference's contract (rl_stream.py:1-12): a finished row is retired
at the step it finishes (no tokens are decoded past EOS), a request's cache starts at position 0 (no left padding;
prompts enter through packed prefill passes at every chunk, or through the decode step), and the sampler draws by
inverse CDF from Philox keyed by the request (a different random stream from Gumbel-max, as the reference's own fused
sampler already is, fused_sample.py:13-15).
"""
from __future__ import annotations

import collections

import torch

from .fast_decode import _engine, refresh_weights
from .scheduler import GpuScheduler


@torch.no_grad()
def sync_weights_inplace(gen_m, raw) -> None:
    """Copy raw's parameters into gen_m and refresh the fused arena in place (rl_stream.py:23-36): every captured
    graph keeps reading the same addresses; rows in flight continue under the new weights."""
    for pg, pt in zip(gen_m.parameters(), raw.parameters()):
        pg.copy_(pt)
    refresh_weights(gen_m)
    torch.cuda.synchronize(gen_m.embed.weight.device)


@torch.no_grad()
def publish_weights(gen_m, raw, sync: bool = True) -> None:
    """In-place weight publication without the intermediate copy: the fused inference weights (wqkv * qkv_scale,
    wo * o_scale, [w_gate; w_up], w_down, tanh(xsa_alpha), the residual lambdas; Attention.fuse / MLP.fuse,
    ultraviolet/model.py:289-300, :384-386) are computed from the TRAINER's parameters `raw` and written straight
    into gen_m's arena.  gen_m's own parameter tensors are not touched (nothing on the decode path reads them), so
    the O(params) parameter copy of sync_weights_inplace (rl_stream.py:23-36) disappears; pointers, captured graphs
    and in-flight rows behave exactly as there.  Follow it with ``dist.broadcast_weights`` when only rank 0 holds
    the trainer."""
    _engine(gen_m).load_from(raw)
    if sync:
        torch.cuda.synchronize(_engine(gen_m).device)


class StreamGen:
    def __init__(self, model, slots, max_prompt, max_new, temperature, eos_id, check_every=16, compile=True,
                 use_graph=True, pad_id=0, dtype=torch.float16, bucket=1024, top_p: float = 1.0,
                 seed: int | None = None, queue_capacity: int = 8192, prefill_lanes: int | None = None,
                 packed_prefill: bool | None = None, overlap_harvest: bool = False, warm: bool = False):
        """seed: Philox key of this generator's draws (request n's stream is keyed by (seed, n)).  None (default)
        takes a fresh seed from torch's generator mixed with the distributed rank, as the reference's sampler draws
        from torch's global generator; pass an int for reproducible rollouts.

        overlap_harvest: chunk() launches its decode steps first and collects, while they run, what had finished
        before them (GpuScheduler.window) -- a finished rollout is returned one chunk later and the device never
        waits for the host.  warm: capture every step / admission graph now instead of at first use."""
        assert temperature > 0
        from .generate import fresh_seed
        seed = fresh_seed() if seed is None else int(seed)
        self.m, self.B, self.max_new, self.T, self.eos = model, slots, max_new, temperature, eos_id
        self.ce, self.pad, self.dtype, self.max_prompt = check_every, pad_id, dtype, max_prompt
        eng = _engine(model)
        self.dev = eng.device
        # How prompts enter the cache.  Default: packed prefill passes -- at every chunk() the slots that the last
        # harvest saw free are refilled by one packed batch through the prefill kernels (the device picks requests
        # and slots; unquantised keys in the prompt's own attention, as in the reference's refill).  packed_prefill
        # = False feeds prompts through the decode step instead, prefill_lanes > 0 several tokens per slot and step.
        if packed_prefill is None:
            packed_prefill = not prefill_lanes
        if packed_prefill:
            prefill_lanes = 0
        elif prefill_lanes is None:  # a quarter more batch rows for prompt tokens once the batch is large enough
            prefill_lanes = slots // 4 if slots >= 32 else 0
        from .generate import _new_state
        self.st = _new_state(model, GpuScheduler.state_rows(slots, prefill_lanes, packed_prefill),
                             max_prompt + max_new + check_every, eng, GpuScheduler.ring_extra(prefill_lanes))
        self.sched = GpuScheduler(eng, self.st, max_new=max_new, temperature=temperature, top_p=top_p, eos_id=eos_id,
                                  pad_id=pad_id, seed=seed, q_cap=queue_capacity, max_prompt=max_prompt,
                                  use_graph=use_graph, prefill_lanes=prefill_lanes, packed_prefill=packed_prefill)
        self.overlap = bool(overlap_harvest)
        if warm:
            self.sched.warm()
        self.queue = collections.deque()   # host-side FIFO of (prompt_ids, meta) not yet on the device
        self._version = 0
        self.n_decode_steps = 0
        self.n_tokens = 0
        self._on_device = 0

    # the caller reads and writes .version (rl_grpo.py:1106, :1172, :1309); the device copy tags admissions
    @property
    def version(self):
        return self._version

    @version.setter
    def version(self, v):
        self._version = int(v)
        self.sched.set_version(self._version)

    def add(self, prompt_ids, meta):
        assert len(prompt_ids) <= self.max_prompt, "prompt longer than max_prompt"
        self.queue.append((list(prompt_ids), meta))

    def n_active(self):
        return self.sched.n_active()

    def n_outstanding(self):
        return len(self.queue) + (self.sched.n_enqueued - self.sched.n_harvested)

    def _upload(self):
        """Move host-queued requests to the device queue (bounded so that at most 2 * slots wait on the device, which
        keeps drop_queued meaningful for everything behind them)."""
        # (overlapped harvest: the live count as of the last counter read, so that the steps in flight are not
        # waited for)
        active = self.sched.counters(cached=True)["active"] if self.overlap else self.sched.n_active()
        waiting = self.sched.n_enqueued - self.sched.n_harvested - active
        room = max(0, 2 * self.B - max(waiting, 0))
        n = min(room, len(self.queue))
        if n:
            items = [self.queue.popleft() for _ in range(n)]
            self.sched.enqueue([p for p, _ in items], metas=[m for _, m in items])

    def chunk(self):
        """Upload queued requests, run check_every decode steps on the device, return what finished:
        [(meta, tokens list (EOS-terminated if it stopped), behaviour logp float32 array, start_version)]."""
        self._upload()
        if self.sched.n_enqueued == self.sched.n_harvested:
            return []
        if self.overlap and self.sched._primed and self.sched.live_bound() == 0:
            out = self.sched.harvest()         # every request is known to have finished: nothing left to step
        elif self.overlap:
            out = self.sched.unpack(self.sched.window(self.ce))
            self.n_decode_steps += self.ce
        else:
            self.sched.run(self.ce)
            self.n_decode_steps += self.ce
            out = self.sched.harvest()
        self.n_tokens += sum(len(t) for _, t, _, _ in out)
        return out

    def drop_queued(self, pred):
        """Remove queued (not yet uploaded) requests whose meta satisfies pred; returns how many."""
        keep = [x for x in self.queue if not pred(x[1])]
        n = len(self.queue) - len(keep)
        self.queue = collections.deque(keep)
        return n
