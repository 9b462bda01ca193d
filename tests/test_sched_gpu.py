"""The scheduler kernels alone (no model): driven by a deterministic fake sampler and compared, field by field, with
a host simulation of the same rules.  Integer work: everything must match exactly."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


class _FakeState:
    def __init__(self, B, max_len):
        self.B, self.max_len = B, max_len
        self.pos = torch.zeros(B, dtype=torch.long, device=DEV)
        self.starts = torch.zeros(B, dtype=torch.long, device=DEV)


class _FakeEngine:
    device = torch.device(DEV)

    def __init__(self, B):
        self._s = dict(tok=torch.zeros(B, dtype=torch.long, device=DEV),
                       logp=torch.zeros(B, dtype=torch.float32, device=DEV))

    def scratch(self, B):
        return self._s


def _fake_token(req, gen, eos_every):
    t = (req * 7919 + gen * 104729) % 1000 + 1
    return np.where((eos_every > 0) & ((req + gen) % np.maximum(eos_every, 1) == eos_every - 1), 0, t)


def _simulate(prompts, limits, B, n_steps, eos, max_len, eos_every, force_eos):
    """Host restatement of sched_step: returns per-request outputs, finishing order and per-step slot state."""
    n = len(prompts)
    req = [-1] * B
    fed, gen, pos, cur = [0] * B, [0] * B, [0] * B, [0] * B
    head, outs, fin, trace = 0, {}, [], []

    def admit(free):
        nonlocal head
        for s in free:
            if head < n:
                req[s], fed[s], gen[s], pos[s], cur[s] = head, 1, 0, 0, prompts[head][0]
                outs[head] = []
                head += 1
            else:
                req[s], pos[s], cur[s] = -1, 0, 0
    admit(list(range(B)))
    for _ in range(n_steps):
        trace.append((list(req), list(cur), list(pos)))
        free = []
        for s in range(B):
            r = req[s]
            if r < 0:
                free.append(s)
                continue
            if fed[s] < len(prompts[r]):
                cur[s] = prompts[r][fed[s]]
                fed[s] += 1
                pos[s] += 1
                continue
            t = int(_fake_token(np.int64(r), np.int64(gen[s]), eos_every))
            if force_eos and gen[s] + 1 >= limits[r]:
                t = eos
            outs[r].append(t)
            gen[s] += 1
            if (eos >= 0 and t == eos) or gen[s] >= limits[r] or pos[s] + 1 >= max_len:
                fin.append(r)
                req[s] = -1
                free.append(s)
            else:
                cur[s] = t
                pos[s] += 1
        admit(free)
    return outs, fin, trace


@pytest.mark.parametrize("B,n,eos_every,force_eos", [(4, 11, 0, False), (8, 40, 5, False), (33, 200, 9, True),
                                                     (1100, 2500, 0, False)])
def test_scheduler_matches_host_simulation(B, n, eos_every, force_eos):
    from ultraviolet_b200.scheduler import GpuScheduler
    r = np.random.default_rng(B)
    prompts = [r.integers(1, 1000, r.integers(1, 9)).tolist() for _ in range(n)]
    limits = r.integers(1, 12, n).tolist()
    max_len, max_new, steps = 24, 12, 160 if B < 1000 else 60
    st, eng = _FakeState(B, max_len), _FakeEngine(B)
    sch = GpuScheduler(eng, st, max_new=max_new, temperature=1.0, eos_id=0, q_cap=max(4096, n), max_prompt=8,
                       force_eos=force_eos, use_graph=False)
    half = n // 2
    sch.enqueue(prompts[:half], limits=limits[:half])
    sch._sched_step()                       # priming pass admits the first requests
    sch._primed = True
    sch.enqueue(prompts[half:], limits=limits[half:])   # more arrive while slots are busy
    outs, fin, trace = _simulate(prompts, limits, B, steps, 0, max_len, eos_every, force_eos)
    if n > B:  # the second enqueue landed before any slot freed up, as in the simulation's single queue
        pass
    got_trace = []
    for k in range(steps):
        req = sch.req.cpu().numpy()
        got_trace.append((req.tolist(), sch.cur_tok.cpu().numpy().tolist(), st.pos.cpu().numpy().tolist()))
        gen = sch.gen.cpu().numpy()
        eng._s["tok"].copy_(torch.from_numpy(_fake_token(req.astype(np.int64), gen.astype(np.int64), eos_every)
                                             .astype(np.int64)))
        eng._s["logp"].copy_(torch.from_numpy((-(req + 1) - gen / 100).astype(np.float32)))
        sch._sched_step()
    if n <= B or half >= B:   # admission order equals the single-queue simulation
        for k in range(steps):
            assert got_trace[k] == (trace[k][0], trace[k][1], trace[k][2]), k
    res = sch.harvest()
    assert [m for m, _, _, _ in res] == fin[:len(res)] and len(res) == len(fin)
    for m, toks, lps, ver in res:
        assert toks == outs[m]
        np.testing.assert_allclose(lps, -(m + 1) - np.arange(len(toks)) / 100, rtol=1e-6)
        assert ver == 0
    c = sch.counters()
    assert c["finished"] == len(fin) and c["tail"] == n and c["status"] == 0
    assert c["active"] == sum(x >= 0 for x in sch.req.cpu().numpy())
