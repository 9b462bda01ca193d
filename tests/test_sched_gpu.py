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

    def check_status(self, B=None):
        return {"attn_status": 0, "kv_oob": 0}


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


@pytest.mark.parametrize("B,L,chunk,ring", [(4, 6, 4, 64), (8, 5, 8, 16), (33, 40, 3, 10)])
def test_prefill_lanes_feed_every_prompt_once_and_change_no_output(B, L, chunk, ring):
    """Prefill lanes: extra batch rows carry further prompt tokens of slots that are still prefilling.  Checked on
    the scheduler alone with the fake sampler: (1) per request, the (position, token) pairs fed over all rows and
    steps are exactly its prompt followed by its generated tokens, every position once, each step's rows of one
    request at consecutive positions ending at the slot's own row; (2) no chunk crosses position ring - 1;
    (3) idle lanes sit on the spare cache row; (4) outputs equal the run without lanes; (5) prompts take fewer steps."""
    from ultraviolet_b200.scheduler import GpuScheduler
    r = np.random.default_rng(B + L)
    n = 5 * B
    prompts = [r.integers(1, 1000, r.integers(1, 30)).tolist() for _ in range(n)]
    limits = r.integers(1, 12, n).tolist()
    max_len, max_new = 48, 12

    def run(lanes):
        st = _FakeState(GpuScheduler.state_rows(B, lanes), max_len)
        st.k = [torch.empty(1, 1, ring, 1), torch.empty(1, 1, max_len, 1)]
        eng = _FakeEngine(B)
        sch = GpuScheduler(eng, st, max_new=max_new, temperature=1.0, eos_id=0, q_cap=4096, max_prompt=32,
                           use_graph=False, prefill_lanes=lanes, lane_chunk=chunk)
        sch.enqueue(prompts, limits=limits)
        sch._sched_step()
        sch._primed = True
        fed = {}       # request -> list of (pos, tok) in feeding order
        steps = 0
        while int(sch.ctl[2].item()) < n:
            req = sch.req.cpu().numpy()
            tok = sch.cur_tok.cpu().numpy()
            pos = (sch.pos_all if lanes else st.pos).cpu().numpy()
            rows = [(int(s), int(s)) for s in range(B) if req[s] >= 0]
            if lanes:
                rm = sch.row_map.cpu().numpy()
                assert (rm[:B] == np.arange(B)).all()
                for l in range(B, B + lanes):
                    if rm[l] == B:                                   # (3) parked on the spare row
                        assert pos[l] == 0 and tok[l] == 0
                    else:
                        assert req[rm[l]] >= 0
                        rows.append((l, int(rm[l])))
            by_slot = {}
            for row, s in rows:
                by_slot.setdefault(s, []).append((int(pos[row]), int(tok[row]), row))
            for s, lst in by_slot.items():
                lst.sort()
                ps = [p for p, _, _ in lst]
                assert ps == list(range(ps[0], ps[0] + len(ps)))      # consecutive positions
                assert lst[-1][2] == s and len(lst) <= chunk          # the slot's own row is the last one
                if len(lst) > 1:
                    assert ps[-1] <= ring - 1                         # (2)
                fed.setdefault(int(req[s]), []).extend((p, t) for p, t, _ in lst)
            gen = sch.gen.cpu().numpy()
            eng._s["tok"].copy_(torch.from_numpy(_fake_token(req.astype(np.int64), gen.astype(np.int64), 7)
                                                 .astype(np.int64)))
            eng._s["logp"].copy_(torch.from_numpy((-(req + 1) - gen / 100).astype(np.float32)))
            sch._sched_step()
            steps += 1
            assert steps < 5000
        res = {m: toks for m, toks, _, _ in sch.harvest()}
        assert sch.counters()["status"] == 0
        return res, fed, steps

    base, fed0, steps0 = run(0)
    got, fed1, steps1 = run(L)
    assert got == base and sorted(got) == list(range(n))              # (4)
    for i in range(n):                                                # (1)
        want = prompts[i] + got[i][:-1]   # the last generated token is never fed back
        for fed in (fed0, fed1):
            assert [p for p, _ in fed[i]] == list(range(len(want))), i
            assert [t for _, t in fed[i]] == want, i
    assert steps1 < steps0                                            # (5)


def test_harvest_packed_is_the_same_payload_on_the_device():
    """harvest_packed() hands the finished rollouts over as device tensors (flat tokens / log-probs + offsets);
    harvest() is its host view."""
    from ultraviolet_b200.scheduler import GpuScheduler
    r = np.random.default_rng(5)
    n, B = 30, 6
    prompts = [r.integers(1, 1000, r.integers(1, 6)).tolist() for _ in range(n)]
    limits = r.integers(1, 9, n).tolist()

    def drive(packed):
        st, eng = _FakeState(B, 24), _FakeEngine(B)
        sch = GpuScheduler(eng, st, max_new=9, temperature=1.0, eos_id=0, q_cap=64, max_prompt=8, use_graph=False)
        sch.enqueue(prompts, limits=limits)
        sch._sched_step()
        sch._primed = True
        out = []
        for _ in range(120):
            req, gen = sch.req.cpu().numpy(), sch.gen.cpu().numpy()
            eng._s["tok"].copy_(torch.from_numpy(_fake_token(req.astype(np.int64), gen.astype(np.int64), 6)
                                                 .astype(np.int64)))
            eng._s["logp"].copy_(torch.from_numpy((-(req + 1) - gen / 100).astype(np.float32)))
            sch._sched_step()
            if packed:
                p = sch.harvest_packed()
                if p is not None:
                    assert p["tokens"].is_cuda and p["logp"].is_cuda and p["offsets"].is_cuda
                    assert p["tokens"].dtype == torch.int32 and p["offsets"][0] == 0
                    assert int(p["offsets"][-1]) == p["tokens"].numel() == p["logp"].numel()
                    off = p["offsets"].cpu().numpy()
                    t, l = p["tokens"].cpu().numpy(), p["logp"].cpu().numpy()
                    out += [(m, t[off[i]:off[i + 1]].tolist(), l[off[i]:off[i + 1]].tolist(), int(p["versions"][i]))
                            for i, m in enumerate(p["metas"])]
            else:
                out += [(m, t, l.tolist(), v) for m, t, l, v in sch.harvest()]
        return out

    a, b = drive(False), drive(True)
    assert len(a) == n and a == b


@pytest.mark.parametrize("B,cap,busy", [(6, 256, (1, 4)), (40, 64, ()), (1500, 4096, tuple(range(0, 1500, 7)))])
def test_admission_pass_kernel_matches_host_model(B, cap, busy):
    """uv_sched_admit alone: queued requests take the free slots in order while their prompts fit the packed rows;
    packed rows, prefix sums, slot state and the queue head against a host model."""
    import ctypes as C
    from ultraviolet_b200 import _lib
    from ultraviolet_b200.kernels._util import stream_ptr
    from ultraviolet_b200.scheduler import GpuScheduler
    r = np.random.default_rng(B)
    n = B + 9
    prompts = [r.integers(1, 900, r.integers(1, 30)).tolist() for _ in range(n)]
    st, eng = _FakeState(B + 1, 64), _FakeEngine(B)
    sch = GpuScheduler(eng, st, max_new=8, temperature=1.0, eos_id=0, q_cap=max(4096, n), max_prompt=32,
                       use_graph=False, packed_prefill=True, prefill_cap=cap)
    sch.enqueue(prompts)
    for s_ in busy:
        sch.req[s_] = 10 ** 6 + s_          # slots that hold some other request
    p = _lib.SchedAdmitArgs()
    p.tok, p.pos, p.row, p.last_pos = (t.data_ptr() for t in (sch.pk_tok, sch.pk_pos, sch.pk_row, sch.pk_last))
    p.cu, p.tile_cu, p.cap = sch.pk_cu.data_ptr(), sch.pk_tile_cu.data_ptr(), cap
    _lib.check(_lib.lib().uv_sched_admit(C.byref(sch.args), C.byref(p), stream_ptr(torch.device(DEV))), "admit")
    torch.cuda.synchronize()
    # host model
    free = [s_ for s_ in range(B) if s_ not in busy]
    rows, k = 0, 0
    exp = dict(tok=[], pos=[], row=[], last=[], cu=[], tcu=[], slot={})
    tiles = 0
    for s_, pr in zip(free, prompts):
        w = len(pr) - 1
        if rows + w > cap:
            break
        exp["cu"].append(rows)
        exp["tcu"].append(tiles)
        exp["tok"] += pr[:-1]
        exp["pos"] += list(range(w))
        exp["row"] += [s_] * w
        exp["last"] += [w - 1] * w
        exp["slot"][s_] = (k, pr[-1], w)
        rows, tiles, k = rows + w, tiles + (w + 15) // 16, k + 1
    assert k > 0
    assert int(sch.ctl[0].item()) == k and int(sch.ctl[11].item()) == rows
    assert sch.pk_tok[:rows].tolist() == exp["tok"] and sch.pk_pos[:rows].tolist() == exp["pos"]
    assert sch.pk_row[:rows].tolist() == exp["row"] and sch.pk_last[:rows].tolist() == exp["last"]
    assert (sch.pk_row[rows:cap] == B).all() and (sch.pk_pos[rows:cap] == 0).all()
    assert sch.pk_cu[:k].tolist() == exp["cu"] and (sch.pk_cu[k:] == rows).all()
    assert sch.pk_tile_cu[:k].tolist() == exp["tcu"] and (sch.pk_tile_cu[k:] == tiles).all()
    req, cur, pos, fed = (t.cpu().numpy() for t in (sch.req, sch.cur_tok, st.pos, sch.fed))
    for s_ in range(B):
        if s_ in exp["slot"]:
            q, last_tok, w = exp["slot"][s_]
            assert req[s_] == q and cur[s_] == last_tok and pos[s_] == w and fed[s_] == w + 1
        elif s_ in busy:
            assert req[s_] == 10 ** 6 + s_
        else:
            assert req[s_] == -1


@pytest.mark.parametrize("B,n", [(6, 40), (64, 300), (1500, 4000)])
def test_compaction_keeps_live_slots_dense_and_changes_no_output(B, n):
    """Slot compaction of the packed-admission mode, on the scheduler alone with the fake sampler: after every step
    the live slots are batch rows [0, active) in their previous order, row_map stays a permutation of the cache rows
    and a request keeps one cache row for its whole life; per-request outputs equal the run without compaction; the
    host's bound on the live rows never undercounts."""
    from ultraviolet_b200.scheduler import GpuScheduler
    r = np.random.default_rng(B)
    prompts = [r.integers(1, 900, r.integers(1, 12)).tolist() for _ in range(n)]
    limits = r.integers(1, 14, n).tolist()

    class _Eng(_FakeEngine):
        def trunk(self, *a, **k):
            return None

    def drive(compact):
        st, eng = _FakeState(B + 1, 32), _Eng(B)
        sch = GpuScheduler(eng, st, max_new=14, temperature=1.0, eos_id=0, q_cap=max(4096, n), max_prompt=16,
                           use_graph=False, packed_prefill=True, prefill_cap=4096, compact=compact)
        assert sch.compact == compact
        sch.enqueue(prompts[:n // 2], limits=limits[:n // 2])
        sch.st.pos.zero_()
        sch.admit(drain=True)
        sch._primed = True
        out, row_of, step = {}, {}, 0
        while len(out) < n and step < 4000:
            if step == 7:
                sch.enqueue(prompts[n // 2:], limits=limits[n // 2:])
            req, gen = sch.req.cpu().numpy(), sch.gen.cpu().numpy()
            if compact:
                live = req >= 0
                k = int(live.sum())
                assert live[:k].all() and not live[k:].any(), step
                assert k <= sch.live_bound() <= B and sch.rows_needed() >= k
                rm = sch.row_map.cpu().numpy()
                assert sorted(rm.tolist()) == list(range(B))
                for s_ in range(k):
                    assert row_of.setdefault(int(req[s_]), int(rm[s_])) == int(rm[s_]), (step, s_)
                assert (np.diff(req[:k]) > 0).all()     # admission order = queue order, and moves keep the order
            eng._s["tok"].copy_(torch.from_numpy(_fake_token(req.astype(np.int64), gen.astype(np.int64), 7)
                                                 .astype(np.int64)))
            eng._s["logp"].copy_(torch.from_numpy((-(req + 1) - gen / 100).astype(np.float32)))
            sch._sched_step()
            step += 1
            if step % 3 == 0:
                for m, toks, lps, ver in sch.harvest():
                    out[m] = (toks, lps.tolist())
                sch.admit()
        return out, step

    (a, steps_a), (b, steps_b) = drive(False), drive(True)
    assert len(a) == n and len(b) == n
    assert a == b


@pytest.mark.parametrize("B,n", [(6, 60), (64, 400), (1500, 5000)])
def test_deferred_admission_beside_the_steps_changes_no_output(B, n):
    """Admission passes launched beside the steps (shadow state + uv_sched_commit), on the scheduler alone with the
    fake sampler: per-request outputs equal the run with ordinary passes; at every step a slot is either live (its
    step row is its cache row), or not (its step row is the spare row B, whether it is free or reserved by a pass
    in flight); no request sits in two slots; the compaction owed while a pass was in flight is made up after the
    commit (dense again once the queue has drained); every launched pass is committed."""
    from ultraviolet_b200.scheduler import GpuScheduler
    r = np.random.default_rng(B + 1)
    prompts = [r.integers(1, 900, r.integers(1, 12)).tolist() for _ in range(n)]
    limits = r.integers(1, 14, n).tolist()

    class _Eng(_FakeEngine):
        def trunk(self, *a, **k):
            return None

    def drive(overlap):
        st, eng = _FakeState(B + 1, 32), _Eng(B)
        sch = GpuScheduler(eng, st, max_new=14, temperature=1.0, eos_id=0, q_cap=max(8192, n), max_prompt=16,
                           use_graph=False, packed_prefill=True, prefill_cap=4096, overlap_admit=overlap)
        sch.enqueue(prompts, limits=limits)
        sch.st.pos.zero_()
        sch.admit(drain=True)
        sch._primed = True
        out, step = {}, 0
        while len(out) < n and step < 6000:
            # one "window" of 3 steps, as window() runs it
            full = sch._commit_pending()
            sch._read_ctl()
            full = sch._admit_beside() or full
            rows = B if full else sch.rows_needed()
            for _ in range(3):
                torch.cuda.synchronize()
                req, gen = sch.req.cpu().numpy(), sch.gen.cpu().numpy()
                pend = sch.pend_req.cpu().numpy()
                rm, sr = sch.row_map.cpu().numpy(), sch.step_row.cpu().numpy()
                live = req >= 0
                assert sorted(rm.tolist()) == list(range(B))
                assert (sr[live] == rm[live]).all() and (sr[~live] == B).all(), step
                assert not (live & (pend >= 0)).any()
                both = np.concatenate([req[live], pend[pend >= 0]])
                assert len(set(both.tolist())) == both.size
                assert not live[rows:].any(), (step, rows)          # everything live is inside the stepped rows
                eng._s["tok"].copy_(torch.from_numpy(_fake_token(req.astype(np.int64), gen.astype(np.int64), 7)
                                                     .astype(np.int64)))
                eng._s["logp"].copy_(torch.from_numpy((-(req + 1) - gen / 100).astype(np.float32)))
                sch._sched_step()
                step += 1
            for m, toks, lps, ver in sch.harvest():
                out[m] = (toks, lps.tolist())
        assert not sch._admit_pending and int(sch.ctl[13].item()) == 0
        return out, sch.n_deferred_passes, sch.n_admit_passes

    (a, da, pa), (b, db, pb) = drive(False), drive(True)
    assert len(a) == n and len(b) == n and a == b
    assert da == 0 and db > 0
