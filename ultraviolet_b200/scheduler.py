"""Host side of the GPU-resident continuous-batching scheduler (csrc/sched.cu).

``GpuScheduler`` owns the device queue (request / prompt-token / output rings), the per-slot state that doubles as the
decode step's inputs (``cur_tok``, and the cache state's ``pos`` / ``starts``), and one CUDA graph holding a whole
step:  trunk -> LM head -> uv_sample (Philox keyed per request) -> uv_sched_step.  ``run(n)`` replays the graph n
times with no host work in between; ``enqueue`` and ``harvest`` are the only host <-> device traffic.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import _lib
from .kernels._util import stream_ptr

(CTL_HEAD, CTL_TAIL, CTL_FIN, CTL_VERSION, CTL_ACTIVE, CTL_STATUS, CTL_STEPS, CTL_TOK_TAIL, CTL_OUT_TAIL,
 CTL_GENERATED, CTL_SLOT_STEPS, CTL_PREFILL_ROWS, CTL_ADMIT_PASSES, CTL_INFLIGHT, CTL_DEFER, CTL_DIRTY) = range(16)


def _pow2(n: int) -> int:
    return 1 << max(1, (n - 1).bit_length())


def _pass_caps(limit: int) -> list[int]:
    """Packed-row capacities an admission pass may be captured at: 256, then four steps per octave (1.25 x, 1.5 x,
    1.75 x, 2 x of each power of two, all multiples of 64) up to `limit` -- a pass is padded by a fifth at most
    instead of up to a factor of two."""
    caps, p = [256], 256
    while p < limit:
        for f in (5, 6, 7, 8):
            c = p * f // 4
            if c <= limit:
                caps.append(c)
        p *= 2
    return caps


class GpuScheduler:
    def __init__(self, engine, st, *, max_new: int, temperature: float, top_p: float = 1.0, eos_id: int | None = 0,
                 pad_id: int = 0, seed: int = 0, q_cap: int = 8192, tok_cap: int | None = None,
                 out_cap: int | None = None, max_prompt: int = 256, force_eos: bool = False, use_graph: bool = True,
                 num_splits: dict | None = None, prefill_lanes: int = 0, lane_chunk: int = 8, top_k: int = 0,
                 packed_prefill: bool = False, prefill_cap: int = 16384, compact: bool = True,
                 overlap_admit: bool = False):
        """prefill_lanes > 0: the decode step runs on slots + prefill_lanes batch rows; the extra rows carry further
        prompt tokens of slots that are still prefilling (up to lane_chunk tokens per slot per step).  The state must
        then hold one spare cache row: st.B == slots + 1 (see ``state_rows``).

        packed_prefill: the step only retires; queued requests are admitted by ADMISSION PASSES that ``run`` launches
        before its steps -- uv_sched_admit picks the requests and slots on the device and lays their prompts out as
        one packed batch, which goes through the prefill path (packed varlen attention over unquantised keys, int8
        cache written on the way) in a single pass of up to prefill_cap rows.  The host only chooses how many packed
        rows the pass gets, from the queue's prompt lengths and the head / finished counters it read at the last
        harvest.  Needs the spare cache row too; excludes prefill_lanes.

        overlap_admit (packed_prefill only; takes effect in ``window``): an admission pass that refills the free
        slots in one go is launched on a second stream and runs BESIDE the window's decode steps; its requests
        wait in a shadow state and go live (uv_sched_commit) at the start of the next window.  A slot then idles
        one window longer, but the device never stops stepping for a prefill.

        compact (packed_prefill only, up to 4096 slots): the step kernel keeps the live slots in batch rows
        [0, active) (a slot's cache row follows it through ``row_map``), and ``run`` replays a step graph over the
        smallest power-of-two fraction of the slots that still covers them -- when the queue has run dry, the tail
        of a job steps 256, 128, ... rows instead of every slot."""
        self.eng, self.st = engine, st
        self.L = int(prefill_lanes)
        self.packed = bool(packed_prefill)
        if self.packed and self.L:
            raise ValueError("packed_prefill and prefill_lanes are two ways to prefill: choose one")
        self.B = st.B - 1 if (self.L > 0 or self.packed) else st.B
        self.dev = engine.device
        self.max_new, self.T, self.top_p, self.seed = int(max_new), float(temperature), float(top_p), int(seed)
        self.top_k = int(top_k or 0)
        self.eos = -1 if eos_id is None else int(eos_id)
        self.pad, self.force_eos = int(pad_id), bool(force_eos)
        self.q_cap = _pow2(q_cap)
        self.tok_cap = int(tok_cap or self.q_cap * max_prompt)
        self.out_cap = int(out_cap or self.q_cap * self.max_new)
        self.use_graph, self.num_splits = use_graph, num_splits
        dev, B, Q = self.dev, self.B, self.q_cap
        i32 = lambda n, v=0: torch.full((n,), v, dtype=torch.int32, device=dev)
        i64 = lambda n, v=0: torch.full((n,), v, dtype=torch.int64, device=dev)
        self.req, self.fed, self.gen = i32(B, -1), i32(B), i32(B)
        self.cur_tok, self.row_key, self.step_ctr = i64(B + self.L, self.pad), i64(B), i64(B)
        if self.L > 0:
            # batch rows = slots then lanes; the slots' pos / starts stay visible as the state's own (first B rows
            # of the cache; row B is the spare row idle lanes are parked on)
            self.pos_all, self.starts_all = i64(B + self.L), i64(B + self.L)
            self.row_map = torch.cat([torch.arange(B, dtype=torch.int64, device=dev), i64(self.L, B)])
            st.pos, st.starts = self.pos_all[:B], self.starts_all[:B]
        if self.packed:
            st.pos, st.starts = i64(B), i64(B)      # the decode step runs on the B slots (cache rows 0 .. B - 1)
            self.prefill_cap = max(256, _pow2(int(prefill_cap)))
            self.pass_caps = _pass_caps(self.prefill_cap)
            cap = self.prefill_cap
            self.pk_tok, self.pk_pos, self.pk_row, self.pk_last = i64(cap), i64(cap), i64(cap, B), i64(cap)
            self.pk_zero = i64(cap)
            self.pk_cu, self.pk_tile_cu = i32(B + 1), i32(B + 1)
            self._plen: dict[int, int] = {}          # request -> prompt length (host copy of the queue)
            self._ctl_fresh = True
            self._admit_graphs: dict[int, torch.cuda.CUDAGraph] = {}
            self.n_admit_passes = 0
            self.row_map = torch.arange(B, dtype=torch.int64, device=dev)   # batch row -> cache row
            # what the decode step uses as cache row: row_map while a slot is live, the spare row B while it is not
            self.step_row = i64(B, B)
            self.pend_req, self.pend_fed = i32(B, -1), i32(B)
            self.pend_tok, self.pend_pos, self.pend_key = i64(B), i64(B), i64(B)
            self._flag_on = torch.ones(2, dtype=torch.int64, device=dev)   # ctl[INFLIGHT], ctl[DEFER] = 1, 1
        self.overlap_admit = bool(overlap_admit) and self.packed
        self._admit_pending, self._admit_ev, self._admit_stream = False, None, None
        self.n_deferred_passes = 0
        self.compact = bool(compact) and self.packed and B <= 4096
        # batch rows a step may run on: all slots, or (compact) a halving ladder down to 32 rows
        self.buckets = sorted({B} | ({B >> k for k in range(1, 12) if (B >> k) >= 32} if self.compact else set()))
        self._head_h = self._fin_h = 0   # head / finished counters as last read from the device
        self._ctl_h = None               # the control words as last read (numpy)
        self._graphs: dict[int, torch.cuda.CUDAGraph] = {}
        self._side = None         # stream of window()'s overlapped harvest
        self.bucket_steps: dict[int, int] = {}   # steps run per batch-row count
        self.prompt_off, self.key, self.out_off = i64(Q), i64(Q), i64(Q)
        self.prompt_len, self.limit, self.out_len, self.start_version = i32(Q), i32(Q), i32(Q, -1), i32(Q)
        self.fin_ring = i32(Q, -1)
        self.tokens = i32(self.tok_cap)
        self.out_tok = i32(self.out_cap)
        self.out_lp = torch.zeros(self.out_cap, dtype=torch.float32, device=dev)
        self.ctl = i64(16)
        sc = engine.scratch(B)
        self.st_rows = B + self.L  # batch rows of one step = the engine scratch set the step's kernels flag into
        self.samp_tok, self.samp_lp = sc["tok"], sc["logp"]
        st.pos.zero_()
        st.starts.zero_()
        a = self.args = _lib.SchedArgs()
        if self.L > 0:
            a.row_map, a.lanes, a.lane_chunk = self.row_map.data_ptr(), self.L, int(lane_chunk)
            # A chunk of lane_chunk consecutive positions of one sequence must not overwrite a ring slot that a row
            # of the same step still reads.  Rings with at least window + lane_chunk - 1 slots (new_state(...,
            # ring_extra=lane_chunk)) can never do that; shorter ones only take chunks while the ring has not
            # wrapped yet (prompts up to the ring length).
            ring = min(int(k.size(2)) for k in st.k)
            window = int(getattr(getattr(st, "cfg", None), "window", 0) or 0)
            a.ring_len = (1 << 40) if window > 0 and ring >= window + int(lane_chunk) - 1 else ring
        for name in ("req", "fed", "gen", "cur_tok", "row_key", "step_ctr", "prompt_off", "prompt_len", "limit",
                     "key", "out_off", "out_len", "start_version", "tokens", "out_tok", "out_lp", "fin_ring", "ctl",
                     "samp_tok", "samp_lp"):
            setattr(a, name, getattr(self, name).data_ptr())
        a.pos, a.starts = st.pos.data_ptr(), st.starts.data_ptr()  # (with lanes: the first rows of pos_all / starts_all)
        a.B, a.q_cap, a.tok_cap, a.out_cap = B, Q, self.tok_cap, self.out_cap
        a.eos, a.pad, a.force_eos, a.max_len = self.eos, self.pad, int(self.force_eos), st.max_len
        a.no_admit = int(self.packed)
        if self.packed:
            a.row_map, a.compact = self.row_map.data_ptr(), int(self.compact)
            a.step_row = self.step_row.data_ptr()
            for name in ("pend_req", "pend_fed", "pend_tok", "pend_pos", "pend_key"):
                setattr(a, name, getattr(self, name).data_ptr())
        # host mirrors
        self.n_enqueued = 0       # == ctl[TAIL]
        self.n_harvested = 0      # finished requests already returned
        self.tok_tail = 0
        self.out_tail = 0
        # ring accounting: offsets of every unharvested request; the oldest one bounds what may be overwritten
        self._span: dict[int, tuple[int, int]] = {}   # request -> (prompt offset, output offset)
        self._oldest = 0
        self.meta: dict[int, object] = {}
        self.steps_run = 0
        self._primed = False

    @staticmethod
    def ring_extra(prefill_lanes: int = 0, lane_chunk: int = 8) -> int:
        """Extra local-ring slots a state should be created with (new_state(..., ring_extra=...)) so that prefill
        lanes keep working on prompts longer than the attention window."""
        return int(lane_chunk) if prefill_lanes > 0 else 0

    @staticmethod
    def state_rows(slots: int, prefill_lanes: int = 0, packed_prefill: bool = False) -> int:
        """Cache rows the decode state needs for `slots` sequences: one spare row when prefill lanes or packed
        admission passes are on (idle lanes / unused packed rows are parked there)."""
        return slots + (1 if (prefill_lanes > 0 or packed_prefill) else 0)

    # ------------------------------------------------------------------------------------------------ queue
    def set_version(self, v: int) -> None:
        self.ctl[CTL_VERSION] = int(v)

    def enqueue(self, prompts, limits=None, keys=None, metas=None) -> None:
        """Append requests: prompts (list of token-id lists), per-request token limits (default max_new), Philox
        keys (default: the request index) and opaque metadata returned by harvest()."""
        n = len(prompts)
        if n == 0:
            return
        lens = np.fromiter((len(p) for p in prompts), dtype=np.int64, count=n)
        if lens.min() < 1:
            raise ValueError("empty prompt")
        lim = np.full(n, self.max_new, np.int64) if limits is None else np.minimum(np.asarray(limits, np.int64),
                                                                                  self.max_new)
        if lim.min() < 1:
            raise ValueError("token limits must be >= 1")
        if int((lens + lim).max()) > self.st.max_len:
            raise ValueError("prompt + limit exceeds the cache length")
        if self.packed and int(lens.max()) - 1 > self.prefill_cap:
            raise ValueError(f"a prompt of {int(lens.max())} tokens does not fit one admission pass "
                             f"(prefill_cap = {self.prefill_cap} packed rows)")
        in_flight = self.n_enqueued - self.n_harvested
        if in_flight + n > self.q_cap:
            raise RuntimeError(f"request ring full ({in_flight} in flight + {n} new > {self.q_cap})")
        tok_floor, out_floor = self._span.get(self._oldest, (self.tok_tail, self.out_tail))
        if (self.tok_tail + int(lens.sum()) - tok_floor > self.tok_cap
                or self.out_tail + int(lim.sum()) - out_floor > self.out_cap):
            raise RuntimeError("prompt-token or output ring too small for the requests in flight")
        r0 = self.n_enqueued
        kk = np.arange(r0, r0 + n, dtype=np.int64) if keys is None else np.asarray(keys, np.int64)
        ridx = torch.from_numpy((np.arange(r0, r0 + n) % self.q_cap).astype(np.int64)).to(self.dev)
        self.prompt_len[ridx] = torch.from_numpy(lens.astype(np.int32)).to(self.dev)
        self.limit[ridx] = torch.from_numpy(lim.astype(np.int32)).to(self.dev)
        self.key[ridx] = torch.from_numpy(kk).to(self.dev)
        flat = np.fromiter((t for p in prompts for t in p), dtype=np.int32, count=int(lens.sum()))
        tidx = torch.from_numpy(((self.tok_tail + np.arange(flat.size)) % self.tok_cap).astype(np.int64)).to(self.dev)
        self.tokens[tidx] = torch.from_numpy(flat).to(self.dev)
        with torch.cuda.device(self.dev):
            _lib.check(_lib.lib().uv_sched_enqueue(C.byref(self.args), n, stream_ptr(self.dev)), "uv_sched_enqueue")
        t_off = self.tok_tail + np.concatenate([[0], np.cumsum(lens)[:-1]])
        o_off = self.out_tail + np.concatenate([[0], np.cumsum(lim)[:-1]])
        for i in range(n):
            self.meta[r0 + i] = metas[i] if metas is not None else r0 + i
            self._span[r0 + i] = (int(t_off[i]), int(o_off[i]))
            if self.packed:
                self._plen[r0 + i] = int(lens[i])
        self.n_enqueued += n
        self.tok_tail += int(lens.sum())
        self.out_tail += int(lim.sum())

    # ------------------------------------------------------------------------------------------------ stepping
    def _sched_step(self) -> None:
        with torch.cuda.device(self.dev):
            _lib.check(_lib.lib().uv_sched_step(C.byref(self.args), stream_ptr(self.dev)), "uv_sched_step")

    def _step_body(self, n: int | None = None) -> None:
        """One decode step on the first n batch rows (default: every slot) + the scheduler kernel over all slots."""
        eng, st = self.eng, self.st
        n = self.B if n is None else n
        if self.L > 0:
            h = eng.trunk(self.cur_tok, st, self.pos_all, self.starts_all, g_len=st.max_len,
                          num_splits=self.num_splits, row_map=self.row_map)[:self.B]  # only slots are sampled
        else:
            h = eng.trunk(self.cur_tok[:n], st, st.pos[:n], st.starts[:n], g_len=st.max_len,
                          num_splits=self.num_splits, row_map=self.step_row[:n] if self.packed else None)
        head = eng.head(h)
        eng.sample(head, self.T, self.top_p, seed=self.seed, row_keys=self.row_key[:n], steps=self.step_ctr[:n],
                   tok_out=self.samp_tok[:n], logp_out=self.samp_lp[:n], top_k=self.top_k)
        self._sched_step()

    # ------------------------------------------------------------------------------------------------ admission
    def _admit_body(self, cap: int) -> None:
        eng, st = self.eng, self.st
        p = _lib.SchedAdmitArgs()
        p.tok, p.pos, p.row, p.last_pos = (t.data_ptr() for t in (self.pk_tok, self.pk_pos, self.pk_row, self.pk_last))
        p.cu, p.tile_cu, p.cap = self.pk_cu.data_ptr(), self.pk_tile_cu.data_ptr(), cap
        with torch.cuda.device(self.dev):
            _lib.check(_lib.lib().uv_sched_admit(C.byref(self.args), C.byref(p), stream_ptr(self.dev)),
                       "uv_sched_admit")
        eng.trunk(self.pk_tok[:cap], st, self.pk_pos[:cap], self.pk_zero[:cap], g_len=st.max_len,
                  row_map=self.pk_row[:cap], scratch_tag="admit",   # buffers of its own: it may run beside a step
                  packed=dict(cu=self.pk_cu, tile_cu=self.pk_tile_cu, n_seq=self.B, max_tiles=cap // 16 + self.B,
                              last_pos=self.pk_last[:cap]))

    def _admit_pass(self, cap: int) -> None:
        """One admission pass of `cap` packed rows (one of pass_caps): captured once per size, replayed after."""
        if not self.use_graph:
            self._admit_body(cap)
        else:
            g = self._admit_graphs.get(cap)
            if g is None:
                # warm-up on a side stream with the queue hidden (tail = head: nothing is admitted, every packed
                # row is a pad row on the spare cache row), then capture
                s = torch.cuda.Stream(self.dev)
                s.wait_stream(torch.cuda.current_stream(self.dev))
                with torch.cuda.stream(s):
                    tail = self.ctl[CTL_TAIL].clone()
                    self.ctl[CTL_TAIL] = self.ctl[CTL_HEAD]
                    self._admit_body(cap)
                    self.ctl[CTL_TAIL] = tail
                torch.cuda.current_stream(self.dev).wait_stream(s)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, capture_error_mode="thread_local"):
                    self._admit_body(cap)
                self._admit_graphs[cap] = g
            g.replay()
        self.n_admit_passes += 1
        self._ctl_fresh = False

    def _read_ctl(self) -> None:
        c = self._ctl_h = self.ctl.cpu().numpy()
        self._head_h, self._fin_h = int(c[CTL_HEAD]), int(c[CTL_FIN])
        self._ctl_fresh = True

    def _plan_admission(self, head: int, free: int) -> tuple[int, int]:
        """(packed rows the next pass should get, requests it will take) for a queue head and a free-slot count --
        (0, 0): nothing to admit.  The pass takes the longest queue prefix of at most `free` requests whose prompts
        fit prefill_cap packed rows (what uv_sched_admit does on the device), padded to the next captured capacity."""
        k = min(self.n_enqueued - head, free)
        need = taken = 0
        for i in range(max(k, 0)):
            w = self._plen[head + i] - 1
            if need + w > self.prefill_cap:
                break
            need, taken = need + w, taken + 1
        if taken == 0:
            return 0, 0
        return next(c for c in self.pass_caps if c >= need), taken

    MAX_PASSES_PER_CALL = 8

    def admit(self, drain: bool = False) -> None:
        """Launch admission passes while the last counters say requests are waiting and slots are free: as many
        back-to-back passes as it takes to fill the free slots (a wave of rollouts that ended together frees more
        prompt tokens than one pass holds), planned on the host from the counters of the last read and its own
        copy of the queue -- no read-back in between.  drain: afterwards read the counters again and repeat until
        nothing more can be admitted (used when the batch is first filled)."""
        if not self.packed:
            return
        if self._commit_pending():       # a deferred pass moved the head: the counters in hand are stale
            if not drain:
                return
        while True:
            if not self._ctl_fresh:
                if not drain:
                    return
                self._read_ctl()
            head, free = self._head_h, self.B - (self._head_h - self._fin_h)
            launched = 0
            while launched < self.MAX_PASSES_PER_CALL:
                cap, taken = self._plan_admission(head, free)
                if cap == 0:
                    break
                self._admit_pass(cap)
                head, free, launched = head + taken, free - taken, launched + 1
            if launched == 0 or not drain:
                return

    def _commit_pending(self) -> bool:
        """If a deferred admission pass is outstanding: order the caller's stream after it and make its requests
        live.  Returns whether it did (the window that follows must then step every slot: the step kernel compacts
        at its first step, not before)."""
        if not self._admit_pending:
            return False
        main = torch.cuda.current_stream(self.dev)
        main.wait_event(self._admit_ev)
        with torch.cuda.device(self.dev):
            _lib.check(_lib.lib().uv_sched_commit(C.byref(self.args), stream_ptr(self.dev)), "uv_sched_commit")
        self._admit_pending = False
        self._ctl_fresh = False
        return True

    def _admit_beside(self) -> bool:
        """window()'s admission: if ONE pass refills the free slots and something is live to step meanwhile, launch it
        deferred on the admission stream (returns True); otherwise admit on the caller's stream as ``admit`` does."""
        head, live = self._head_h, self._head_h - self._fin_h
        free = self.B - live
        cap, taken = self._plan_admission(head, free)
        if cap == 0:
            return False
        more, _ = self._plan_admission(head + taken, free - taken)
        if not self.overlap_admit or live <= 0 or more:
            self.admit()
            return False
        main = torch.cuda.current_stream(self.dev)
        # the step kernels of this window must see "a pass is in flight" (no compaction under it) before the pass
        # starts: the marks are written on their stream, and the pass waits for that write
        self.ctl[CTL_INFLIGHT:CTL_DEFER + 1].copy_(self._flag_on, non_blocking=True)
        if self._admit_stream is None:
            self._admit_stream = torch.cuda.Stream(self.dev)
        self._admit_stream.wait_event(main.record_event())
        with torch.cuda.stream(self._admit_stream):
            self._admit_pass(cap)
            self._admit_ev = self._admit_stream.record_event()
        self._admit_pending = True
        self.n_deferred_passes += 1
        return True

    def prime(self) -> None:
        """First scheduling pass (admits queued requests into the idle slots) and graph capture."""
        if not self._primed:
            if self.packed:
                self.st.pos.zero_()
                self.admit(drain=True)
            else:
                self._sched_step()
            self._primed = True
        if self.use_graph and not self._graphs:
            self._step_graph(self.rows_needed())

    def warm(self) -> None:
        """Capture every graph a job can need -- the step over each batch-row bucket, the admission pass at each
        packed-row capacity -- while no request is live, so that none of these one-time costs (buffer allocation,
        library handles, capture, instantiation) lands between two steps of a running job.  The steps run here
        touch parked slots only (cache position 0 of idle rows); the counters they advance are reset."""
        if not self.use_graph:
            return
        if self.n_enqueued or self._primed:
            raise RuntimeError("warm() must run before the first request is enqueued")
        for n in self.buckets:
            self._step_graph(n)
        if self.packed:
            for cap in self.pass_caps:
                self._admit_pass(cap)
            self.n_admit_passes = 0
        # the harvest's device ops (index, scan, repeat_interleave, the small D2H copies), on both streams they
        # run on, at the size of a whole batch of rollouts finishing together: their one-time module loads and --
        # worse -- the allocator's first cudaMalloc calls for buffers of that size (each of which waits for the
        # steps in flight) would otherwise land in the first windows that have finishers.  A stand-in record
        # (request 0 owning that many output tokens) is gathered and put back; the blocks stay in the allocator's
        # per-stream pools.
        if self._side is None:
            self._side = torch.cuda.Stream(self.dev, priority=-1)
        keep = (self.fin_ring[0].clone(), self.out_len[0].clone(), self.prompt_len[0].clone())
        self.fin_ring[0] = 0
        self.out_len[0] = min(self.out_cap, self.B * self.max_new)
        self.prompt_len[0] = min(self.tok_cap, self.B * 256)
        for stream in (torch.cuda.current_stream(self.dev), self._side):
            stream.wait_stream(torch.cuda.current_stream(self.dev))
            with torch.cuda.stream(stream):
                p = self._gather(0, 1, True)
                p["requests"].cpu(), p["tokens"].cpu(), p["offsets"].cpu()
            torch.cuda.current_stream(self.dev).wait_stream(stream)
        self.fin_ring[0], self.out_len[0], self.prompt_len[0] = keep
        self.steps_run = 0
        self.bucket_steps.clear()
        for w in (CTL_STEPS, CTL_SLOT_STEPS, CTL_PREFILL_ROWS, CTL_ADMIT_PASSES, CTL_GENERATED, CTL_ACTIVE,
                  CTL_INFLIGHT, CTL_DEFER, CTL_DIRTY):
            self.ctl[w] = 0
        self.st.pos.zero_()
        self._ctl_fresh = True
        self.eng.check_status(None if self.packed else self.st_rows)

    def _step_graph(self, n: int) -> int:
        """Capture the step over n batch rows if it has not been yet; returns the steps that took (the warm-up on
        a side stream is a real step: state advances, nothing is rolled back, it counts towards the run)."""
        if n in self._graphs:
            return 0
        s = torch.cuda.Stream(self.dev)
        s.wait_stream(torch.cuda.current_stream(self.dev))
        with torch.cuda.stream(s):
            self._step_body(n)
        torch.cuda.current_stream(self.dev).wait_stream(s)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, capture_error_mode="thread_local"):
            self._step_body(n)
        self._graphs[n] = g
        self.steps_run += 1
        self.bucket_steps[n] = self.bucket_steps.get(n, 0) + 1
        return 1

    def rows_needed(self) -> int:
        """Batch rows the next steps run on: the smallest bucket that covers every slot that can be live."""
        if not self.compact:
            return self.B
        return next(b for b in self.buckets if b >= self.live_bound())

    def live_bound(self) -> int:
        """Upper bound of the live slots: requests enqueued minus requests known to have finished (the finished
        count may be stale; it only grows).  Whatever an admission pass takes from the queue is covered."""
        return min(self.B, self.n_enqueued - self._fin_h)

    def run(self, n_steps: int) -> None:
        self.prime()
        full = self._commit_pending()   # the step kernel compacts at its first step after a commit, not before it
        self.admit()   # packed prefill mode: refill the slots that the last harvest saw free
        self._steps(n_steps, self.B if full else self.rows_needed())

    def _steps(self, n_steps: int, n: int) -> None:
        if self.use_graph:
            n_steps -= min(n_steps, self._step_graph(n))
            g = self._graphs[n]
            for _ in range(n_steps):
                g.replay()
        else:
            for _ in range(n_steps):
                self._step_body(n)
        self.steps_run += n_steps
        self.bucket_steps[n] = self.bucket_steps.get(n, 0) + n_steps

    # ------------------------------------------------------------------------------------------------ harvest
    def counters(self, cached: bool = False) -> dict:
        """The control words; cached: as last read by a harvest / window call (no device access)."""
        c = self._ctl_h if (cached and self._ctl_h is not None) else self.ctl.cpu().numpy()
        return dict(head=int(c[CTL_HEAD]), tail=int(c[CTL_TAIL]), finished=int(c[CTL_FIN]),
                    active=int(c[CTL_ACTIVE]), status=int(c[CTL_STATUS]), steps=int(c[CTL_STEPS]),
                    generated=int(c[CTL_GENERATED]), slot_steps=int(c[CTL_SLOT_STEPS]))

    def window(self, n_steps: int, with_prompts: bool = False):
        """``run(n_steps)`` and, overlapped with it, the harvest of everything that had finished when it was
        launched: one small D2H of the counters (which waits for the steps launched earlier), then the next steps
        and admission pass go to the device, and only then is the finished requests' payload gathered -- on a side
        stream, while those steps run, so the device does not idle while the host collects rollouts.  Returns what
        ``harvest_packed`` returns (requests that finish during the steps launched here come with the next call;
        call ``harvest_packed`` after the last window)."""
        self.prime()
        full = self._commit_pending()    # (before the read: the counters then include what the pass admitted)
        if self.packed:
            self._read_ctl()
            fin = self._fin_h
            full = self._admit_beside() or full
            self._steps(n_steps, self.B if full else self.rows_needed())
        else:
            fin = self._fin_h = int(self.ctl[CTL_FIN].item())
            self.run(n_steps)
        if fin == self.n_harvested:
            return None
        if self._side is None:
            self._side = torch.cuda.Stream(self.dev, priority=-1)
        main = torch.cuda.current_stream(self.dev)
        with torch.cuda.stream(self._side):
            # everything this reads was complete before the counters were read: no event to wait for
            p = self._collect(fin, with_prompts)
        for v in p.values():
            if isinstance(v, torch.Tensor):
                v.record_stream(main)
        main.wait_stream(self._side)   # later work of the caller's stream (enqueue reuses ring space) comes after
        return p

    def harvest_packed(self, with_prompts: bool = False):
        """Finished requests since the last call as DEVICE tensors (the packed hand-off a trainer consumes without a
        host round trip of the payload; role of perf.py:55-95's packed micro-batches): dict with ``tokens`` int32 and
        ``logp`` fp32 (total,), ``offsets`` int64 (n + 1,) delimiting each request's span, ``versions`` int32 (n,),
        ``requests`` int64 (n,) request indices in finishing order, and ``metas`` (host list); with_prompts adds the
        requests' prompt tokens in the same form (``prompt_tokens`` int32, ``prompt_offsets`` int64), read from the
        device-side prompt ring before its space is released (``handoff.build_packed_device`` wants them).  One
        small D2H (the finished count and the span lengths' total); None when nothing finished."""
        if self.packed:
            self._read_ctl()   # head and finished count in one small D2H: the next admission pass is planned on them
            fin = self._fin_h
        else:
            fin = self._fin_h = int(self.ctl[CTL_FIN].item())
        if fin == self.n_harvested:
            return None
        return self._collect(fin, with_prompts)

    def _collect(self, fin: int, with_prompts: bool) -> dict:
        """Payload of the requests [n_harvested, fin) of the finishing order, gathered on the current stream."""
        # rollouts from a step (or an admission pass) whose kernels flagged a failure are not handed out
        self.eng.check_status(None if self.packed else self.st_rows)
        p = self._gather(self.n_harvested, fin, with_prompts)
        rid_h = p["requests"].cpu().tolist()
        p["metas"] = [self.meta.pop(r) for r in rid_h]
        for r in rid_h:
            self._span.pop(r, None)
            if self.packed:
                self._plen.pop(r, None)
        self.n_harvested = fin
        while self._oldest < self.n_enqueued and self._oldest not in self._span:
            self._oldest += 1
        return p

    def _gather(self, lo: int, hi: int, with_prompts: bool) -> dict:
        """Device tensors of the finished requests [lo, hi) of the finishing order (no host bookkeeping)."""
        k = torch.arange(lo, hi, device=self.dev) % self.q_cap
        rid = self.fin_ring[k].long()
        ri = rid % self.q_cap
        lens, offs, ver = self.out_len[ri].long(), self.out_off[ri], self.start_version[ri]
        ends = torch.cumsum(lens, 0)
        total = int(ends[-1].item())
        seg = torch.repeat_interleave(torch.arange(rid.numel(), device=self.dev), lens, output_size=total)
        within = torch.arange(total, device=self.dev) - (ends - lens)[seg]
        flat = (offs[seg] + within) % self.out_cap
        extra = {}
        if with_prompts:
            pl, po = self.prompt_len[ri].long(), self.prompt_off[ri]
            pends = torch.cumsum(pl, 0)
            ptotal = int(pends[-1].item())
            pseg = torch.repeat_interleave(torch.arange(rid.numel(), device=self.dev), pl, output_size=ptotal)
            pflat = (po[pseg] + torch.arange(ptotal, device=self.dev) - (pends - pl)[pseg]) % self.tok_cap
            extra = dict(prompt_tokens=self.tokens[pflat], prompt_offsets=torch.cat([pends.new_zeros(1), pends]))
        return dict(tokens=self.out_tok[flat], logp=self.out_lp[flat],
                    offsets=torch.cat([ends.new_zeros(1), ends]), versions=ver, requests=rid, **extra)

    def harvest(self):
        """Return the requests that finished since the last call as [(meta, tokens list, logp float32 array,
        start_version)] in finishing order (one small D2H for the counters, one gather + D2H for the payload)."""
        return self.unpack(self.harvest_packed())

    @staticmethod
    def unpack(p):
        """Host view of a harvest_packed() / window() result: [(meta, tokens, logp, start_version)]."""
        if p is None:
            return []
        toks, lps = p["tokens"].cpu().numpy(), p["logp"].cpu().numpy()
        off, ver_h = p["offsets"].cpu().numpy(), p["versions"].cpu().numpy()
        return [(m, toks[off[i]:off[i + 1]].tolist(), lps[off[i]:off[i + 1]].copy(), int(ver_h[i]))
                for i, m in enumerate(p["metas"])]

    def n_active(self) -> int:
        return int(self.ctl[CTL_ACTIVE].item())
