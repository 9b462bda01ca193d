"""DecodeRunner / sample / generate / generate_continuous with the reference's signatures (ultraviolet/model.py:
1075-1354) on the B200 decode engine."""
from __future__ import annotations

import os

import numpy as np
import torch
from torch import Tensor

from .fast_decode import _engine
from .scheduler import GpuScheduler


def fresh_seed() -> int:
    """Philox seed for a call that was given none: drawn from torch's global generator, so ``torch.manual_seed``
    governs it and successive calls see fresh noise (as the reference's ``torch.rand_like`` draws do); the
    distributed rank is mixed in so that ranks seeded alike do not replay one stream."""
    s = int(torch.randint(0, 2 ** 62, (1,)).item())
    rank = int(os.environ.get("RANK", "0") or 0)
    return (s ^ (rank * 0xD1B54A32D192ED03)) & (2 ** 63 - 1)


def sample(logits: Tensor, temperature: float, top_k: int = 0, top_p: float = 1.0) -> Tensor:
    """model.py:1194-1211 on softcapped logits (B, V): temperature <= 0 -> argmax, else a draw from
    softmax(logits / T) restricted to the top_k largest logits (ties with the k-th kept) and then to the top_p
    nucleus.  One uniform per row from torch's CUDA generator (so torch.manual_seed governs it), inverse-CDF instead
    of Gumbel-max: the same distribution from a different random stream."""
    from . import _lib
    from .kernels._util import DTYPE_CODE, need_cuda, stream_ptr
    import ctypes as C
    need_cuda(logits)
    if logits.stride(-1) != 1:
        logits = logits.contiguous()
    B, V = logits.shape
    tok = torch.empty(B, dtype=torch.int64, device=logits.device)
    lp = torch.empty(B, dtype=torch.float32, device=logits.device)
    u = torch.rand(B, device=logits.device, dtype=torch.float32) if temperature > 0 else None
    with torch.cuda.device(logits.device):
        rc = _lib.lib().uv_sample_topk(logits.data_ptr(), DTYPE_CODE[logits.dtype], logits.stride(0), B, V, 1, 0.0,
                                       0.0, 1.0, float(temperature), int(top_k or 0), float(top_p),
                                       None if u is None else u.data_ptr(), C.c_uint64(0), None, None,
                                       tok.data_ptr(), lp.data_ptr(), None, None, stream_ptr(logits.device))
    _lib.check(rc, "uv_sample_topk")
    return tok


class DecodeRunner:
    """One decode step + sample per call, replayed from a CUDA graph per global-context bucket (model.py:1075-1150).
    ``out_tok`` / ``out_logp`` are static buffers (callers clone).  ``compile`` is accepted and ignored: the step is
    already a fixed kernel sequence."""

    def __init__(self, model, st, bucket: int = 1024, use_graph: bool = True, temperature: float = 1.0,
                 top_k: int = 0, compile: bool = False, skip_attn: bool = False, top_p: float = 1.0,
                 seed: int | None = None):
        """seed: Philox key of this runner's draws; None (the default) takes a fresh one from torch's generator
        (``fresh_seed``), an int makes the token streams reproducible."""
        self.m, self.st, self.bucket = model, st, bucket
        self.eng = _engine(model)
        self.use_graph = use_graph
        self.temperature, self.top_k, self.top_p = temperature, int(top_k or 0), top_p
        self.seed = fresh_seed() if seed is None else int(seed)
        dev = st.pos.device
        self.tok = torch.zeros(st.B, dtype=torch.long, device=dev)
        # The sampler writes the new tokens straight into the step's input buffer: feeding step() its own output
        # costs no copy.
        self.out_tok, self.out_logp = self.tok, self.eng.scratch(st.B)["logp"]
        self.want_logp = True
        self.row_keys = torch.arange(st.B, dtype=torch.int64, device=dev)
        self.steps = torch.zeros(st.B, dtype=torch.int64, device=dev)
        self.graphs: dict[tuple, torch.cuda.CUDAGraph] = {}
        self.skip_attn = skip_attn
        self.host_in = self.host_out = self.host_logp = None   # pinned buffers of step_host, made on first use

    def g_len(self, p: int) -> int:
        return min(self.st.max_len, ((p + 1 + self.bucket - 1) // self.bucket) * self.bucket)

    @property
    def out_logits(self) -> Tensor:
        """fp32 softcapped logits of the last step (computed on demand from the raw head output)."""
        a, b, c = self.eng.cfg.softcap
        return a * torch.sigmoid((self.eng.head_buffer(self.st.B).float() + b) / c)

    def _body(self, g_len: int) -> None:
        st, eng = self.st, self.eng
        h = eng.trunk(self.tok, st, st.pos, st.starts, g_len=g_len, num_splits=self.m.__dict__.get(
            "decode_num_splits", getattr(type(self.m), "decode_num_splits", None)), skip_attn=self.skip_attn)
        eng.sample(eng.head(h), self.temperature, self.top_p, seed=self.seed, row_keys=self.row_keys,
                   steps=self.steps, tok_out=self.tok, inc_a=st.pos, inc_b=self.steps,  # advances both counters
                   top_k=self.top_k)

    def step(self, tok: Tensor) -> Tensor:
        p = int(self.st.host_pos.max())
        assert p < self.st.max_len, "cache full"
        gl = self.g_len(p)
        if tok.data_ptr() != self.tok.data_ptr():
            self.tok.copy_(tok)
        if not self.use_graph:
            self._body(gl)
        else:
            self._graph(gl, host=False).replay()
        self.st.host_pos += 1
        return self.out_tok

    def _graph(self, gl: int, host: bool) -> torch.cuda.CUDAGraph:
        """The step's graph for global-context bucket gl; host: with the copy of the input tokens from the pinned
        host buffer in front and the copy of the sampled tokens (and log-probs) to pinned host buffers behind."""
        g = self.graphs.get((gl, host))
        if g is None:
            dev = self.st.pos.device

            def body():
                if host:
                    self.tok.copy_(self.host_in, non_blocking=True)
                self._body(gl)
                if host:
                    self.host_out.copy_(self.out_tok, non_blocking=True)
                    self.host_logp.copy_(self.out_logp, non_blocking=True)
            pos0, steps0, tok0 = self.st.pos.clone(), self.steps.clone(), self.tok.clone()
            s = torch.cuda.Stream(dev)
            s.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(s):  # warm-up: the slot written now is rewritten by the real replay
                self._body(gl)
                self.st.pos.copy_(pos0)
                self.steps.copy_(steps0)
                self.tok.copy_(tok0)
            torch.cuda.current_stream(dev).wait_stream(s)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, capture_error_mode="thread_local"):
                body()
            self.graphs[(gl, host)] = g
            self.eng.check_status(self.st.B)  # the warm-up run of a new bucket is also the failure check
        return g

    def step_host(self, tok: Tensor | None = None) -> Tensor:
        """``step`` for callers whose tokens live on the host: the input tokens are read from the pinned buffer
        ``host_in`` (tok, if given, is copied there first; writing into ``host_in`` directly saves that), the
        sampled tokens and their log-probs land in the pinned buffers ``host_out`` / ``host_logp``, and the call
        returns ``host_out`` after the device has finished.  Both copies are nodes of the step's CUDA graph: one
        graph launch and one synchronisation per step."""
        if self.host_in is None:
            B = self.st.B
            self.host_in = torch.zeros(B, dtype=torch.long).pin_memory()
            self.host_out = torch.zeros(B, dtype=torch.long).pin_memory()
            self.host_logp = torch.zeros(B, dtype=torch.float32).pin_memory()
        if tok is not None and tok.data_ptr() != self.host_in.data_ptr():
            self.host_in.copy_(tok)
        p = int(self.st.host_pos.max())
        assert p < self.st.max_len, "cache full"
        gl = self.g_len(p)
        dev = self.st.pos.device
        if not self.use_graph:
            self.tok.copy_(self.host_in, non_blocking=True)
            self._body(gl)
            self.host_out.copy_(self.out_tok, non_blocking=True)
            self.host_logp.copy_(self.out_logp, non_blocking=True)
        else:
            self._graph(gl, host=True).replay()
        torch.cuda.current_stream(dev).synchronize()
        self.st.host_pos += 1
        return self.host_out


def _new_state(model, rows, max_len, eng, ring_extra):
    """model.new_state with the extra ring slots prefill lanes want; models patched by another library's
    patch_model (no ring_extra argument) get the plain state, and lanes then stop at the window as before."""
    if ring_extra:
        try:
            return model.new_state(rows, max_len, eng.dtype, eng.device, ring_extra=ring_extra)
        except TypeError:
            pass
    return model.new_state(rows, max_len, eng.dtype, eng.device)


def _left_pad(prompts, pad_id, dev):
    Tp = max(len(p) for p in prompts)
    idx = torch.full((len(prompts), Tp), pad_id, dtype=torch.long)
    starts = torch.zeros(len(prompts), dtype=torch.long)
    for b, p in enumerate(prompts):
        idx[b, Tp - len(p):] = torch.as_tensor(p, dtype=torch.long)
        starts[b] = Tp - len(p)
    return idx.to(dev), starts.to(dev)


@torch.no_grad()
def generate(model, prompts, max_new: int, temperature: float = 1.0, top_k: int = 0, eos_id: int | None = None,
             pad_id: int = 0, max_len: int | None = None, use_graph: bool = True, bucket: int = 1024,
             dtype=None, compile: bool = True, top_p: float = 1.0, seed: int | None = None):
    """Static-batch generation (model.py:1228-1263): left-padded prefill, lockstep decode, rows cut after EOS.
    seed: None draws a fresh Philox seed per call from torch's generator; an int reproduces the streams."""
    eng = _engine(model)
    dev = eng.device
    B = len(prompts)
    idx, starts = _left_pad(prompts, pad_id, dev)
    max_len = max_len or (idx.size(1) + max_new)
    st = model.new_state(B, max_len, eng.dtype, dev)
    runner = DecodeRunner(model, st, bucket=bucket, use_graph=use_graph, temperature=temperature, top_k=top_k,
                          top_p=top_p, seed=seed)
    # prefill every position but the last through the decode kernels, then let the runner take the last prompt
    # token so that token 0 is drawn by the same fused sampler as every later token
    T = idx.size(1)
    if T > 1:
        model.prefill(idx[:, :-1], starts, st)
    st.starts.copy_(starts)
    tok = runner.step(idx[:, -1]).clone()
    out = [tok]
    done = torch.zeros(B, dtype=torch.bool, device=dev)
    if eos_id is not None:
        done |= tok == eos_id
    for i in range(max_new - 1):
        if st.host_pos.max() >= max_len:
            break
        tok = runner.step(tok).clone()
        out.append(tok)
        if eos_id is not None:
            done |= tok == eos_id
            if i % 64 == 63 and bool(done.all()):
                break
    eng.check_status(B)  # raises if a kernel flagged a timed-out tile copy or a skipped cache write
    res = []
    for row in torch.stack(out, 1).tolist():
        if eos_id is not None and eos_id in row:
            row = row[:row.index(eos_id) + 1]
        res.append(row)
    return res


@torch.no_grad()
def generate_continuous(model, prompts, max_new: int, batch: int, temperature: float = 1.0, top_k: int = 0,
                        eos_id: int | None = None, pad_id: int = 0, check_every: int = 16, use_graph: bool = True,
                        bucket: int = 1024, dtype=None, compile: bool = True, target_lens=None, stats=None,
                        top_p: float = 1.0, seed: int | None = None, prefill_lanes: int = 0,
                        packed_prefill: bool | None = None):
    """Continuous batching over `batch` cache slots (model.py:1266-1354), scheduled on the device; completions in
    prompt order.  target_lens[i] caps request i's length (the reference's benchmarking hook, model.py:1312).
    seed: None draws a fresh Philox seed per call from torch's generator (request i's stream is keyed by (seed, i));
    an int reproduces the streams whatever slot a request lands in.
    Prompts enter the cache through packed prefill passes at admission (packed_prefill, the default: every
    check_every steps the freed slots are refilled in one packed batch, as the reference refills with a batched
    prefill), or through the decode step itself (packed_prefill=False; prefill_lanes > 0 then feeds several prompt
    tokens of a slot per step)."""
    if packed_prefill is None:
        packed_prefill = prefill_lanes == 0
    eng = _engine(model)
    n = len(prompts)
    B = min(batch, n)
    max_prompt = max(len(p) for p in prompts)
    st = _new_state(model, GpuScheduler.state_rows(B, prefill_lanes, packed_prefill),
                    max_prompt + max_new + check_every, eng, GpuScheduler.ring_extra(prefill_lanes))
    sched = GpuScheduler(eng, st, max_new=max_new, temperature=temperature, top_p=top_p, top_k=top_k, eos_id=eos_id,
                         pad_id=pad_id, seed=fresh_seed() if seed is None else int(seed), q_cap=max(n, 2), max_prompt=max_prompt, use_graph=use_graph,
                         prefill_lanes=prefill_lanes, packed_prefill=packed_prefill,
                         tok_cap=sum(len(p) for p in prompts) + 1,
                         out_cap=(int(np.minimum(np.asarray(target_lens), max_new).sum()) if target_lens is not None
                                  else n * max_new) + 1)
    sched.enqueue([list(p) for p in prompts], limits=target_lens, metas=list(range(n)))
    results = [None] * n
    got = 0
    while got < n:
        # check_every steps go to the device first; what had finished before them is collected while they run
        for i, toks, _, _ in sched.unpack(sched.window(check_every)):
            results[i] = toks
            got += 1
        if got < n and sched.live_bound() == 0:   # every request is known to have finished: collect without stepping
            for i, toks, _, _ in sched.harvest():
                results[i] = toks
                got += 1
    if stats is not None:
        stats.update(steps=sched.steps_run, prefilled=n, slots=B)
    return results
