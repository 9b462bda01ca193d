"""Whole decode path on the GPU against the oracle and the reference-generated golden logits.

Tolerances: logits within 2e-2 relative (bf16 activations, int8 KV) of the fp32 reference path; the reference's own
int8-vs-fp16 bound is max abs < 0.25 with argmax agreement > 0.9 (tests/test_math_kernels.py:167-171)."""
import numpy as np
import pytest
import torch

from oracle import model as om
from tests import golden_inputs as gi
from tests.helpers import build_model, golden, oracle_weights

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _gpu_model(spec, dtype=torch.bfloat16):
    m = build_model(spec).to(DEV).to(dtype)
    return m.fuse_for_inference(dtype)


def _teacher_forced_gpu(m, idx, starts, cont, max_len):
    st = m.new_state(idx.shape[0], max_len)
    t = lambda a: torch.from_numpy(a).to(DEV)
    outs = [m.prefill(t(idx), t(starts), st)]
    for i in range(cont.shape[1]):
        outs.append(m.decode_step(t(np.ascontiguousarray(cont[:, i])), st, max_len))
    return torch.stack(outs, 1).float().cpu().numpy(), st


@pytest.mark.parametrize("name", sorted(gi.model_specs()))
def test_teacher_forced_logits(name):
    g = golden("model")
    spec = gi.model_specs()[name]
    m = _gpu_model(spec)
    idx, starts, cont, max_len = gi.teacher_inputs(spec)
    lg, st = _teacher_forced_gpu(m, idx, starts, cont, max_len)
    assert np.isfinite(lg).all()
    # (1) the reference itself (fp32 weights and activations), stored columns
    cols = gi.logit_columns(spec, lg.shape[-1])
    ref = g[name + ".logits"]
    err = np.abs(lg[..., cols] - ref)
    # the path's stated tolerance is 2e-2 relative; measured on B200: 0.6e-3 .. 1.3e-3 of the largest logit, and the
    # same elementwise (|err| / max(|ref|, 1) <= 1.9e-3), so the bound is set four times tighter than stated
    assert err.max() <= 5e-3 * np.abs(ref).max(), (err.max(), np.abs(ref).max())
    assert (err / np.maximum(np.abs(ref), 1.0)).max() <= 5e-3
    assert err.mean() < 0.01
    assert (lg.argmax(-1) == g[name + ".argmax"]).mean() > 0.98
    # (2) the oracle on the same bf16-rounded weights
    mc = build_model(spec)
    W = oracle_weights(mc, "bf16")
    ost = om.State(mc.cfg, idx.shape[0], max_len)
    outs = [om.prefill(W, mc.cfg, idx, starts, ost)]
    for i in range(cont.shape[1]):
        outs.append(om.decode_step(W, mc.cfg, cont[:, i], ost))
    olg = np.stack(outs, 1)
    err = np.abs(lg - olg)
    assert err.max() <= 5e-3 * np.abs(olg).max(), (err.max(), np.abs(olg).max())
    assert np.array_equal(st.pos.cpu().numpy(), ost.pos) and np.array_equal(st.starts.cpu().numpy(), ost.starts)
    # int8 cache of the first layer: same bytes up to bf16 rounding of the projections (one quantisation step)
    # (slots of real tokens only: the packed prefill never computes or writes the left padding, exactly as the
    # reference's packed route does not -- rows read keys >= start.  Slot s of a ring holds position t, the newest
    # one with t % S == s.)
    d = np.abs(st.k[0].cpu().numpy().astype(np.int16) - ost.k[0].astype(np.int16))
    S0 = ost.k[0].shape[2]
    d = d[:, :, :S0]
    slot = np.arange(S0)[None, :]
    if m.cfg.is_global(0):
        held = np.broadcast_to(slot, (idx.shape[0], S0))
    else:
        last = ost.pos[:, None] - 1
        held = last - np.remainder(last - slot, S0)
    valid = (held >= starts[:, None]) & (held >= 0) & (held < ost.pos[:, None])
    dv = d[np.broadcast_to(valid[:, None, :, None], d.shape)]
    assert dv.max() <= 3 and (dv != 0).mean() < 0.35, (dv.max(), (dv != 0).mean())


def test_greedy_stream_random_init_128_tokens():
    """UV-50M, random init seed 0 (unperturbed): greedy streams identical to the oracle's for 128 tokens.  With
    zero-initialised output projections the stream is constant, so this pins the embedding / head / sampler path;
    the informative comparison is the teacher-forced one above."""
    from ultraviolet_b200.generate import generate
    spec = dict(gi.model_specs()["uv50m"], perturb="none")
    torch.manual_seed(0)
    from ultraviolet_b200.model import MathLM, make_config
    m = MathLM(make_config("uv-50m-alpha", vocab_size=16384))
    prompts = [[5, 9, 200, 3000], [17, 4242, 16000]]
    W = oracle_weights(m, "bf16")
    ref = om.generate(W, m.cfg, prompts, 8)            # the oracle is slow: 8 tokens, then the stream is constant
    mg = m.to(DEV).to(torch.bfloat16).fuse_for_inference(torch.bfloat16)
    out = generate(mg, prompts, 128, temperature=0.0)
    assert [r[:8] for r in out] == ref
    assert all(len(r) == 128 for r in out)
    assert all(len(set(r[8:])) == len(set(ref[i][-1:])) for i, r in enumerate(out))  # constant continuation


def test_generate_and_continuous_tiny():
    from ultraviolet_b200.generate import generate, generate_continuous
    g = golden("model")
    spec = gi.model_specs()["tiny"]
    m = _gpu_model(spec)
    ge, c = spec["generate"], spec["continuous"]
    out = generate(m, ge["prompts"], ge["max_new"], temperature=0.0, use_graph=True)
    ref = gi.unpack_lists(g["tiny.generate"])
    assert [len(r) for r in out] == [len(r) for r in ref]
    agree = np.mean([a == b for r, s in zip(out, ref) for a, b in zip(r, s)])
    assert agree > 0.95, agree  # measured on B200: identical to the reference's streams (a bf16 near-tie may flip)
    eager = generate(m, ge["prompts"], ge["max_new"], temperature=0.0, use_graph=False)
    assert eager == out         # graph replay == eager launches (tests/test_math_kernels.py:176-189)
    cref = gi.unpack_lists(g["tiny.continuous"])
    # prompts through the decode step: measured identical to the reference's continuous streams
    step = generate_continuous(m, c["prompts"], c["max_new"], batch=c["batch"], temperature=0.0, eos_id=c["eos_id"],
                               check_every=c["check_every"], target_lens=c["target_lens"], packed_prefill=False)
    assert [len(r) for r in step] == c["target_lens"]
    agree = np.mean([a == b for r, s in zip(step, cref) for a, b in zip(r, s)])
    assert agree > 0.95, agree
    # packed admission passes (the default): the prompts' keys come out of GEMMs over a few hundred packed rows
    # instead of the slots' rows, so a near-tie of this random tiny model can flip (measured agreement 0.82)
    cont = generate_continuous(m, c["prompts"], c["max_new"], batch=c["batch"], temperature=0.0,
                               eos_id=c["eos_id"], check_every=c["check_every"], target_lens=c["target_lens"])
    assert [len(r) for r in cont] == c["target_lens"]
    agree = np.mean([a == b for r, s in zip(cont, cref) for a, b in zip(r, s)])
    assert agree > 0.7, agree
    # continuous batching vs static generation per prompt (tests/test_math_model.py:198-210).  The two prefill
    # differently here -- generate() through the packed kernel over unquantised keys, the device scheduler through the
    # decode step over the int8 cache -- so a near-tie of this random tiny model can flip and the greedy tails then
    # part ways: the first token must agree, and most tokens overall
    sames = []
    for i, p in enumerate(c["prompts"][:4]):
        solo = generate(m, [p], c["target_lens"][i], temperature=0.0, use_graph=False)[0]
        assert solo[0] == cont[i][0], (i, solo, cont[i])
        sames += [a == b for a, b in zip(solo, cont[i])]
    assert np.mean(sames) > 0.5, np.mean(sames)


def test_continuous_with_prefill_lanes_matches_without():
    """Prefill lanes only change how fast prompts enter the cache: per-request greedy outputs stay the same (up to
    the batch-size dependent bf16 GEMM rounding that the other comparisons of this file also allow), with the
    graph and without."""
    from ultraviolet_b200.generate import generate_continuous
    spec = gi.model_specs()["tiny"]
    m = _gpu_model(spec)
    c = spec["continuous"]
    r = np.random.default_rng(8)
    prompts = [r.integers(1, 500, r.integers(3, 40)).tolist() for _ in range(14)]
    kw = dict(batch=4, temperature=0.0, eos_id=c["eos_id"], check_every=4)
    s0 = {}
    base = generate_continuous(m, prompts, 10, stats=s0, packed_prefill=False, **kw)
    for graph in (False, True):
        s1 = {}
        lanes = generate_continuous(m, prompts, 10, prefill_lanes=6, use_graph=graph, stats=s1, **kw)
        assert [len(x) for x in lanes] == [len(x) for x in base]
        agree = np.mean([a == b for x, y in zip(lanes, base) for a, b in zip(x, y)])
        assert agree > 0.9, (graph, agree)
        # prompts of up to 39 tokens against a window of 8: the local rings carry lane_chunk extra slots, so the
        # lanes keep feeding chunks after the ring has wrapped and the job needs far fewer steps
        assert s1["steps"] < 0.7 * s0["steps"], (s0, s1)


def test_patch_reference_style_object_and_weight_refresh():
    """patch_model binds onto any object with MathLM's parameter layout; refresh keeps the arena pointers."""
    from ultraviolet_b200.fast_decode import patch_model, refresh_weights, unpatch_model
    spec = gi.model_specs()["tiny"]
    m = build_model(spec).to(DEV).to(torch.bfloat16)
    patch_model(m, "int8")
    eng = m._uvb200_engine
    ptr = eng.arena.data_ptr()
    st = m.new_state(3, 16)
    tok = torch.tensor([1, 2, 3], device=DEV)
    a = m.decode_step(tok, st, 16).clone()
    with torch.no_grad():
        m.blocks[0].attn.wo.mul_(0.5)
    refresh_weights(m)
    assert eng.arena.data_ptr() == ptr
    st2 = m.new_state(3, 16)
    b = m.decode_step(tok, st2, 16)
    assert not torch.equal(a, b)
    unpatch_model(m)
    assert "decode_step" not in m.__dict__


def test_device_failure_words_are_read_and_raise():
    """The kernels flag silent failures in two device words (a cache tile copy that timed out, a skipped cache
    write); the engine reads them.  The words are set by hand here -- no kernel is made to fail."""
    from ultraviolet_b200 import _lib
    from ultraviolet_b200.generate import generate
    spec = gi.model_specs()["tiny"]
    m = _gpu_model(spec)
    eng = m.engine
    out = generate(m, [[1, 2, 3], [4, 5]], 4, temperature=0.0, use_graph=False)
    assert eng.device_status() == {"attn_status": 0, "kv_oob": 0} and len(out) == 2
    B = next(iter(eng._scratch))
    eng.scratch(B)["flags"][0] = 1          # attention status bit 0
    with pytest.raises(_lib.UvError, match="status"):
        eng.check_status()
    assert eng.device_status() == {"attn_status": 0, "kv_oob": 0}   # raising clears the words
    eng.scratch(B)["flags"][1] = 3          # skipped cache writes
    with pytest.raises(_lib.UvError, match="3 KV"):
        eng.check_status(B)


def test_seed_rule_top_k_and_skip_attn():
    from ultraviolet_b200.generate import DecodeRunner, generate
    spec = gi.model_specs()["tiny"]
    m = _gpu_model(spec)
    prompts = [[5, 6, 7, 8], [9, 10, 11], [12, 13, 14, 15, 16]]
    # no seed: every call draws a fresh Philox seed from torch's generator -> torch.manual_seed reproduces a call
    # sequence, successive calls differ
    torch.manual_seed(1)
    a1 = generate(m, prompts, 24, temperature=1.5, use_graph=False)
    a2 = generate(m, prompts, 24, temperature=1.5, use_graph=False)
    torch.manual_seed(1)
    b1 = generate(m, prompts, 24, temperature=1.5, use_graph=False)
    assert a1 != a2 and len({tuple(r) for r in a1}) > 1
    assert b1 == a1
    c1 = generate(m, prompts, 24, temperature=1.5, use_graph=False, seed=17)
    c2 = generate(m, prompts, 24, temperature=1.5, use_graph=True, seed=17)
    assert c1 == c2
    # top_k = 1 is greedy whatever the temperature
    greedy = generate(m, prompts, 12, temperature=0.0, use_graph=False)
    k1 = generate(m, prompts, 12, temperature=2.0, top_k=1, use_graph=False, seed=3)
    assert k1 == greedy
    # skip_attn: the profiling switch runs (attention kernel left out) and still produces tokens
    st = m.new_state(3, 32)
    runner = DecodeRunner(m, st, bucket=32, use_graph=False, temperature=0.0, skip_attn=True)
    tok = runner.step(torch.tensor([1, 2, 3], device=DEV)).clone()
    assert tok.shape == (3,) and int(st.pos[0]) == 1
    # step_host: tokens in and out through pinned host buffers (copies inside the step's graph) = step on device
    # tensors, token for token and log-prob for log-prob
    first = torch.tensor([4, 5, 6])
    for graph in (False, True):
        ra = DecodeRunner(m, m.new_state(3, 32), bucket=32, use_graph=graph, temperature=1.3, seed=9)
        rb = DecodeRunner(m, m.new_state(3, 32), bucket=32, use_graph=graph, temperature=1.3, seed=9)
        ta, tb = first.to(DEV), first.clone()
        for _ in range(6):
            ta = ra.step(ta).clone()
            la = ra.out_logp.clone()
            tb = rb.step_host(tb)
            assert tb.is_pinned() and not tb.is_cuda and tb.tolist() == ta.tolist()
            assert torch.equal(rb.host_logp, la.cpu())


@pytest.mark.parametrize("name", ["uv50m", "tiny_hd64"])
def test_cache_bytes_against_the_reference_in_bf16(name):
    """The reference itself run in bfloat16 on the CPU (tests/golden/model_bf16.npz) rounds where this path rounds,
    so the first layer's int8 cache bytes agree far more tightly than against the fp32 run: a quantisation step on
    a small fraction of the bytes (GEMM summation order), never more."""
    g = golden("model_bf16")
    spec = gi.model_specs()[name]
    m = _gpu_model(spec)
    idx, starts, cont, max_len = gi.teacher_inputs(spec)
    lg, st = _teacher_forced_gpu(m, idx, starts, cont, max_len)
    cols = gi.logit_columns(spec, lg.shape[-1])
    ref = g[name + ".logits"]
    err = np.abs(lg[..., cols] - ref)
    assert err.max() <= 2e-2 * np.abs(ref).max(), (err.max(), np.abs(ref).max())
    assert (lg.argmax(-1) == g[name + ".argmax"]).mean() > 0.9
    pos = g[name + ".pos"]
    stats = {}
    for l in spec["cache_layers"]:
        S = g[f"{name}.k{l}"].shape[2]
        slot = np.arange(S)[None, :]
        if m.cfg.is_global(l):
            held = np.broadcast_to(slot, (idx.shape[0], S))
        else:
            last = pos[:, None] - 1
            held = last - np.remainder(last - slot, S)
        valid = (held >= starts[:, None]) & (held >= 0) & (held < pos[:, None])
        for kind, cache in (("k", st.k[l]), ("v", st.v[l])):
            d = np.abs(cache.cpu().numpy()[:, :, :S].astype(np.int16) - g[f"{name}.{kind}{l}"].astype(np.int16))
            dv = d[np.broadcast_to(valid[:, None, :, None], d.shape)]
            stats[(kind, l)] = (int(dv.max()), float((dv != 0).mean()))
    first = spec["cache_layers"][0]
    for kind in ("k", "v"):
        mx, frac = stats[(kind, first)]
        # first layer (embedding -> norm -> one GEMM -> norm / RoPE -> quantiser): measured bit-identical to the
        # reference's bytes on B200; a GEMM summation-order flip may cost a step on a few bytes
        assert mx <= 1 and frac < 0.01, stats
    for (kind, l), (mx, frac) in stats.items():
        # deeper layers: the residual stream is carried with the lambdas folded into the weights, so it rounds at
        # other points than the reference's op-by-op bf16 chain (measured: up to 4 steps, ~42 % of the bytes)
        assert mx <= 5 and frac < 0.5, stats


def test_continuous_with_packed_admission_matches_static_generation():
    """Packed admission passes (the default of generate_continuous): requests enter through one packed prefill batch
    per refill, the way generate() prefills.  Per-request greedy outputs agree with static generation (the frames
    differ -- position 0 here, left-padded there -- so only bf16 rounding separates them) and with the
    decode-step route; every request comes back with its length; far fewer steps than feeding prompts token by token."""
    from ultraviolet_b200.generate import generate, generate_continuous
    spec = gi.model_specs()["tiny"]
    m = _gpu_model(spec)
    r = np.random.default_rng(9)
    prompts = [r.integers(1, 500, r.integers(1, 40)).tolist() for _ in range(19)]    # includes 1-token prompts
    lens = r.integers(1, 12, len(prompts)).tolist()
    s_p, s_s = {}, {}
    for graph in (False, True):
        got = generate_continuous(m, prompts, 12, batch=5, temperature=0.0, eos_id=None, check_every=4,
                                  target_lens=lens, stats=s_p, use_graph=graph)
        assert [len(x) for x in got] == lens
        sames = []
        for i, p in enumerate(prompts):
            solo = generate(m, [p], lens[i], temperature=0.0, use_graph=False)[0]
            sames += [a == b for a, b in zip(solo, got[i])]
        assert np.mean(sames) > 0.8, (graph, np.mean(sames))
    step = generate_continuous(m, prompts, 12, batch=5, temperature=0.0, eos_id=None, check_every=4,
                               target_lens=lens, stats=s_s, packed_prefill=False)
    assert [len(x) for x in step] == lens
    assert np.mean([a == b for x, y in zip(step, got) for a, b in zip(x, y)]) > 0.6
    assert s_p["steps"] < 0.6 * s_s["steps"], (s_p, s_s)


def test_admission_pass_writes_the_same_cache_as_host_prefill():
    """The cache an admission pass leaves (device-built packed batch, padded to a power of two of rows, slots chosen
    on the device) against prefill() of the same prompts (host-built packed batch): same positions, same slots,
    bytes equal up to the GEMMs' batch-size dependent rounding; the slot holds the last prompt token at position
    P - 1."""
    from ultraviolet_b200.scheduler import GpuScheduler
    spec = gi.model_specs()["tiny_hd64"]
    m = _gpu_model(spec)
    cfg, eng = m.cfg, m.engine
    r = np.random.default_rng(23)
    n, P = 6, 21                                  # equal lengths: the left-padded frame is the position frame
    prompts = [r.integers(1, cfg.vocab_size, P).tolist() for _ in range(n)]
    idx = torch.tensor(prompts, device=DEV)
    ref = m.new_state(n, 64)
    m.prefill(idx[:, :-1], torch.zeros(n, dtype=torch.long, device=DEV), ref)
    st = m.new_state(GpuScheduler.state_rows(n, 0, True), 64)
    sch = GpuScheduler(eng, st, max_new=4, temperature=1.0, eos_id=0, seed=1, q_cap=16, max_prompt=32,
                       packed_prefill=True, use_graph=False)
    sch.enqueue(prompts)
    sch.prime()
    torch.cuda.synchronize()
    assert sch.n_admit_passes == 1 and sch.counters()["head"] == n
    assert st.pos.tolist() == [P - 1] * n and sch.cur_tok[:n].tolist() == [p[-1] for p in prompts]
    for l in range(cfg.n_layers):
        S = ref.k[l].shape[2]
        t = np.arange(max(0, P - 1 - S) if not cfg.is_global(l) else 0, P - 1)
        sl = t % S if not cfg.is_global(l) else t
        for a, b in ((st.k[l], ref.k[l]), (st.v[l], ref.v[l])):
            d = (a[:n][:, :, sl].int() - b[:, :, sl].int()).abs()
            assert int(d.max()) <= (1 if l == 0 else 3) and (d > 0).float().mean().item() < (0.02 if l == 0 else 0.3), \
                (l, int(d.max()), (d > 0).float().mean().item())
    eng.check_status()


def test_window_harvest_and_compaction_change_no_rollout():
    """The same seeded job three ways: run + harvest per window; window() (harvest overlapped with the next
    steps); window() without slot compaction.  Request outputs (tokens, log-probs, start versions) are keyed by
    request, so every route returns the same rollouts -- tokens equal, log-probs equal up to the batch-size dependent
    rounding of the GEMMs when the step runs on fewer rows -- and compaction really shrinks the step."""
    from ultraviolet_b200.scheduler import GpuScheduler
    spec = gi.model_specs()["tiny_hd64"]
    m = _gpu_model(spec)
    cfg, eng = m.cfg, m.engine
    r = np.random.default_rng(31)
    n, B = 150, 64
    prompts = [r.integers(1, cfg.vocab_size, r.integers(1, 24)).tolist() for _ in range(n)]
    limits = r.integers(1, 40, n).tolist()

    def drive(route, compact, beside=False):
        st = m.new_state(GpuScheduler.state_rows(B, 0, True), 80)
        sch = GpuScheduler(eng, st, max_new=40, temperature=0.0, eos_id=None, seed=5, q_cap=256, max_prompt=32,
                           packed_prefill=True, compact=compact, overlap_admit=beside)
        if route == "window":
            sch.warm()                          # every graph captured up front: nothing a request sees changes
            assert sch.counters()["steps"] == 0 and set(sch._graphs) == set(sch.buckets)
        sch.enqueue(prompts, limits=limits)
        out, guard = {}, 0

        def take(p):
            if p is not None:
                off = p["offsets"].tolist()
                t, l = p["tokens"].tolist(), p["logp"].tolist()
                for i, meta in enumerate(p["metas"]):
                    out[meta] = (t[off[i]:off[i + 1]], l[off[i]:off[i + 1]])
        while len(out) < n and guard < 400:
            guard += 1
            if route == "window":
                p = sch.window(4)
            else:
                sch.run(4)
                p = sch.harvest_packed()
            take(p)
        take(sch.harvest_packed())              # what finished during the last window
        eng.check_status()
        assert not sch._admit_pending and (sch.n_deferred_passes > 0) == beside
        return out, dict(sch.bucket_steps)

    base, b0 = drive("run", False)
    assert len(base) == n and [len(base[i][0]) for i in range(n)] == limits and set(b0) == {B}
    # (beside: admission passes on a second stream next to the steps, requests live one window later)
    for route, compact, beside in (("window", False, False), ("run", True, False), ("window", True, False),
                                   ("window", True, True), ("window", False, True)):
        got, buckets = drive(route, compact, beside)
        assert len(got) == n
        same = np.mean([a == b for i in range(n) for a, b in zip(base[i][0], got[i][0])])
        assert [len(got[i][0]) for i in range(n)] == limits
        if not compact and not beside:
            assert got == base, route           # same kernels on the same rows: bit-identical
        elif not compact:
            assert same > 0.97, (route, same)   # same rows per step, another co-admitted set: GEMM rounding only
        else:
            assert same > 0.97, (route, same)
            assert min(buckets) < B, buckets    # the tail of the job stepped fewer rows


@pytest.mark.parametrize("lanes", [0, 6])
def test_window_harvest_without_admission_passes(lanes):
    """window() on the scheduler modes that admit inside the step kernel (prompts through the decode step, with and
    without prefill lanes): the same rollouts as run + harvest_packed, bit for bit."""
    from ultraviolet_b200.scheduler import GpuScheduler
    spec = gi.model_specs()["tiny_hd64"]
    m = _gpu_model(spec)
    r = np.random.default_rng(41)
    n, B = 40, 8
    prompts = [r.integers(1, m.cfg.vocab_size, r.integers(1, 12)).tolist() for _ in range(n)]
    limits = r.integers(1, 16, n).tolist()

    def drive(route):
        st = m.new_state(GpuScheduler.state_rows(B, lanes, False), 48, ring_extra=GpuScheduler.ring_extra(lanes, 4))
        sch = GpuScheduler(m.engine, st, max_new=16, temperature=0.9, eos_id=None, seed=3, q_cap=64, max_prompt=16,
                           prefill_lanes=lanes, lane_chunk=4)
        sch.enqueue(prompts, limits=limits)
        out = {}
        for _ in range(200):
            if route == "window":
                p = sch.window(4)
            else:
                sch.run(4)
                p = sch.harvest_packed()
            for meta, toks, lps, _v in GpuScheduler.unpack(p):
                out[meta] = (toks, lps.tolist())
            if len(out) == n:
                break
        for meta, toks, lps, _v in sch.harvest():
            out[meta] = (toks, lps.tolist())
        m.engine.check_status()
        return out

    a, b = drive("run"), drive("window")
    assert len(a) == n and a == b


def test_runner_logp_across_graph_bucket_boundaries():
    """DecodeRunner.out_logp is log softmax(out_logits / T)[sampled token] at every step, also on the steps where the
    global-context bucket -- and with it the replayed graph -- changes (the reference's own check,
    tests/test_perf_opt.py:194-222); graph and eager runs draw the same tokens."""
    from ultraviolet_b200.generate import DecodeRunner
    spec = gi.model_specs()["tiny_hd64"]
    m = _gpu_model(spec)
    T, B = 0.9, 4
    res = []
    for graph in (False, True):
        st = m.new_state(B, 80)
        st.set_pos(10)                      # positions 10 .. 49: buckets of 16 change at 16, 32 and 48
        run = DecodeRunner(m, st, bucket=16, use_graph=graph, temperature=T, seed=21)
        tok = torch.arange(1, B + 1, device=DEV)
        toks, buckets = [], set()
        for _ in range(40):
            buckets.add(run.g_len(int(st.host_pos.max())))
            tok = run.step(tok).clone()
            ref = torch.log_softmax(run.out_logits.float() / T, -1).gather(1, tok[:, None])[:, 0]
            assert (run.out_logp - ref).abs().max().item() < 2e-3
            toks.append(tok)
        assert len(buckets) >= 3
        res.append(torch.stack(toks))
    assert torch.equal(res[0], res[1])
