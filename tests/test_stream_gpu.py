"""StreamGen on the GPU scheduler: the reference's own acceptance criteria for the streaming generator
(tests/test_rl_stream.py:82-147): every request comes back exactly once, EOS only as the last token, behaviour
log-probs agree with teacher-forced log-probs, in-place weight sync keeps the arena and tags later admissions."""
import numpy as np
import pytest
import torch

from tests import golden_inputs as gi
from tests.helpers import build_model

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _model():
    spec = gi.model_specs()["tiny"]
    from ultraviolet_b200.fast_decode import patch_model
    m = build_model(spec).to(DEV).to(torch.bfloat16)
    return patch_model(m, "int8")


def _teacher_logp(m, prompt, toks, T):
    """log softmax(logits / T)[tok] of every generated token, one sequence from position 0 (the scheduler's frame)."""
    st = m.new_state(1, len(prompt) + len(toks) + 1)
    seq = list(prompt) + list(toks)
    out = []
    for i, t in enumerate(seq[:-1]):
        lg = m.decode_step(torch.tensor([t], device=DEV), st, st.max_len)
        if i >= len(prompt) - 1:
            lp = torch.log_softmax(lg.float() / T, -1)[0, seq[i + 1]]
            out.append(float(lp))
    return np.array(out, np.float32)


def test_streamgen_contract_and_logprobs():
    from ultraviolet_b200.rl_stream import StreamGen, sync_weights_inplace
    m = _model()
    raw = build_model(gi.model_specs()["tiny"]).to(DEV)
    T, eos, max_new = 1.0, 0, 12
    gen = StreamGen(m, slots=4, max_prompt=9, max_new=max_new, temperature=T, eos_id=eos, check_every=4, seed=3)
    r = np.random.default_rng(0)
    prompts = {i: r.integers(1, 500, r.integers(2, 9)).tolist() for i in range(22)}
    for i in range(12):
        gen.add(prompts[i], meta=i)
    assert gen.n_outstanding() == 12 and len(gen.queue) == 12
    got, chunks = {}, 0
    arena_ptr = m._uvb200_engine.arena.data_ptr()
    while gen.n_outstanding():
        for meta, toks, lp, v0 in gen.chunk():
            assert meta not in got
            got[meta] = (toks, lp, v0)
        chunks += 1
        if chunks == 3:   # a weight sync in the middle: later admissions carry the new version
            sync_weights_inplace(m, raw)
            gen.version += 1
            for i in range(12, 22):
                gen.add(prompts[i], meta=i)
        assert chunks < 400
    assert sorted(got) == list(range(22))
    assert m._uvb200_engine.arena.data_ptr() == arena_ptr
    assert gen.n_tokens == sum(len(t) for t, _, _ in got.values())
    assert gen.n_decode_steps == 4 * chunks and gen.n_active() == 0
    assert {v for _, _, v in got.values()} <= {0, 1} and all(got[i][2] == 1 for i in range(12, 22))
    errs = []
    for i, (toks, lp, _) in got.items():
        assert 1 <= len(toks) <= max_new and len(lp) == len(toks) and lp.dtype == np.float32
        assert eos not in toks[:-1]                      # EOS only as the last token
        assert len(toks) == max_new or toks[-1] == eos   # stopped early only on EOS
        assert np.isfinite(lp).all() and (lp <= 1e-4).all()
        if got[i][2] == 1 and len(errs) < 6:             # generated entirely under the synced weights
            errs.append(np.abs(_teacher_logp(m, prompts[i], toks, T) - lp).mean())
    assert errs and max(errs) < 0.05, errs               # tests/test_rl_stream.py:93: mean |diff| < 0.05


def test_streamgen_is_deterministic_per_request():
    """A request's tokens depend on its Philox key and token index only, not on the slot or on what else is
    running: the same requests through 2 slots and through 5 slots give the same rollouts."""
    from ultraviolet_b200.generate import generate_continuous
    m = _model()
    r = np.random.default_rng(1)
    prompts = [r.integers(1, 500, r.integers(2, 7)).tolist() for _ in range(9)]
    a = generate_continuous(m, prompts, 10, batch=2, temperature=0.8, eos_id=0, seed=5, check_every=3)
    b = generate_continuous(m, prompts, 10, batch=5, temperature=0.8, eos_id=0, seed=5, check_every=8)
    same = np.mean([x == y for x, y in zip(a, b)])
    assert same >= 0.75, (a, b)   # identical unless a bf16 GEMM rounding (batch-size dependent) flips a draw
    c = generate_continuous(m, prompts, 10, batch=5, temperature=0.8, eos_id=0, seed=6, check_every=8)
    assert c != b                 # another seed, another stream


def test_streamgen_with_prefill_lanes_contract():
    """32 slots -> 8 prefill lanes by default: the output contract and the behaviour log-probs hold as without."""
    from ultraviolet_b200.rl_stream import StreamGen
    m = _model()
    T, max_new = 1.0, 8
    gen = StreamGen(m, slots=32, max_prompt=30, max_new=max_new, temperature=T, eos_id=0, check_every=4, seed=9,
                    packed_prefill=False)
    assert gen.sched.L == 8 and not gen.sched.packed
    r = np.random.default_rng(12)
    prompts = {i: r.integers(1, 500, r.integers(2, 31)).tolist() for i in range(48)}
    for i, p in prompts.items():
        gen.add(p, meta=i)
    got = {}
    for _ in range(200):
        for meta, toks, lp, _ in gen.chunk():
            assert meta not in got
            got[meta] = (toks, lp)
        if not gen.n_outstanding():
            break
    assert sorted(got) == list(range(48))
    errs = []
    for i, (toks, lp) in got.items():
        assert 1 <= len(toks) <= max_new and len(lp) == len(toks)
        assert 0 not in toks[:-1] and (len(toks) == max_new or toks[-1] == 0)
        if i % 6 == 0:
            errs.append(np.abs(_teacher_logp(m, prompts[i], toks, T) - lp).mean())
    assert max(errs) < 0.05, errs


def test_streamgen_top_p_stays_in_the_nucleus():
    """With top_p < 1 every drawn token lies in the smallest prefix of the sorted teacher-forced distribution whose
    mass reaches top_p (first token always kept, model.py:1200-1208), and the behaviour log-prob stays the
    UNTRUNCATED one (rl_stream.py:119)."""
    from ultraviolet_b200.rl_stream import StreamGen
    m = _model()
    T, top_p, max_new = 1.0, 0.6, 8
    gen = StreamGen(m, slots=3, max_prompt=6, max_new=max_new, temperature=T, eos_id=0, check_every=4, seed=11,
                    top_p=top_p)
    r = np.random.default_rng(4)
    prompts = {i: r.integers(1, 500, r.integers(2, 6)).tolist() for i in range(6)}
    for i, p in prompts.items():
        gen.add(p, meta=i)
    got = {}
    for _ in range(100):
        for meta, toks, lp, _ in gen.chunk():
            got[meta] = (toks, lp)
        if not gen.n_outstanding():
            break
    assert sorted(got) == list(range(6))
    outside, total, lp_err = 0, 0, []
    for i, (toks, lp) in got.items():
        st = m.new_state(1, len(prompts[i]) + len(toks) + 1)
        seq = list(prompts[i]) + list(toks)
        for j, t in enumerate(seq[:-1]):
            lg = m.decode_step(torch.tensor([t], device=DEV), st, st.max_len)
            if j < len(prompts[i]) - 1:
                continue
            logp = torch.log_softmax(lg.float() / T, -1)[0]
            prob, order = torch.sort(logp.exp(), descending=True)
            keep = int((torch.cumsum(prob, 0) - prob < top_p).sum())   # tokens whose preceding mass is < top_p
            nxt = seq[j + 1]
            total += 1
            outside += int(nxt not in order[:keep + 1].tolist())       # one slack entry for bf16 ties at the edge
            lp_err.append(abs(float(logp[nxt]) - float(lp[j - len(prompts[i]) + 1])))
    assert total >= 12 and outside == 0, (outside, total)
    assert np.mean(lp_err) < 0.05


def test_fused_sample_api():
    from ultraviolet_b200.kernels import fused_sample, fused_sample_ok
    x = torch.randn(5, 16384, device=DEV).half()
    u = torch.rand(5, device=DEV)
    assert fused_sample_ok(x, 16384, (23.0, 5.0, 7.5), 1.0) and not fused_sample_ok("cpu", 16384, (23.0, 5.0, 7.5), 1.0)
    tok, lp = fused_sample(x, u, (23.0, 5.0, 7.5), 1.0)
    assert tok.dtype == torch.int64 and lp.dtype == torch.float32 and tok.shape == (5,) and bool((lp < 0).all())


def test_grpo_group_of_identical_prompts_gets_distinct_streams():
    """The GRPO rollout shape (scripts/rl_grpo.py:1181: every prompt is sampled `group` times): 8 copies of one
    prompt carry 8 Philox keys, so they produce 8 different rollouts, and a copy's rollout depends on its key alone --
    the same (seed, request order) through another slot count, with and without prefill lanes, gives the same
    rollouts."""
    from ultraviolet_b200.rl_stream import StreamGen
    m = _model()
    r = np.random.default_rng(21)
    base = [r.integers(1, 500, r.integers(3, 9)).tolist() for _ in range(3)]
    reqs = [(p, (gi_, c)) for gi_, p in enumerate(base) for c in range(8)]      # 3 groups of 8

    def rollouts(slots, lanes, packed, overlap=False):
        gen = StreamGen(m, slots=slots, max_prompt=9, max_new=10, temperature=1.2, eos_id=0, check_every=4, seed=77,
                        prefill_lanes=lanes, packed_prefill=packed, overlap_harvest=overlap, warm=overlap)
        assert gen.sched.packed == packed
        for p, meta in reqs:
            gen.add(p, meta)
        got = {}
        while gen.n_outstanding():
            for meta, toks, lp, v0 in gen.chunk():
                assert meta not in got and len(toks) == len(lp) and v0 == 0
                got[meta] = toks
        return got

    a = rollouts(4, 0, True)       # packed admission passes (the default)
    assert sorted(a) == sorted(meta for _, meta in reqs)
    for g_ in range(3):
        assert len({tuple(a[(g_, c)]) for c in range(8)}) >= 7     # identical prompts, different keys: different text
    b = rollouts(24, 0, True)
    a2 = rollouts(4, 0, True, overlap=True)    # harvest overlapped with the next chunk's steps
    assert sorted(a2) == sorted(a)
    c = rollouts(7, 4, False)      # prompts through the decode step, with lanes ...
    d = rollouts(5, 0, False)      # ... and one token per step
    for x, y in ((a, b), (a, a2), (c, d), (a, d)):
        same = np.mean([x[k] == y[k] for k in x])
        assert same >= 0.75, same    # equal unless a bf16 rounding (batch size, prefill route) flips a draw


def test_device_handoff_of_a_real_harvest_and_direct_weight_publication():
    """harvest_packed(with_prompts=True) -> build_packed_device: the micro-batches hold exactly the prompts,
    generated tokens and behaviour log-probs of the finished rollouts, all on the device.  publish_weights writes the
    trainer's parameters straight into the arena (same arena contents as sync_weights_inplace, same pointer)."""
    from ultraviolet_b200.handoff import build_packed_device
    from ultraviolet_b200.rl_stream import StreamGen, publish_weights, sync_weights_inplace
    m = _model()
    gen = StreamGen(m, slots=6, max_prompt=9, max_new=12, temperature=1.0, eos_id=0, check_every=4, seed=5)
    r = np.random.default_rng(4)
    prompts = {i: r.integers(1, 500, r.integers(2, 9)).tolist() for i in range(15)}
    for i, p in prompts.items():
        gen.add(p, meta=i)
    gen._upload()
    seen = {}
    for _ in range(200):
        gen._upload()
        gen.sched.run(4)
        p = gen.sched.harvest_packed(with_prompts=True)
        if p is None:
            if len(seen) == len(prompts):
                break
            continue
        assert p["tokens"].is_cuda and p["prompt_tokens"].is_cuda
        adv = [float(mm) + 1 for mm in p["metas"]]
        for mb in build_packed_device(p, adv, budget=64, pad_id=0, seg_max=16):
            assert mb["x"].is_cuda and mb["x"].shape == (1, 64) and int(mb["cu"][-1]) == 64
            x, y, A, OL, cu = (mb[k].cpu().numpy() for k in ("x", "y", "A", "OL", "cu"))
            for a, b in zip(cu[:-1], cu[1:]):
                if A[0, a] <= 0:
                    continue          # a pad segment
                i = int(A[0, a]) - 1
                pr = prompts[i]
                n_gen = (b - a) + 1 - len(pr)
                assert list(x[0, a:a + len(pr)]) == pr and (y[0, a:a + len(pr) - 1] == -1).all()
                gen_toks = list(y[0, a + len(pr) - 1:b])
                assert len(gen_toks) == n_gen and i not in seen
                seen[i] = (gen_toks, OL[0, a + len(pr) - 1:b].copy())
    assert sorted(seen) == sorted(prompts)
    for i, (toks, lps) in seen.items():
        assert 1 <= len(toks) <= 12 and (lps < 0).all() and (0 not in toks[:-1])
    # direct publication == the reference-style sync, same arena pointer
    raw = build_model(gi.model_specs()["tiny"]).to(DEV)
    with torch.no_grad():
        raw.blocks[1].mlp.w_down.mul_(1.5)
    eng = m._uvb200_engine
    ptr, v0 = eng.arena.data_ptr(), eng.version
    publish_weights(m, raw)
    a = eng.arena.clone()
    sync_weights_inplace(m, raw)
    assert eng.arena.data_ptr() == ptr and torch.equal(a, eng.arena) and eng.version == v0 + 2


def _uv50m():
    from ultraviolet_b200.model import MathLM, make_config
    torch.manual_seed(0)
    m = MathLM(make_config("uv-50m-alpha", vocab_size=16384))
    return m.to(DEV).to(torch.bfloat16).fuse_for_inference(torch.bfloat16)


def test_continuous_batching_job_at_full_size_properties():
    """The continuous-batching benchmark job at its full size (UV-50M, 4096 requests, prompts U[16,256], stop length
    ~ Geometric(600) <= 2048 with EOS forced there, 512 slots, T = 1) through the device scheduler with admission
    passes, slot compaction and the overlapped harvest.  Too large for the oracle, so size-independent properties:
    every request comes back exactly once; it ends with EOS and holds no EOS before its end; it is no longer than its
    stop length and exactly that long unless the model drew EOS earlier (rare: a 1-in-16384 event per token); one
    finite log-prob <= 0 per token; the device counters agree with the payload; compaction really shrank the step;
    nothing flagged a failure."""
    from ultraviolet_b200.scheduler import GpuScheduler
    r = np.random.default_rng(3)
    n, slots, max_prompt, max_new, V = 4096, 512, 256, 2048, 16384
    lens = r.integers(16, max_prompt + 1, n)
    stops = np.minimum(r.geometric(1.0 / 600.0, n), max_new)
    prompts = [r.integers(1, V, int(L)).tolist() for L in lens]
    m = _uv50m()
    st = m.new_state(GpuScheduler.state_rows(slots, 0, True), max_prompt + max_new + 16)
    sch = GpuScheduler(m.engine, st, max_new=max_new, temperature=1.0, eos_id=0, seed=7, q_cap=n, max_prompt=max_prompt,
                       force_eos=True, tok_cap=int(lens.sum()) + 1, out_cap=int(stops.sum()) + 1, packed_prefill=True)
    sch.warm()
    sch.enqueue(prompts, limits=stops.tolist())
    got, windows = {}, 0
    while len(got) < n and windows < 400:
        windows += 1
        for meta, toks, lps, ver in sch.unpack(sch.window(32)):
            assert meta not in got
            got[meta] = (toks, lps, ver)
    for meta, toks, lps, ver in sch.harvest():
        assert meta not in got
        got[meta] = (toks, lps, ver)
    assert sorted(got) == list(range(n))
    early = 0
    for i in range(n):
        toks, lps, ver = got[i]
        assert 1 <= len(toks) <= stops[i] and len(lps) == len(toks) and ver == 0
        assert toks[-1] == 0 and 0 not in toks[:-1]
        assert np.isfinite(lps).all() and (lps <= 0).all()
        early += len(toks) < stops[i]
    assert early < 0.08 * n, early          # expected about 0.035 n early stops
    c = sch.counters()
    total = sum(len(got[i][0]) for i in range(n))
    assert c["generated"] == total and c["finished"] == n and c["head"] == n and c["status"] == 0
    # a slot is counted as occupied after every step it survives: all of a request's tokens but its last
    assert c["slot_steps"] == total - n and min(sch.bucket_steps) < slots
    assert m.engine.device_status() == {"attn_status": 0, "kv_oob": 0}


def test_grpo_round_at_full_size_properties():
    """The GRPO benchmark round at its full size (256 prompts U[64,256] x group 8 = 2048 sequences, max_new 2048,
    T = 1, one Philox key per sequence): every sequence comes back once with at most max_new tokens, EOS only as a
    last token; the 8 members of a group share a prompt and differ in their text (distinct keys); members of a group
    agree on their FIRST token's log-prob distribution support (same prompt, same weights: the first log-prob is the
    log-probability of a token under one and the same distribution, so equal first tokens carry equal log-probs)."""
    from ultraviolet_b200.scheduler import GpuScheduler
    r = np.random.default_rng(5)
    lens = r.integers(64, 257, 256)
    base = [r.integers(1, 16384, int(L)).tolist() for L in lens]
    prompts = [p for p in base for _ in range(8)]
    n, slots, max_new = len(prompts), 512, 2048
    m = _uv50m()
    st = m.new_state(GpuScheduler.state_rows(slots, 0, True), 256 + max_new + 16)
    sch = GpuScheduler(m.engine, st, max_new=max_new, temperature=1.0, eos_id=0, seed=11, q_cap=n, max_prompt=256,
                       tok_cap=sum(len(p) for p in prompts) + 1, out_cap=n * max_new + 1, packed_prefill=True)
    sch.warm()
    sch.enqueue(prompts, keys=list(range(n)))
    got, windows = {}, 0
    while len(got) < n and windows < 400:
        windows += 1
        for meta, toks, lps, ver in sch.unpack(sch.window(32)):
            got[meta] = (toks, lps)
    for meta, toks, lps, ver in sch.harvest():
        got[meta] = (toks, lps)
    assert sorted(got) == list(range(n))
    for i in range(n):
        toks, lps = got[i]
        assert 1 <= len(toks) <= max_new and len(lps) == len(toks)
        assert 0 not in toks[:-1] and (len(toks) == max_new or toks[-1] == 0)
        assert np.isfinite(lps).all() and (lps <= 0).all()
    for g in range(256):
        members = [got[8 * g + c] for c in range(8)]
        assert len({tuple(t[:64]) for t, _ in members}) == 8, g       # 8 keys, 8 different continuations
        first = {}
        for t, l in members:                                          # same first token -> same log-prob (bf16 GEMMs
            first.setdefault(t[0], []).append(float(l[0]))            # at one batch size: up to rounding)
        for v in first.values():
            assert max(v) - min(v) < 0.05, (g, v)
    assert m.engine.device_status() == {"attn_status": 0, "kv_oob": 0}
