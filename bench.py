#!/usr/bin/env python
"""Benchmark of the UV-50M rollout-decode path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload fixed|continuous|attn] [--impl reference]

Default workload ("fixed"): UV-50M (uv-50m-alpha preset, vocab 16384, random init seed 0, bf16 weights, int8 KV)
decoding 256 concurrent sequences per GPU, prompts uniform in [32, 128] tokens, greedy, no retirement.  One STEP is
one decode step of the whole batch (256 tokens per GPU); K defaults to 512 = the configuration's max_new.
Under torchrun every rank runs its own replica on its own 256 sequences (weak scaling, no collective inside a step);
the bf16 weight arena is NCCL-broadcast from rank 0 before the rollout and the generated tokens are gathered to rank 0
after it (both timed separately and reported in "config").

Prints ONE JSON line (rank 0).  `value` is device-resident throughput (inputs already in HBM); `e2e` is the same
metric through the public step API with pinned-host token buffers copied in and out every step.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

VOCAB = 16384
SLOTS = 256
PROMPT_LO, PROMPT_HI = 32, 128
# DRAM bytes (read + write) per launch of attn_split_kernel divided by its algorithmic bytes, from the ncu captures
# summarised under profiles/ (traffic grows in proportion to the keys read, so the ratio scales to any launch)
NCU_TRAFFIC_RATIO = {"long_context": 1.013, "step": 0.993}


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


# ------------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every interval_ms while the timed region runs (read-only)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int, interval_ms: int = 200):
        self.index, self.rows, self.proc, self.interval_ms = index, [], None, int(interval_ms)

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", str(self.interval_ms), "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc is not None:
            time.sleep(0.25)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except Exception:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------ workload pieces
def make_prompts(n, lo, hi, seed):
    r = np.random.default_rng(seed)
    lens = r.integers(lo, hi + 1, n)
    return [r.integers(1, VOCAB, int(L)).tolist() for L in lens]


def build_model(device, dtype):
    import torch
    from ultraviolet_b200.model import MathLM, make_config
    torch.manual_seed(0)
    m = MathLM(make_config("uv-50m-alpha", vocab_size=VOCAB))
    return m.to(device).to(dtype).fuse_for_inference(dtype)


def attn_bytes(pos, starts, window, S=None, ring=False):
    """Algorithmic bytes of one attention launch: 132 per attended key + q in and out."""
    p, s = np.asarray(pos, np.int64), np.asarray(starts, np.int64)
    lo = np.maximum(s, 0)
    if window:
        lo = np.maximum(lo, p - window + 1)
    if ring and S:
        lo = np.maximum(lo, p - S + 1)
    return int(np.maximum(p + 1 - lo, 0).sum()) * 132 + 2 * len(p) * 8 * 64 * 2


def graph_ms(body, reps=5):
    """Median device time (ms, CUDA events on the launching stream) of one replay of `body` captured as a CUDA
    graph: launches are enqueued back to back by the device, not paced by the host."""
    import torch
    body()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        body()
    g.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    return float(np.median(ts))


def cupti_kernel_times(replay, n=20):
    """Per-kernel device time of `replay()` (a CUDA-graph replay) from CUPTI activity records (torch.profiler with
    the CUDA activity only): kernels run back to back as in the real step, not serialised as under ncu.  Returns
    {"kernels": {name: {"per_replay": launches, "us_each": mean duration}}, "kernel_us_per_replay": sum of kernel
    time, "replay_us": wall time of a replay by CUDA events without the profiler}."""
    import collections
    import torch
    from torch.profiler import ProfilerActivity, profile
    replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        replay()
    e1.record()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(n):
            replay()
        torch.cuda.synchronize()
    agg = collections.defaultdict(lambda: [0, 0.0])
    for ev in prof.events():
        if (ev.device_type == torch.autograd.DeviceType.CUDA and ev.name and "Memcpy" not in ev.name
                and "Memset" not in ev.name):
            k = ev.name.split("(")[0][:72]
            agg[k][0] += 1
            agg[k][1] += ev.device_time
    kernels = {k: {"per_replay": c / n, "us_each": round(t / c, 2)} for k, (c, t) in
               sorted(agg.items(), key=lambda kv: -kv[1][1])}
    return {"kernels": kernels, "kernel_us_per_replay": round(sum(t for _, t in agg.values()) / n, 1),
            "replay_us": round(e0.elapsed_time(e1) * 1e3 / n, 1)}


def time_attention_layers(eng, st, pos, starts, rounds=4):
    """Average device time of one decode-attention launch at the cache state of the run, per layer kind, exactly as
    the step issues it (XSA + precomputed head gates in the epilogue).  The run's own layer caches plus clones of
    them -- together more than L2 holds -- are visited in turn inside one CUDA graph, so every launch reads its KV
    bytes from HBM as it does inside a real step (where 100 MB of weights pass through L2 between two visits of a
    layer's cache).  No flush, no subtraction: graph time / launches."""
    import torch
    from ultraviolet_b200 import _lib
    from ultraviolet_b200.kernels.decode_attn import attn_args, attn_launch, default_splits
    cfg, B = eng.cfg, st.B
    s = eng.scratch(B)
    qkv3 = s["qkv"].view(B, cfg.n_heads + 2 * cfg.n_kv_heads, cfg.head_dim)
    q, out = qkv3[:, :cfg.n_heads], s["z"].view(B, cfg.n_heads, cfg.head_dim)
    v_cur = qkv3[:, cfg.n_heads + cfg.n_kv_heads:]
    gates = s["gate"]
    res = {}
    for kind in ("global", "local"):
        layers = [l for l in range(cfg.n_layers) if cfg.is_global(l) == (kind == "global")]
        S = st.k[layers[0]].size(2)
        ctx = S if kind == "local" else min(int(pos.max().item()) + 1, S)
        splits = default_splits(B * cfg.n_kv_heads, ctx, eng.device)
        window, ring = (0, False) if kind == "global" else (cfg.window, True)
        ws = eng._workspace(s, B, splits)
        bufs = [(st.k[l], st.v[l], st.k_scale[l], st.v_scale[l]) for l in layers]
        per = sum(t.numel() * t.element_size() for t in bufs[0])
        while per * len(bufs) < (160 << 20):
            # clones keep the padded row allocation of the originals (slices of a clone of the full storage)
            k0, v0, ks0, vs0 = bufs[len(bufs) % len(layers)]
            bufs.append(tuple(_clone_like(t) for t in (k0, v0, ks0, vs0)))
        kw = dict(v_cur=v_cur, xsa_alpha=eng.xsa[layers[0]] if cfg.xsa else None, xsa_eps=cfg.xsa_eps,
                  gate_vals=gates if cfg.gate_channels else None, counters=s["counters"], status=s["status"])

        def run():
            for _ in range(rounds):
                for k, v, ks, vs in bufs:
                    attn_launch(q, k, v, pos, starts, cfg.attn_scale, window, ring, ks, vs, splits, out, ws, **kw)
        ms = graph_ms(run) / (rounds * len(bufs))
        byt = attn_bytes(pos.cpu().numpy(), starts.cpu().numpy(), window if kind == "local" else 0, S, ring)
        a = attn_args(q, *bufs[0][:2], pos, starts, cfg.attn_scale, window, ring, *bufs[0][2:], splits, out, ws)
        path = "bulk-copy (TMA) tiles" if _lib.lib().uv_decode_attn_uses_bulk(a) == 1 else "cp.async tiles"
        res[kind] = {"ms": ms, "bytes": byt, "gbs": byt / ms / 1e6, "launches_per_step": len(layers),
                     "splits": splits, "slots_per_row": S, "path": path, "cache_copies_visited": len(bufs)}
    return res


def _clone_like(t):
    """A copy of a (B, K, S, ...) cache tensor inside an allocation with the same (possibly padded) row length."""
    import torch
    inner = t.stride(2)
    alloc = t.stride(1) // inner
    full = torch.empty((t.size(0), t.size(1), alloc) + tuple(t.shape[3:]), dtype=t.dtype, device=t.device)
    out = full[:, :, :t.size(2)]
    out.copy_(t)
    return out


def long_context_attention(eng, rounds=4, ctx=8192):
    """The long-context stress shape: 64 sequences with 8192 int8 keys each, one global-layer launch per cache copy
    (three 69 MB copies visited in turn: more than L2 holds), captured in a CUDA graph."""
    import torch
    from ultraviolet_b200.kernels.decode_attn import attn_launch, default_splits, workspace_for
    dev, B, S, H, hd = eng.device, 64, ctx + 256, 8, 64
    g = torch.Generator(device=dev).manual_seed(1)
    bufs = []
    for _ in range(3):
        bufs.append((torch.randint(-127, 128, (B, 1, S, hd), device=dev, dtype=torch.int8, generator=g),
                     torch.randint(-127, 128, (B, 1, S, hd), device=dev, dtype=torch.int8, generator=g),
                     (torch.rand(B, 1, S, device=dev, generator=g) * 0.02 + 0.01).half(),
                     (torch.rand(B, 1, S, device=dev, generator=g) * 0.02 + 0.01).half()))
    q = torch.randn(B, H, hd, device=dev, generator=g).to(eng.dtype)
    pos = torch.full((B,), ctx - 1, device=dev, dtype=torch.long)
    st0 = torch.zeros(B, device=dev, dtype=torch.long)
    out = torch.empty_like(q)
    splits = default_splits(B, ctx, dev)
    ws = workspace_for(B, 1, H, hd, splits, dev)
    cnt = torch.zeros(B, dtype=torch.int32, device=dev)

    def run():
        for _ in range(rounds):
            for k, v, ks, vs in bufs:
                attn_launch(q, k, v, pos, st0, 0.14125, 0, False, ks, vs, splits, out, ws, counters=cnt)
    ms = graph_ms(run) / (rounds * len(bufs))
    byt = B * ctx * 132 + 2 * B * H * hd * 2
    return {"ms": ms, "bytes": byt, "gbs": byt / ms / 1e6, "splits": splits}


# ------------------------------------------------------------------------------------------------ CPU baseline
def step_shape_attention(eng, rounds=4):
    """The attention launch of a local layer as the fixed-batch decode step issues it, in isolation: 256 rows, ring
    cache of 256 slots, window 256, positions U[131, 323], XSA + precomputed head gates in the epilogue.  Sixteen
    cache copies (138 MB, more than L2) are visited in turn inside one CUDA graph."""
    import torch
    from ultraviolet_b200.kernels.decode_attn import attn_launch
    dev, B, S, H, hd = eng.device, SLOTS, 256, 8, 64
    g = torch.Generator(device=dev).manual_seed(2)
    bufs = []
    for _ in range(16):
        bufs.append((torch.randint(-127, 128, (B, 1, S, hd), device=dev, dtype=torch.int8, generator=g),
                     torch.randint(-127, 128, (B, 1, S, hd), device=dev, dtype=torch.int8, generator=g),
                     (torch.rand(B, 1, S, device=dev, generator=g) * 0.02 + 0.01).half(),
                     (torch.rand(B, 1, S, device=dev, generator=g) * 0.02 + 0.01).half()))
    q = torch.randn(B, H, hd, device=dev, generator=g).to(eng.dtype)
    v_cur = torch.randn(B, 1, hd, device=dev, generator=g).to(eng.dtype)
    gates = torch.rand(B, H, device=dev, generator=g) * 2
    alpha = torch.tanh(torch.randn(H, device=dev, generator=g) * 0.3)
    pos = torch.randint(131, 324, (B,), device=dev, generator=g)
    st0 = torch.zeros(B, device=dev, dtype=torch.long)
    out = torch.empty_like(q)

    def run():
        for _ in range(rounds):
            for k, v, ks, vs in bufs:
                attn_launch(q, k, v, pos, st0, 0.14125, 256, True, ks, vs, 1, out, None, v_cur=v_cur,
                            xsa_alpha=alpha, gate_vals=gates)
    ms = graph_ms(run) / (rounds * len(bufs))
    n = torch.clamp(pos + 1, max=256).sum().item()
    byt = int(n) * 132 + 2 * B * H * hd * 2
    return {"ms": ms, "bytes": byt, "gbs": byt / ms / 1e6, "splits": 1}


def workload_config(K: int) -> dict:
    """The workload both arms run (identical dictionaries in the two JSON lines)."""
    return {"workload": "UV-50M fixed-batch decode (benchmark configuration 2): 256 sequences/GPU, prompts U[32,128] of "
                        "uniform token ids, greedy, int8 KV, decode steps after prefill (step = 256 tokens/GPU)",
            "slots_per_gpu": SLOTS, "vocab": VOCAB, "weights": "random init seed 0",
            "prompts": "numpy default_rng(100 + rank): lengths then ids"}


def port_decode_tokens_per_s(n_steps: int, slots: int = SLOTS, ctx: int = 160, seed: int = 0):
    """Fallback when oracle/_ref is not installed: the numpy restatement's int8-KV decode step on the host cores
    (random-filled cache at context ~ctx).  Returns (tokens/s, seconds, threads)."""
    import torch
    from oracle import model as om
    from ultraviolet_b200.model import MathLM, make_config
    torch.manual_seed(0)
    m = MathLM(make_config("uv-50m-alpha", vocab_size=VOCAB))
    params = {k: om.round_bf16(v.detach().float().numpy()) for k, v in m.state_dict().items()}
    W = om.fuse_weights(params, m.cfg, "bf16")
    st = om.State(m.cfg, slots, ctx + n_steps + 2)
    r = np.random.default_rng(seed)
    for l in range(m.cfg.n_layers):
        for c in (st.k[l], st.v[l]):
            c[...] = r.integers(-127, 128, c.shape, dtype=np.int8)
        for c in (st.k_scale[l], st.v_scale[l]):
            c[...] = (r.random(c.shape) * 0.02 + 0.01).astype(np.float16)
    st.pos[:] = r.integers(ctx - 48, ctx + 1, slots)
    tok = r.integers(1, VOCAB, slots)
    om.decode_step(W, m.cfg, tok, st)  # warm the BLAS threads
    t0 = time.perf_counter()
    for _ in range(n_steps):
        tok = om.sample_greedy(om.decode_step(W, m.cfg, tok, st))
    dt = time.perf_counter() - t0
    return slots * n_steps / dt, dt, os.cpu_count()


def cpu_baseline(n_steps: int, warmup: int = 1) -> dict:
    """The reference's own CPU decode route (oracle/_ref: MathLM prefill + decode_step_fast with the attention call
    bound to decode_attention_ref, fp32 torch, every host thread) on the GPU arm's rank-0 prompts; the numpy port
    only when the reference is not installed.  Returns the cpu_baseline object plus seconds per step."""
    from oracle import ref_arm
    if ref_arm.available():
        r = ref_arm.cpu_decode(make_prompts(SLOTS, PROMPT_LO, PROMPT_HI, seed=100), n_steps, warmup, vocab=VOCAB)
        return {"value": r["tokens_per_s"], "unit": "tokens/s", "cores": r["threads"], "kind": "reference",
                "sample": f"{n_steps} greedy decode steps of the same 256 prompts after the reference's own prefill "
                          f"({r['prefill_s']:.1f} s, not timed), mean context {r['context']:.0f}: ultraviolet "
                          "decode_step_fast + decode_attention_ref, fp32 torch on "
                          f"{r['threads']} threads ({r['seconds']:.1f} s timed)",
                "ms_per_step": r["seconds"] / n_steps * 1e3}
    v, dt, threads = port_decode_tokens_per_s(n_steps)
    return {"value": v, "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": f"{n_steps} decode steps of 256 sequences at context ~160 (numpy fp32 restatement, BLAS threads; "
                      f"oracle/_ref not installed) ({dt:.1f} s)", "ms_per_step": dt / n_steps * 1e3}


def reference_gpu_attention() -> dict:
    """Second comparator: the reference's own GPU kernels (Triton, NVRTC) for the attention step on this GPU."""
    try:
        import torch
        from oracle import ref_arm
        if not (torch.cuda.is_available() and ref_arm.available()):
            return {"unavailable": "no CUDA device or oracle/_ref not installed"}
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
        return ref_arm.gpu_attention()
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"{type(e).__name__}: {str(e)[:300]}"}


def reference_gpu_attention_subprocess(timeout_s: int = 300) -> dict:
    """The same, run as `bench.py --impl reference --reference-gpu-only` in a child process so that a kernel of the
    reference that fails to compile or run here cannot take this process down."""
    try:
        r = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference", "--reference-gpu-only"],
                           capture_output=True, text=True, timeout=timeout_s)
        for ln in reversed(r.stdout.strip().splitlines()):
            if ln.startswith("{"):
                return json.loads(ln)
        return {"unavailable": f"no output (rc {r.returncode}): {r.stderr[-300:]}"}
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"{type(e).__name__}: {str(e)[:200]}"}


def run_reference_arm(args, rank, world):
    """`--impl reference`: the reference's own CPU implementation of the path on the host cores (rank 0 only)."""
    if rank != 0:
        return
    if args.reference_gpu_only:
        print(json.dumps(reference_gpu_attention()), flush=True)
        return
    steps = max(1, min(args.steps, 64))  # bounded sample: the timed part stays within ~10 s of host work
    cb = cpu_baseline(steps, warmup=max(1, min(args.warmup, 3)))
    v = cb["value"]
    line = {"impl": "reference", "metric": "rollout decode tokens/s", "value": v, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": cb.pop("ms_per_step"),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
            "config": workload_config(args.steps), "cpu_baseline": cb,
            "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    if args.reference_gpu:
        line["attention_reference_gpu"] = reference_gpu_attention()
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------ GEMM micro-benchmark
def run_gemm_workload(args, dev):
    """`--workload gemm`: the four GEMM shapes of a layer at `--rows` batch rows, as dependent launches inside one
    CUDA graph over rotating weight copies: library GEMM alone, library GEMM + the row kernel that follows it in the
    step, and this library's fused-epilogue tcgen05 kernel in several tilings (batch tile, split-K).  Microseconds
    per launch (or per pair)."""
    import torch
    from ultraviolet_b200 import _lib
    L, lib = _lib, _lib.lib()
    sp = lambda: torch.cuda.current_stream().cuda_stream
    M, NW = args.rows, 20
    d, f = 640, 1664
    lam = torch.tensor([0.9, 1.1], device=dev)
    res = {}
    for name, N, K, cfgs in (("qkv", 640, 640, ((32, 1), (32, 2), (32, 4), (64, 2), (64, 4))),
                             ("wo", 640, 512, ((32, 1), (32, 2), (32, 4), (64, 4))),
                             ("down", 640, 1664, ((32, 2), (32, 4), (64, 4), (64, 8))),
                             ("gate_up", 2 * f, 640, ((32, 1), (64, 1), (128, 1)))):
        ws = [(torch.randn(N, K, device=dev) * 0.05).bfloat16() for _ in range(NW)]
        x = torch.randn(M, K, device=dev).bfloat16()
        c = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        xr = torch.randn(M, d, device=dev).bfloat16()
        h, hn = torch.empty_like(xr), torch.empty_like(xr)
        ss = torch.ones(d // 128, M, device=dev)
        act = torch.empty(M, f, device=dev, dtype=torch.bfloat16)

        def lib_chain():
            for w in ws:
                torch.mm(x, w.t(), out=c)
        res[name + ".library"] = graph_ms(lib_chain) * 1e3 / NW
        if name in ("wo", "down"):
            def acc_chain():
                for w in ws:
                    xr.addmm_(x, w.t())
            res[name + ".library_accumulate"] = graph_ms(acc_chain) * 1e3 / NW

            def pair():
                for w in ws:
                    torch.mm(x, w.t(), out=c)
                    lib.uv_resid_norm(xr.data_ptr(), c.data_ptr(), lam.data_ptr(), 2, d, h.data_ptr(), hn.data_ptr(), M,
                                      sp())
            res[name + ".library+resid_norm"] = graph_ms(pair) * 1e3 / NW
        if name == "gate_up":
            def pair():
                for w in ws:
                    torch.mm(x, w.t(), out=c)
                    lib.uv_swiglu(c.data_ptr(), 2, f, act.data_ptr(), M, sp())
            res[name + ".library+swiglu"] = graph_ms(pair) * 1e3 / NW

            def pair2():
                for w in ws:
                    torch.mm(x, w.t(), out=c)
                    lib.uv_swiglu_rs(c.data_ptr(), x.data_ptr(), 2, d, f, act.data_ptr(), M, sp())
            res[name + ".library+swiglu_rs"] = graph_ms(pair2) * 1e3 / NW
        for bn, ks in cfgs:
            if name in ("wo", "down"):
                def own():
                    for w in ws:
                        L.check(lib.uv_gemm_sw_resid(x.data_ptr(), K, w.data_ptr(), xr.data_ptr(), lam.data_ptr(),
                                                     h.data_ptr(), d, ss.data_ptr(), M, 2, M, N, K, bn, ks, None, sp()),
                                "uv_gemm_sw_resid")
            elif name == "gate_up":
                def own():
                    for w in ws:
                        L.check(lib.uv_gemm_sw_swiglu(x.data_ptr(), K, w.data_ptr(), act.data_ptr(), 2, M, K, f,
                                                      ss.data_ptr(), d // 128, M, bn, None, sp()), "uv_gemm_sw_swiglu")
            else:
                def own():
                    for w in ws:
                        L.check(lib.uv_gemm_sw(x.data_ptr(), K, w.data_ptr(), c.data_ptr(), N, 2, M, N, K,
                                               ss.data_ptr(), d // 128, M, bn, ks, None, sp()), "uv_gemm_sw")
            res[f"{name}.own_fused.bn{bn}.ks{ks}"] = graph_ms(own) * 1e3 / NW
    print(json.dumps({"metric": "GEMM us per launch", "rows": M, "pdl": os.environ.get("UVDECODE_PDL", "0"),
                      "unit": "us", "config": {"workload": "decode-step GEMM shapes, dependent launches in a CUDA "
                                                            "graph, 20 rotating weight copies"},
                      "us_per_launch": {k: round(v, 2) for k, v in res.items()}}), flush=True)


# ------------------------------------------------------------------------------------------------ rollout jobs
def rollout_job(m, rank, world, dev, *, prompts_all, stops_all, slots, max_new, max_prompt, lanes, lane_chunk, seed,
                force_eos, timed_steps=0, warmup=3, broadcast=False, gather=False, packed=True, compact=True, overlap=True,
                kernel_times=False, overlap_admit=False, window=0):
    """One rollout round on the device-resident scheduler: the requests are sharded i % W == rank, every rank runs
    its replica until its share is drained (timed_steps > 0: that many steps only), finished rollouts are harvested
    as device tensors.  Optionally the weight arena is broadcast from rank 0 first and the rollouts (tokens int32,
    log-probs fp32, lengths and start versions int32) are gathered to rank 0 afterwards, each collective timed.
    overlap: each window of steps is launched before the payload of the requests that finished in the window before
    it is gathered (GpuScheduler.window), so the device does not wait for the host's harvest.
    Windows of 32 (packed admission) or 64 steps are timed separately so that the steady state (slot occupancy >=
    0.95) can be told from the
    straggler tail.  Returns a dict on every rank (aggregates are all-reduced)."""
    import torch
    import torch.distributed as dist
    from ultraviolet_b200 import dist as uvdist
    from ultraviolet_b200.scheduler import GpuScheduler
    eng = m.engine
    n_req = len(prompts_all)
    mine = uvdist.shard_requests(n_req, rank, world)
    t_bcast = uvdist.broadcast_weights(eng) if (world > 1 and broadcast) else 0.0
    lens = np.array([len(p) for p in prompts_all])
    lim = np.full(n_req, max_new) if stops_all is None else np.asarray(stops_all)
    if packed:
        lanes = 0
    st = m.new_state(GpuScheduler.state_rows(slots, lanes, packed), max_prompt + max_new + 16,
                     ring_extra=GpuScheduler.ring_extra(lanes, lane_chunk))
    sch = GpuScheduler(eng, st, max_new=max_new, temperature=1.0, eos_id=0, seed=seed, q_cap=max(len(mine), 2),
                       max_prompt=max_prompt, force_eos=force_eos, tok_cap=int(lens[mine].sum()) + 1,
                       out_cap=int(lim[mine].sum()) + 1, prefill_lanes=lanes, lane_chunk=lane_chunk,
                       packed_prefill=packed, compact=compact, overlap_admit=overlap_admit and overlap)
    # steps between harvests (= between admission passes in packed mode: a pass costs 0.4-0.9 ms whatever it admits,
    # a freed slot idles half a window on average; 32 measured best of 16 / 24 / 32 / 48 on config 3)
    W_STEPS = window or (32 if packed else 64)
    sch.warm()                       # every step / admission graph captured before the job, as a server would
    sch.enqueue([prompts_all[i] for i in mine], limits=None if stops_all is None else lim[mine].tolist(), keys=mine,
                metas=mine)
    sch.run(max(warmup, 3))
    torch.cuda.synchronize()
    c_prev = c0 = sch.counters()
    if world > 1:
        dist.barrier()
    harvested, windows, steps, n_done = [], [], 0, 0
    ev = lambda: torch.cuda.Event(enable_timing=True)
    e_begin, e_end = ev(), ev()
    clk = ClockSampler(dev.index if dev.index is not None else 0)
    clk.__enter__()
    e_begin.record()
    last = None   # (start event, end event, steps) of the window in flight

    def close_window(c):
        nonlocal c_prev
        a_, b_, n_ = last
        windows.append((a_.elapsed_time(b_), c["generated"] - c_prev["generated"],
                        (c["slot_steps"] - c_prev["slot_steps"]) / (n_ * slots)))
        c_prev = c
    while True:
        n = W_STEPS if timed_steps <= 0 else min(W_STEPS, timed_steps - steps)
        a, b = ev(), ev()
        a.record()
        # launches the window, then gathers -- while it runs -- what had finished when it was launched; the
        # counters it read (one small D2H, which waited for the window before) close that window's record
        p = sch.window(n) if overlap else sch.run(n)
        b.record()
        steps += n
        if overlap:
            if last is not None:
                close_window(sch.counters(cached=True))
            last = (a, b, n)
        else:
            p = sch.harvest_packed()      # syncs: the window's events are complete after it
            last = (a, b, n)
            close_window(sch.counters())
        if p is not None:
            harvested.append(p)
            n_done += len(p["metas"])
        if (timed_steps > 0 and steps >= timed_steps) or (timed_steps <= 0 and n_done >= len(mine)):
            break
    if overlap:
        p = sch.harvest_packed()          # what finished during the last window
        close_window(sch.counters())
        if p is not None:
            harvested.append(p)
            n_done += len(p["metas"])
    e_end.record()
    torch.cuda.synchronize()
    clk.__exit__(None, None, None)
    ms = e_begin.elapsed_time(e_end)
    steady = [(t, g) for t, g, occ in windows if occ >= 0.95]
    agg = torch.tensor([c_prev["generated"] - c0["generated"], c_prev["slot_steps"] - c0["slot_steps"], steps,
                        sum(g for _, g in steady), n_done], dtype=torch.float64, device=dev)
    mx = torch.tensor([ms, sum(t for t, _ in steady)], dtype=torch.float64, device=dev)
    t_gather, gathered = 0.0, None
    if world > 1:
        dist.all_reduce(agg)
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
    if gather and harvested:
        toks = torch.cat([p["tokens"] for p in harvested])
        lps = torch.cat([p["logp"] for p in harvested])
        lens_d = torch.cat([p["offsets"][1:] - p["offsets"][:-1] for p in harvested]).to(torch.int32)
        vers = torch.cat([p["versions"] for p in harvested]).to(torch.int32)
        ids = torch.tensor([i for p in harvested for i in p["metas"]], dtype=torch.int32, device=dev)
        gathered, t_gather = uvdist.gather_packed(toks, lps, lens_d, vers, ids)
    res = {"tokens_per_s": float(agg[0].item()) / (float(mx[0].item()) / 1e3), "ms": float(mx[0].item()),
           "generated_tokens": int(agg[0].item()), "requests_finished": int(agg[4].item()),
           "steps_all_ranks": int(agg[2].item()), "ms_per_step_rank0": ms / max(steps, 1),
           "slot_occupancy": float(agg[1].item()) / max(float(agg[2].item()) * slots, 1.0),
           "steady_state_tokens_per_s": (float(agg[3].item()) / (float(mx[1].item()) / 1e3)) if mx[1].item() > 0 else None,
           "steady_state": f"{W_STEPS}-step windows with slot occupancy >= 0.95 (max window time over ranks)",
           "prefill": "packed admission passes" if packed else (f"{lanes} prefill lanes" if lanes else "decode step"),
           "admission_passes": getattr(sch, "n_admit_passes", 0),
           "admission_passes_beside_steps": sch.n_deferred_passes,
           "steps_by_batch_rows_rank0": {str(k): v for k, v in sorted(sch.bucket_steps.items())},
           "weight_broadcast_ms": t_bcast * 1e3, "rollout_gather_ms": t_gather * 1e3,
           "device_status": eng.device_status(), "sched_status": c_prev["status"], "clocks_rank0": clk.summary()}
    if kernel_times and rank == 0 and slots in sch._graphs:
        # per-kernel device times of the full-batch step at the job's current cache state (CUPTI; the extra replays
        # advance the job, which is over)
        res["kernel_times_cupti"] = cupti_kernel_times(sch._graphs[slots].replay)
        res["kernel_times_cupti"]["mean_context"] = float(st.pos[:slots].float().mean().item())
    if gathered is not None:
        res["gathered"] = {"requests": int(sum(int(g[2].numel()) for g in gathered)),
                           "tokens": int(sum(int(g[0].numel()) for g in gathered)),
                           "payload": "tokens int32 + log-probs fp32 (flat, unpadded) + lengths, start versions, "
                                      "request ids int32"}
    del sch, st
    return res


def config3_requests():
    """benchmark configuration 3: 4096 requests, prompts U[16,256], stop length Geometric(mean 600) capped at 2048."""
    r = np.random.default_rng(3)
    n_req, max_prompt, max_new = 4096, 256, 2048
    lens = r.integers(16, max_prompt + 1, n_req)
    stops = np.minimum(r.geometric(1.0 / 600.0, n_req), max_new)
    return [r.integers(1, VOCAB, int(L)).tolist() for L in lens], stops, max_prompt, max_new


def config5_requests():
    """benchmark configuration 5: 256 prompts U[64,256] x group 8 = 2048 sequences, max_new 2048, T = 1, top-p 1."""
    r = np.random.default_rng(5)
    lens = r.integers(64, 257, 256)
    base = [r.integers(1, VOCAB, int(L)).tolist() for L in lens]
    return [p for p in base for _ in range(8)], 256, 2048


def run_continuous(args, m, rank, world, dev):
    """`--workload continuous`: benchmark configuration 3 as the headline line (whole job, or --steps timed steps)."""
    import torch.distributed as dist
    prompts, stops, max_prompt, max_new = config3_requests()
    r = rollout_job(m, rank, world, dev, prompts_all=prompts, stops_all=stops, slots=512, max_new=max_new,
                    max_prompt=max_prompt, lanes=args.lanes, lane_chunk=args.lane_chunk, seed=7, force_eos=True,
                    timed_steps=args.steps, warmup=args.warmup, broadcast=True, packed=args.prefill == "packed",
                    compact=not args.no_compact, overlap=not args.no_overlap, kernel_times=args.kernel_times,
                    overlap_admit=args.overlap_admit, window=args.window)
    if rank == 0:
        line = {"metric": "rollout decode tokens/s", "value": r["tokens_per_s"], "unit": "tokens/s",
                "n_gpus": world, "steps": r["steps_all_ranks"] // world, "warmup": max(args.warmup, 3),
                "ms_per_step": r["ms_per_step_rank0"], "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": "continuous batching: 4096 requests sharded over ranks, prompts U[16,256], "
                                       "stop ~ Geometric(mean 600) <= 2048 (EOS forced), 512 slots/GPU, T=1.0, "
                                       "device-side retire/refill, prefill through the decode step",
                           "prefill_lanes": args.lanes, "lane_chunk": args.lane_chunk},
                "run": r, "gpu_launches": (m.engine.launches_per_step() + 2) * (r["steps_all_ranks"] // world)}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------ main arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=512)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="fixed", choices=["fixed", "continuous", "attn", "gemm"])
    ap.add_argument("--rows", type=int, default=256, help="--workload gemm: batch rows")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--profile", action="store_true",
                    help="profiling runs (under ncu): one round of the attention timing loops instead of four")
    ap.add_argument("--no-rollouts", action="store_true",
                    help="skip the continuous-batching and GRPO-shaped rollout jobs reported beside the headline")
    ap.add_argument("--reference-gpu", action="store_true",
                    help="with --impl reference: also time the reference's Triton / NVRTC attention kernels on the GPU")
    ap.add_argument("--reference-gpu-only", action="store_true",
                    help="with --impl reference: print only that GPU comparator object")
    ap.add_argument("--prefill", default="packed", choices=["packed", "lanes"],
                    help="rollout jobs: how prompts enter the cache (packed admission passes, or prefill lanes through "
                         "the decode step)")
    ap.add_argument("--kernel-times", action="store_true",
                    help="add per-kernel device times of the step from CUPTI records (taken after the timed region)")
    ap.add_argument("--window", type=int, default=0,
                    help="rollout jobs: steps between harvests / admissions (default 32 with admission passes, else 64)")
    ap.add_argument("--overlap-admit", action="store_true",
                    help="rollout jobs: admission passes on a second stream beside the decode steps")
    ap.add_argument("--no-overlap", action="store_true",
                    help="rollout jobs: harvest after every window of steps instead of while the next one runs")
    ap.add_argument("--no-compact", action="store_true",
                    help="rollout jobs: keep every slot in the step (no slot compaction / smaller step graphs)")
    ap.add_argument("--lanes", type=int, default=128,
                    help="continuous workload: extra batch rows that carry prompt tokens of refilling slots (0 = "
                         "one prompt token per slot per step)")
    ap.add_argument("--lane-chunk", type=int, default=8, help="prompt tokens one slot may feed per step with lanes")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        return run_reference_arm(args, rank, world)

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the decode path has no CPU fallback")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    from ultraviolet_b200.generate import DecodeRunner
    from ultraviolet_b200 import dist as uvdist
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        uvdist.warmup(dev)

    dtype = torch.bfloat16
    m = build_model(dev, dtype)
    eng = m.engine
    hbm_peak, peak_kind = measured_peaks()

    if args.workload == "gemm":
        if rank == 0:
            run_gemm_workload(args, dev)
        return
    if args.workload == "attn":
        res = long_context_attention(eng, rounds=max(1, min(args.steps, 8)))
        stp = step_shape_attention(eng, rounds=max(1, min(args.steps, 4)))
        if rank == 0:
            print(json.dumps({"metric": "decode attention HBM GB/s", "value": res["gbs"], "unit": "GB/s",
                              "config": {"workload": "64 x 8192 int8 keys, one global-layer launch"},
                              "roofline": {"bound": "hbm", "achieved": res["gbs"], "peak": hbm_peak, "unit": "GB/s",
                                           "frac": res["gbs"] / hbm_peak,
                                           "traffic": res["bytes"] * NCU_TRAFFIC_RATIO["long_context"]},
                              "ms_per_launch": res["ms"], "splits": res["splits"],
                              "step_shape_256x256": {**stp, "frac": stp["gbs"] / hbm_peak}}), flush=True)
        return
    if args.workload == "continuous":
        return run_continuous(args, m, rank, world, dev)

    # ---- weights: rank 0's arena is the policy; everyone else receives it over NCCL
    t_bcast = uvdist.broadcast_weights(eng) if world > 1 else 0.0

    K, W = args.steps, max(args.warmup, 3)
    R = 5 if K <= 128 else 1   # short runs: the K-step block is timed R times back to back, the median is reported
    prompts = make_prompts(SLOTS, PROMPT_LO, PROMPT_HI, seed=100 + rank)
    # cache sized like production (max_prompt + max_new + slack, never below the configuration's 128 + 512): local
    # layers then keep their full 256-slot ring whatever --steps is
    max_len = max(PROMPT_HI + R * K + W + min(K, 64) + 16, PROMPT_HI + 512)
    st = m.new_state(SLOTS, max_len)
    from ultraviolet_b200.generate import _left_pad
    idx, starts = _left_pad(prompts, 0, dev)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    m.prefill(idx[:, :-1], starts, m.new_state(SLOTS, max_len))   # first call: buffers, library handles, kernel loads
    torch.cuda.synchronize()
    prefill_first_s = time.perf_counter() - t0
    t0 = time.perf_counter()
    m.prefill(idx[:, :-1], starts, st)
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0
    runner = DecodeRunner(m, st, bucket=max_len, use_graph=True, temperature=0.0)
    tok = runner.step(idx[:, -1].contiguous()).clone()
    for _ in range(W):
        tok = runner.step(tok).clone()
    torch.cuda.synchronize()
    pos_begin = st.pos.clone()

    # ---- timed region: K decode steps, device resident (R such blocks, each bracketed; median block reported)
    all_tok = torch.empty(K, SLOTS, dtype=torch.long, device=dev)
    block_ms = []
    clk = ClockSampler(local, interval_ms=50)   # the region is tens of milliseconds long at the default --steps
    clk.__enter__()   # samples until the end-to-end loop below is over: both are the same step under load
    for _ in range(R):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(K):
            tok = runner.step(tok)
            all_tok[i].copy_(tok)
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dist.barrier()
        block_ms.append(float(t.item()))
    ms = float(np.median(block_ms))
    value = world * SLOTS * K / (ms / 1e3)
    kernel_times = None
    if args.kernel_times and rank == 0:   # per-kernel device times of this step (CUPTI), after the timed region
        gl = runner.g_len(int(st.host_pos.max()))
        g = runner._graph(gl, host=False)
        pos0, steps0, tok0 = st.pos.clone(), runner.steps.clone(), runner.tok.clone()
        kernel_times = cupti_kernel_times(g.replay)
        st.pos.copy_(pos0), runner.steps.copy_(steps0), runner.tok.copy_(tok0)   # the replays advanced the device side only

    # ---- rollout gather (token ids of every rank to rank 0)
    t_gather = uvdist.gather_rollouts(all_tok.t().contiguous())[1] if world > 1 else 0.0

    # ---- e2e: the same steps through the public step API with pinned host buffers in and out
    #      (DecodeRunner.step_host: every step copies its 256 input tokens from pinned host memory, runs, copies the
    #      sampled tokens and log-probs back to pinned host memory and synchronises; the host feeds the tokens it
    #      read back as the next step's input)
    K2 = min(K, 64)
    tok_h = tok.cpu()
    runner.step_host(tok_h)            # captures the graph with its copy nodes (untimed)
    tok_h = runner.host_out.clone()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(K2):
        tok_h = runner.step_host(tok_h)
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e = world * SLOTS * K2 / e2e_s
    clk.__exit__(None, None, None)

    # ---- roofline of the dominant kernel of this library (decode attention), at the run's final cache state
    #      (rank 0 measures; the other ranks wait at the next job's barrier)
    if rank == 0:
        att = time_attention_layers(eng, st, st.pos - 1, st.starts, rounds=1 if args.profile else 4)
        att_mid = att["local"] if att["local"]["ms"] * 8 >= att["global"]["ms"] * 2 else att["global"]
        lc = long_context_attention(eng, rounds=1 if args.profile else 4)
        lc2 = lc if args.profile else long_context_attention(eng, ctx=16384)
        context_end = int(st.pos.float().mean().item())
        torch.cuda.empty_cache()

    # ---- the two rollout-shaped jobs of the configuration list, bounded, on all ranks (whole-box tokens/s under
    #      continuous batching is what the path is for; the fixed workload above is the per-step headline)
    cont = grpo = None
    if not args.no_rollouts:
        prompts3, stops3, mp3, mn3 = config3_requests()
        cont = rollout_job(m, rank, world, dev, prompts_all=prompts3, stops_all=stops3, slots=512, max_new=mn3,
                           max_prompt=mp3, lanes=args.lanes, lane_chunk=args.lane_chunk, seed=7, force_eos=True,
                           packed=args.prefill == "packed", compact=not args.no_compact, overlap=not args.no_overlap,
                           overlap_admit=args.overlap_admit, window=args.window)
        cont["workload"] = ("benchmark configuration 3: 4096 requests sharded i % W, prompts U[16,256], stop ~ "
                            "Geometric(600) <= 2048 (EOS forced), 512 slots/GPU, T = 1.0; whole job until drained")
        torch.cuda.empty_cache()
        prompts5, mp5, mn5 = config5_requests()
        grpo = rollout_job(m, rank, world, dev, prompts_all=prompts5, stops_all=None, slots=512, max_new=mn5,
                           max_prompt=mp5, lanes=args.lanes, lane_chunk=args.lane_chunk, seed=11, force_eos=False,
                           broadcast=True, gather=True, packed=args.prefill == "packed",
                           compact=not args.no_compact, overlap=not args.no_overlap,
                           overlap_admit=args.overlap_admit, window=args.window)
        grpo["workload"] = ("benchmark configuration 5: 256 prompts U[64,256] x group 8 = 2048 sequences sharded i % W, "
                            "max_new 2048, T = 1.0, top-p 1.0, Philox key per sequence; arena broadcast before the "
                            "round, rollouts (tokens, log-probs, versions) gathered to rank 0 after it")

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # bytes one decode step must move: weights once (99.6 MB bf16) + KV reads + KV appends (132 B per row per layer)
    kv_read = 8 * att["local"]["bytes"] + 2 * att["global"]["bytes"]
    step_bytes = 99_614_720 + kv_read + SLOTS * 10 * 132
    status = eng.check_status(SLOTS)
    line = {
        "metric": "rollout decode tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K,
        "warmup": W, "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "config": workload_config(K),
        "run": {"timed_blocks_ms": block_ms, "timed": f"median of {R} blocks of {K} steps", "max_len": max_len,
                "l2": "per-step working set (99.6 MB weights + KV of 10 layers) exceeds L2; no flush",
                "prefill_s": prefill_s, "prefill_first_call_s": prefill_first_s, "prefill_tokens": int(sum(len(p) - 1 for p in prompts)),
                "context_begin": int(pos_begin.float().mean().item()),
                "context_end": context_end,
                "weight_broadcast_ms": t_bcast * 1e3, "rollout_gather_ms": t_gather * 1e3,
                "step_bytes_floor": step_bytes,
                "step_hbm_frac": step_bytes / (ms / K / 1e3) / 1e9 / hbm_peak,
                "launches_per_step": eng.launches_per_step() + 1, "device_status": status},
        "e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": SLOTS * 8, "d2h_bytes_per_step": SLOTS * 12,
                "steps": K2},
        "gpu_launches": (eng.launches_per_step() + 1) * K,
        **({"kernel_times_cupti": kernel_times} if kernel_times is not None else {}),
        "clocks": clk.summary(),
        "roofline": {"bound": "hbm", "kernel": "attn_split_kernel (local-layer launches, 8 per step)"
                     if att_mid is att["local"] else "attn_split_kernel (global-layer launches, 2 per step)",
                     "achieved": att_mid["gbs"], "peak": hbm_peak, "peak_kind": peak_kind, "unit": "GB/s",
                     "frac": att_mid["gbs"] / hbm_peak,
                     "traffic": att_mid["bytes"] * NCU_TRAFFIC_RATIO["step"],
                     "traffic_source": "algorithmic bytes x 0.993, the DRAM-bytes / algorithmic-bytes ratio of the "
                                       "ncu capture of this launch shape (profiles/attn_split_kernel_step_shape.md)",
                     "bytes_per_launch": att_mid["bytes"], "ms_per_launch": att_mid["ms"], "path": att_mid["path"]},
        "attention": {"local": att["local"], "global": att["global"], "long_context_64x8192": lc,
                      "long_context_frac_of_measured": lc["gbs"] / hbm_peak,
                      "long_context_frac_of_nominal_8TBs": lc["gbs"] / 8000.0,
                      "long_context_64x16384": lc2, "long_context_64x16384_frac_of_measured": lc2["gbs"] / hbm_peak},
    }
    line["continuous"], line["grpo"] = cont, grpo
    if not args.no_cpu_baseline and world == 1:
        cb = cpu_baseline(32)  # the reference's prefill (~10 s) + ~3 s of timed steps on the host cores
        cb.pop("ms_per_step", None)
        line["cpu_baseline"] = cb
        line["attention"]["reference_gpu"] = reference_gpu_attention_subprocess()
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
