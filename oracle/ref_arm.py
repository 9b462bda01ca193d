"""Drive the reference implementation installed under ``oracle/_ref`` (see make_ref.py) for the benchmark's
reference arm and CPU-baseline leg.  TEST / BENCHMARK INFRASTRUCTURE ONLY; the library never imports this.

``cpu_decode`` runs the reference's own int8-KV decode route on the host cores: ``MathLM`` with
``decode_impl = "kernel-int8"`` -> ``prefill_fast`` / ``decode_step_fast`` (ultraviolet/kernels/fast_decode.py:70-114,
:272-334) with the GPU attention kernel rebound to the reference's own torch implementation
``decode_attention_ref`` (ultraviolet/kernels/decode_attn.py:233-263) -- the reference's CPU-runnable form of the path.

``gpu_attention`` times the reference's GPU kernels for the attention step on the current CUDA device: the Triton
split / combine kernels (decode_attn.py:24-115) and the NVRTC tensor-core kernel (decode_attn_cuda.py:94-227).
"""
from __future__ import annotations

import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")


def available() -> bool:
    return os.path.isfile(os.path.join(REF_DIR, "ultraviolet", "model.py"))


def _import():
    if not available():
        raise RuntimeError("oracle/_ref is missing: run `python oracle/make_ref.py` where the reference checkout is")
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    import ultraviolet.kernels.fast_decode as ref_fd
    from ultraviolet.kernels import decode_attention_ref

    def _ref_attn(q, k, v, pos, starts, scale, *, window=0, ring=None, k_scale=None, v_scale=None, **_):
        return decode_attention_ref(q, k, v, pos, starts, scale, window=window, ring=ring, k_scale=k_scale,
                                    v_scale=v_scale)

    ref_fd.decode_attention = _ref_attn
    return ref_fd


def host_threads() -> int:
    """Use every host core, whatever OMP_NUM_THREADS the launcher exported (torchrun sets it to 1)."""
    import torch
    n = os.cpu_count() or 1
    torch.set_num_threads(n)
    return torch.get_num_threads()


def cpu_decode(prompts, n_steps: int, warmup: int = 1, vocab: int = 16384, seed: int = 0, max_len: int | None = None):
    """The reference's CPU decode of `prompts` (list of token-id lists): left-padded prefill of all but the last
    prompt token, then `warmup` untimed and `n_steps` timed greedy decode steps in fp32.  Returns a dict with
    tokens/s over the timed steps, seconds, prefill seconds, threads and the mean context."""
    import torch
    _import()
    from ultraviolet.model import MathLM, _left_pad, make_config, sample
    threads = host_threads()
    torch.manual_seed(seed)
    m = MathLM(make_config("uv-50m-alpha", vocab_size=vocab))
    m.decode_impl = "kernel-int8"
    m = m.float().fuse_for_inference(torch.float32)
    B = len(prompts)
    with torch.no_grad():
        idx, starts = _left_pad(prompts, 0, "cpu")
        T = idx.size(1)
        max_len = max_len or (T + warmup + n_steps + 2)
        st = m.new_state(B, max_len, torch.float32, "cpu")
        t0 = time.perf_counter()
        m.prefill(idx[:, :-1], starts, st)
        prefill_s = time.perf_counter() - t0
        tok = idx[:, -1].contiguous()
        for _ in range(max(warmup, 0)):
            tok = sample(m.decode_step(tok, st, max_len), 0.0)
        ctx0 = float((st.pos - st.starts).float().mean())
        t0 = time.perf_counter()
        for _ in range(n_steps):
            tok = sample(m.decode_step(tok, st, max_len), 0.0)
        dt = time.perf_counter() - t0
    return {"tokens_per_s": B * n_steps / dt, "seconds": dt, "prefill_s": prefill_s, "threads": threads,
            "context": ctx0, "steps": n_steps}


def _time_cuda(fn, reps: int):
    """(milliseconds per call of fn, whether it was graph-timed): captured once into a CUDA graph (after an eager call that compiles / warms the
    kernels) and replayed, so the figure is device time and not the host's launch rate; eager timing if the
    function cannot be captured."""
    import torch
    fn()
    torch.cuda.synchronize()
    g = None
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream().wait_stream(side)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        g.replay()
        torch.cuda.synchronize()
    except Exception:  # noqa: BLE001
        g = None
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay() if g is not None else fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps, g is not None


def gpu_attention(shapes=("long", "step"), reps: int = 4) -> dict:
    """Microseconds per attention call of the reference's GPU kernels on the current device, per shape:
    "long" = 64 rows x 8192 keys, linear cache (global layer); "step" = 256 rows x ring of 256 slots, window 256,
    positions U[131, 323] (local layer inside the fixed-batch step).  Several cache copies larger than L2 together
    are visited in turn.  Backends: Triton in bf16 and fp16, NVRTC ("cuda") in fp16.  A backend that fails to
    compile or run reports the error text instead of a time."""
    import torch
    ref_fd = _import()  # noqa: F841  (makes the package importable)
    from ultraviolet.kernels.decode_attn import decode_attention
    dev = torch.device("cuda", torch.cuda.current_device())
    out = {}
    for shape in shapes:
        g = torch.Generator(device=dev).manual_seed(1 if shape == "long" else 2)
        if shape == "long":
            B, S, n_copies, window, ring = 64, 8192, 3, 0, False
            pos = torch.full((B,), S - 1, device=dev, dtype=torch.long)
        else:
            B, S, n_copies, window, ring = 256, 256, 16, 256, True
            pos = torch.randint(131, 324, (B,), device=dev, generator=g)
        H, hd = 8, 64
        bufs = [(torch.randint(-127, 128, (B, 1, S, hd), device=dev, dtype=torch.int8, generator=g),
                 torch.randint(-127, 128, (B, 1, S, hd), device=dev, dtype=torch.int8, generator=g),
                 (torch.rand(B, 1, S, device=dev, generator=g) * 0.02 + 0.01).half(),
                 (torch.rand(B, 1, S, device=dev, generator=g) * 0.02 + 0.01).half()) for _ in range(n_copies)]
        st0 = torch.zeros(B, device=dev, dtype=torch.long)
        q32 = torch.randn(B, H, hd, device=dev, generator=g)
        n_keys = int(torch.clamp(pos + 1, max=S if ring else 1 << 30).sum().item())
        res = {"bytes": n_keys * 132 + 2 * B * H * hd * 2}
        for name, backend, dt in (("triton_bf16", "triton", torch.bfloat16), ("triton_fp16", "triton", torch.float16),
                                  ("nvrtc_fp16", "cuda", torch.float16)):
            q = q32.to(dt)

            def run():
                for k, v, ks, vs in bufs:
                    decode_attention(q, k, v, pos, st0, 0.14125, window=window, ring=ring, k_scale=ks, v_scale=vs,
                                     ctx_hint=S, backend=backend)
            try:
                ms, graphed = _time_cuda(run, reps)
                ms /= len(bufs)
                res[name] = {"us": ms * 1e3, "gbs": res["bytes"] / ms / 1e6,
                             "timed": "CUDA graph replays" if graphed else "eager launches"}
            except Exception as e:  # noqa: BLE001  (a backend that cannot compile here is reported, not fatal)
                res[name] = {"unavailable": f"{type(e).__name__}: {str(e)[:300]}"}
        out[shape] = res
    return out
