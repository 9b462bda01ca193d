"""Seeded inputs shared by tests/golden/make_golden.py (which runs the reference on them) and the parity tests (which
run the oracle and the CUDA path on them).  Everything here is deterministic given numpy / torch CPU generators."""
from __future__ import annotations

import hashlib

import numpy as np
import torch


def sha(*arrays) -> str:
    h = hashlib.sha256()
    for a in arrays:
        a = np.ascontiguousarray(a)
        h.update(str(a.dtype).encode() + str(a.shape).encode() + a.tobytes())
    return h.hexdigest()


def state_sha(sd: dict) -> str:
    return sha(*[sd[k].detach().float().numpy() for k in sorted(sd)])


def pack_lists(rows) -> np.ndarray:
    """list[list[int]] -> 1-D int64 [n, len_0, ..., len_{n-1}, tokens...]."""
    flat = [len(rows)] + [len(r) for r in rows] + [t for r in rows for t in r]
    return np.asarray(flat, dtype=np.int64)


def unpack_lists(a: np.ndarray):
    n = int(a[0])
    lens = a[1:1 + n].tolist()
    out, o = [], 1 + n
    for L in lens:
        out.append(a[o:o + L].tolist())
        o += L
    return out


def f16(x: np.ndarray) -> np.ndarray:
    """Round to fp16 values, keep fp32 storage (the reference tests feed fp16 tensors)."""
    return x.astype(np.float16).astype(np.float32)


# ------------------------------------------------------------------------------------------------ quantiser
def quant_cases() -> dict:
    r = np.random.default_rng(11)
    cases = {}
    x = f16(r.standard_normal((64, 3, 128)).astype(np.float32) * 3)
    x[0, 0] = 0
    cases["normal_hd128"] = x
    cases["normal_hd64"] = r.standard_normal((257, 64)).astype(np.float32)
    # rounding ties: rows whose scale is exactly 1 (max 127) and whose entries sit on .5 boundaries
    t = (r.integers(-126, 126, (32, 64)) + 0.5).astype(np.float32)
    t[:, 0] = 127.0
    cases["ties"] = t
    # degenerate magnitudes: tiny (fp16 scale underflows to 0), subnormal scales, huge (fp16 scale overflows to inf)
    e = np.zeros((6, 64), np.float32)
    e[0, 3] = 1e-9
    e[1] = r.standard_normal(64).astype(np.float32) * 1e-6
    e[2] = r.standard_normal(64).astype(np.float32) * 3e-4
    e[3] = r.standard_normal(64).astype(np.float32) * 1e7
    e[4, 5] = -65504.0 * 127
    e[5] = 0.0
    cases["extremes"] = e
    cases["bf16_like"] = (r.standard_normal((128, 64)).astype(np.float32).view(np.uint32) & np.uint32(0xFFFF0000)
                          ).view(np.float32)
    return cases


def kv_write_case():
    r = np.random.default_rng(12)
    x = r.standard_normal((8, 64)).astype(np.float32)
    # flat index (b*K + h)*S + slot with B=4, K=2, S=16
    idx = np.array([(b * 2 + h) * 16 + s for b, h, s in
                    [(0, 0, 3), (0, 1, 15), (1, 0, 0), (1, 1, 7), (2, 0, 9), (2, 1, 9), (3, 0, 1), (3, 1, 14)]],
                   dtype=np.int64)
    return x, idx


# ------------------------------------------------------------------------------------------------ attention
def config1() -> dict:
    """The CPU-runnable decode-attention configuration: 16 sequences, KV lengths uniform in [32, 512], H=8, K=1,
    hd=64, fp32 N(0,1) from torch generator seed 0, drawn in the order lens, q, k, v."""
    g = torch.Generator().manual_seed(0)
    lens = torch.randint(32, 513, (16,), generator=g)
    q = torch.randn(16, 8, 64, generator=g)
    k = torch.randn(16, 1, 512, 64, generator=g)
    v = torch.randn(16, 1, 512, 64, generator=g)
    return {"lens": lens.numpy().astype(np.int64), "q": q.numpy(), "k": k.numpy(), "v": v.numpy()}


def _attn_case(seed, B, KH, G, hd, S, int8, pos, starts, scale, window=0, ring=None):
    r = np.random.default_rng(seed)
    q = f16(r.standard_normal((B, KH * G, hd)).astype(np.float32))
    k = f16(r.standard_normal((B, KH, S, hd)).astype(np.float32))
    v = f16(r.standard_normal((B, KH, S, hd)).astype(np.float32))
    return dict(q=q, k=k, v=v, pos=np.asarray(pos, np.int64), starts=np.asarray(starts, np.int64), scale=float(scale),
                window=int(window), ring=ring, int8=int8, B=B, KH=KH, G=G, hd=hd, S=S)


def attn_cases() -> dict:
    """The shape / position grids of the reference's kernel tests (tests/test_math_kernels.py:36-112)."""
    cases = {}
    for i, (B, KH, G, hd) in enumerate([(1, 1, 1, 128), (3, 1, 4, 128), (17, 1, 5, 128), (5, 2, 4, 64),
                                        (9, 1, 8, 64), (4, 2, 2, 16), (6, 1, 7, 128)]):
        for int8 in (True, False):
            S = 700
            r = np.random.default_rng(100 + i)
            pos = r.integers(0, S, B)
            pos[0] = S - 1
            starts = (r.random(B) * (pos + 1)).astype(np.int64)
            starts[0] = 0
            cases[f"global.{B}x{KH}x{G}x{hd}.{'i8' if int8 else 'f16'}"] = _attn_case(
                200 + i, B, KH, G, hd, S, int8, pos, starts, 1.13 / hd ** 0.5)
    for i, (W, hd, G) in enumerate([(128, 128, 5), (256, 64, 8), (1024, 128, 4), (100, 128, 4)]):
        pos = [0, 5, W - 2, W - 1, W, W + 1, 2 * W + 7, 3 * W - 1, 5 * W + 3, W + 10, 4 * W, 7]
        starts = [0, 2, 0, 3, 0, 4, 0, 2 * W + 5, 0, 30, 4 * W - 3, 7]
        for int8 in (True, False):
            cases[f"ring.W{W}.hd{hd}.G{G}.{'i8' if int8 else 'f16'}"] = _attn_case(
                300 + i, 12, 1, G, hd, W, int8, pos, starts, 0.1, window=W)
    cases["window_linear"] = _attn_case(400, 6, 1, 4, 128, 500, False, [10, 63, 64, 200, 499, 300],
                                        [0, 0, 1, 180, 0, 290], 0.1, window=64, ring=False)
    cases["window_linear.i8"] = _attn_case(401, 6, 1, 8, 64, 500, True, [10, 63, 64, 200, 499, 300],
                                           [0, 0, 1, 180, 0, 290], 0.1, window=64, ring=False)
    # cache[:, :, :g_len] views: the case itself is dense; the test slices it (positions stay below 256)
    cases["slice.i8"] = _attn_case(402, 5, 2, 4, 128, 512, True, [0, 100, 255, 17, 200], [0, 3, 0, 17, 150], 0.1)
    # model shapes at the preset's sizes: H=8, K=1, hd=64, window 256 ring and a longer global cache
    r = np.random.default_rng(403)
    pos = r.integers(0, 2300, 33)
    cases["uv.global"] = _attn_case(404, 33, 1, 8, 64, 2304, True, pos, np.minimum(pos, r.integers(0, 40, 33)),
                                    0.14125)
    pos = r.integers(0, 3000, 33)
    cases["uv.local"] = _attn_case(405, 33, 1, 8, 64, 256, True, pos, np.minimum(pos, r.integers(0, 40, 33)),
                                   0.14125, window=256)
    return cases


# ------------------------------------------------------------------------------------------------ model
def model_specs() -> dict:
    tiny_prompts = [[1, 2, 3, 4, 5, 6], [7, 8, 9], [10, 11, 12, 13]]
    cont_prompts = [[(7 * i + 3 * j) % 500 + 1 for j in range(3 + (i * 5) % 7)] for i in range(9)]
    gen = dict(generate=dict(prompts=tiny_prompts, max_new=25, eos_id=None),
               continuous=dict(prompts=cont_prompts, max_new=20, batch=4, eos_id=None, check_every=4,
                               target_lens=[5, 20, 9, 1, 13, 20, 7, 16, 3]))
    return {
        # the reference tests' tiny model (tests/test_math_kernels.py:131-140): K=2 GQA, hd 16, window 8
        "tiny": dict(preset="tiny", over=dict(xsa=True), seed=0, perturb="outputs", B=6, P=5, N=30,
                     cache_layers=[0, 1], **gen),
        # MQA, hd 64, XSA: the production head geometry at toy width
        "tiny_hd64": dict(preset="tiny", over=dict(xsa=True, head_dim=64, n_kv_heads=1), seed=0, perturb="outputs",
                          B=6, P=5, N=30, cache_layers=[0, 3]),
        # UV-50M at the benchmark's sizes, random init seed 0, every 2-D weight perturbed so no projection is zero
        "uv50m": dict(preset="uv-50m-alpha", over=dict(vocab_size=16384), seed=0, perturb="all2d", B=4, P=40, N=6,
                      cache_layers=[0, 4]),
    }


def perturb_(m, spec) -> None:
    """outputs: N(0, 0.3) on the zero-initialised output-side parameters (tests/test_math_kernels.py:132-140);
    all2d: p += 0.02 * randn on every 2-D parameter plus N(0, 0.3) gates / alphas (tests/test_perf_opt.py:24-36)."""
    g = torch.Generator().manual_seed(spec["seed"] + 1000)
    with torch.no_grad():
        for n, p in sorted(m.named_parameters()):
            small = n.endswith(("ve_gate", "attn_gate", "xsa_alpha"))
            if spec["perturb"] == "outputs":
                if small or n.endswith(("wo", "w_down")):
                    p.copy_(torch.randn(p.shape, generator=g) * 0.3)
            else:
                if small:
                    p.copy_(torch.randn(p.shape, generator=g) * 0.3)
                elif p.dim() == 2:
                    p.add_(torch.randn(p.shape, generator=g) * 0.02)
                elif n.endswith(("resid_attn", "post_attn", "resid_mlp", "post_mlp", "qkv_scale", "o_scale")):
                    p.add_(torch.randn(p.shape, generator=g) * 0.05)


def teacher_inputs(spec):
    r = np.random.default_rng(spec["seed"] + 77)
    B, P, N = spec["B"], spec["P"], spec["N"]
    V = 512 if spec["preset"] == "tiny" else spec["over"]["vocab_size"]
    idx = r.integers(1, V, (B, P)).astype(np.int64)
    starts = (np.arange(B) % P).astype(np.int64)
    starts[-1] = 0
    cont = r.integers(1, V, (B, N)).astype(np.int64)
    return idx, starts, cont, P + N + 1


def logit_columns(spec, V: int) -> np.ndarray:
    return np.arange(V) if V <= 512 else np.arange(0, V, 16)


# ------------------------------------------------------------------------------------------------ samplers
def fused_sample_case():
    r = np.random.default_rng(21)
    x = f16(r.standard_normal((12, 16384)).astype(np.float32) * 4)
    u = r.random(12).astype(np.float32)
    u[0], u[1] = 0.0, np.float32(1.0 - 2 ** -24)
    return x, u, (23.0, 5.0, 7.5), (1.0, 0.7)


def top_p_case():
    r = np.random.default_rng(22)
    lg = (r.standard_normal((6, 12)) * 2).astype(np.float32)
    lg[1, 3] = lg[1, 5]  # a tie at some rank
    return lg, 0.8, 0.9, 4000


def varlen_case():
    """Packed causal attention with a window (prompt prefill): ragged segments including an empty one."""
    r = np.random.default_rng(31)
    lens = [5, 0, 33, 70]
    N, H, K, hd = sum(lens), 4, 2, 16
    q = r.standard_normal((N, H, hd)).astype(np.float32)
    k = r.standard_normal((N, K, hd)).astype(np.float32)
    v = r.standard_normal((N, K, hd)).astype(np.float32)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    return dict(q=q, k=k, v=v, cu=cu, scale=0.25, window=24)


def packing_case():
    """Rollouts for the trainer's packed micro-batches (layout test of the reference, tests/test_perf_opt.py:93-118):
    (tokens, prompt length, advantage, behaviour log-probs) per rollout, budget 1024, pad segments of 512."""
    rng = np.random.default_rng(0)
    items = []
    for i in range(20):
        L, s = int(rng.integers(5, 300)), int(rng.integers(2, 5))
        t = rng.integers(1, 100, size=L)
        items.append((t, s, float(i + 1), rng.normal(size=L - s).astype(np.float32)))
    return items, 1024, 0, 512
