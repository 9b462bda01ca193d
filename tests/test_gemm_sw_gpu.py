"""Fused-epilogue tcgen05 GEMMs of the decode step (csrc/gemm_sw.cu) against fp32 PyTorch references of the same
products, against the unfused kernel pairs they replace (library GEMM + uv_swiglu / uv_resid_norm / uv_qkv_post), and
the deferred RMS norm against normalise-then-multiply.

Tolerance: one bf16 rounding of an fp32-accumulated product (2^-8 of the largest magnitude) plus summation order;
deferred norm: the product is scaled after the GEMM instead of before, which moves results by at most one more bf16
rounding."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _lib():
    from ultraviolet_b200 import _lib
    return _lib, _lib.lib()


def _sp():
    return torch.cuda.current_stream().cuda_stream


def _ss_parts(x, parts=5):
    """Sums of squares of x's rows split into `parts` column groups, as a producing epilogue leaves them."""
    M, d = x.shape
    w = d // parts
    return torch.stack([x[:, i * w:(i + 1) * w].float().pow(2).sum(1) for i in range(parts)]).contiguous()


@pytest.mark.parametrize("bn,ks", [(0, 0), (32, 1), (32, 2), (64, 4), (128, 1), (64, 8)])
@pytest.mark.parametrize("M,N,K", [(256, 640, 640), (256, 640, 512), (200, 640, 1664), (37, 128, 64),
                                   (512, 16384, 640), (300, 3328, 640)])
def test_gemm_sw_matches_fp32_reference(M, N, K, bn, ks):
    L, lib = _lib()
    g = torch.Generator(device=DEV).manual_seed(M + N + K)
    x = (torch.randn(M, K, device=DEV, generator=g) * 0.5).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.1).bfloat16()
    c = torch.full((M, N), 7.0, device=DEV, dtype=torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    L.check(lib.uv_gemm_sw(x.data_ptr(), K, w.data_ptr(), c.data_ptr(), N, 2, M, N, K, None, 0, 0, bn, ks,
                           status.data_ptr(), _sp()), "uv_gemm_sw")
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    ref = x.float() @ w.float().t()
    tol = ref.abs().max().item() * 2.0 ** -8
    assert (c.float() - ref).abs().max().item() <= tol


def test_gemm_sw_deferred_norm_equals_norm_then_gemm():
    L, lib = _lib()
    g = torch.Generator(device=DEV).manual_seed(3)
    M, N, K = 256, 640, 640
    x = (torch.randn(M, K, device=DEV, generator=g) * 3.0).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.1).bfloat16()
    ss = _ss_parts(x)
    c = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    L.check(lib.uv_gemm_sw(x.data_ptr(), K, w.data_ptr(), c.data_ptr(), N, 2, M, N, K, ss.data_ptr(), 5, M, 0, 0,
                           None, _sp()), "uv_gemm_sw")
    xn = torch.nn.functional.rms_norm(x.float(), (K,), eps=torch.finfo(torch.float32).eps)
    ref = xn @ w.float().t()
    tol = ref.abs().max().item() * 2.0 ** -7
    assert (c.float() - ref).abs().max().item() <= tol
    lib_way = torch.mm(xn.bfloat16(), w.t()).float()     # what the unfused path computes
    assert (c.float() - lib_way).abs().max().item() <= tol


@pytest.mark.parametrize("M,bn", [(256, 0), (512, 64), (100, 32)])
def test_gemm_sw_swiglu_vs_unfused_pair(M, bn):
    L, lib = _lib()
    K, f = 640, 1664
    g = torch.Generator(device=DEV).manual_seed(M)
    h = (torch.randn(M, K, device=DEV, generator=g) * 2.0).bfloat16()
    w = (torch.randn(2 * f, K, device=DEV, generator=g) * 0.05).bfloat16()
    ss = _ss_parts(h)
    act = torch.full((M, f), 7.0, device=DEV, dtype=torch.bfloat16)
    L.check(lib.uv_gemm_sw_swiglu(h.data_ptr(), K, w.data_ptr(), act.data_ptr(), 2, M, K, f, ss.data_ptr(), 5, M, bn,
                                  None, _sp()), "uv_gemm_sw_swiglu")
    hn = torch.nn.functional.rms_norm(h.float(), (K,), eps=torch.finfo(torch.float32).eps).bfloat16()
    gu = torch.mm(hn, w.t())
    ref = torch.empty_like(act)
    L.check(lib.uv_swiglu(gu.data_ptr(), 2, f, ref.data_ptr(), M, _sp()), "uv_swiglu")
    torch.cuda.synchronize()
    diff = (act.float() - ref.float()).abs().max().item()
    assert diff <= ref.float().abs().max().item() * 2.0 ** -6, diff
    gf = hn.float() @ w.float().t()
    exact = torch.nn.functional.silu(gf[:, :f]) * gf[:, f:]
    assert (act.float() - exact).abs().max().item() <= exact.abs().max().item() * 2.0 ** -6


@pytest.mark.parametrize("M,K,ks", [(256, 512, 0), (256, 1664, 4), (130, 1664, 2), (512, 1664, 0)])
def test_gemm_sw_resid_vs_unfused_pair(M, K, ks):
    L, lib = _lib()
    N = 640
    g = torch.Generator(device=DEV).manual_seed(M + K)
    a = (torch.randn(M, K, device=DEV, generator=g) * 0.5).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.1).bfloat16()
    x = torch.randn(M, N, device=DEV, generator=g).bfloat16()
    lam = torch.tensor([0.9375, 1.125], device=DEV)
    h = torch.full((M, N), 7.0, device=DEV, dtype=torch.bfloat16)
    ss = torch.full((N // 128, M), -1.0, device=DEV)
    L.check(lib.uv_gemm_sw_resid(a.data_ptr(), K, w.data_ptr(), x.data_ptr(), lam.data_ptr(), h.data_ptr(), N,
                                 ss.data_ptr(), M, 2, M, N, K, 0, ks, None, _sp()), "uv_gemm_sw_resid")
    prod = torch.mm(a, w.t())
    h_ref, hn_ref = torch.empty_like(h), torch.empty_like(h)
    L.check(lib.uv_resid_norm(x.data_ptr(), prod.data_ptr(), lam.data_ptr(), 2, N, h_ref.data_ptr(),
                              hn_ref.data_ptr(), M, _sp()), "uv_resid_norm")
    torch.cuda.synchronize()
    assert (h.float() - h_ref.float()).abs().max().item() <= h_ref.float().abs().max().item() * 2.0 ** -7
    want = torch.stack([h[:, i * 128:(i + 1) * 128].float().pow(2).sum(1) for i in range(N // 128)])
    torch.testing.assert_close(ss, want, rtol=1e-5, atol=1e-5)      # partial sums of squares of what was stored


def test_gemm_sw_qkv_equals_gemm_then_qkv_post():
    """QKV projection with the post-processing in the epilogue: same q / k / v rows, same int8 cache bytes and the
    same head gates as library GEMM on the normalised rows followed by uv_qkv_post_args."""
    L, lib = _lib()
    g = torch.Generator(device=DEV).manual_seed(7)
    B, H, K, hd, d, S, vocab, n_pairs, ve_ch, gate_ch = 200, 8, 1, 64, 640, 256, 512, 16, 12, 128
    x = (torch.randn(B, d, device=DEV, generator=g) * 2.0).bfloat16()
    xn = torch.nn.functional.rms_norm(x.float(), (d,), eps=torch.finfo(torch.float32).eps).bfloat16()
    w = (torch.randn((H + 2 * K) * hd, d, device=DEV, generator=g) * 0.06).bfloat16()
    tok = torch.randint(0, vocab, (B,), device=DEV, generator=g)
    ve = torch.randn(vocab, K * hd, device=DEV, generator=g).bfloat16()
    ve_gate = (torch.randn(K, ve_ch, device=DEV, generator=g) * 0.3).bfloat16()
    gate_w = (torch.randn(H, gate_ch, device=DEV, generator=g) * 0.2).bfloat16()
    pos = torch.randint(0, 700, (B,), device=DEV, generator=g)
    inv_freq = ((1.0 / 1024) ** torch.linspace(0, 1, n_pairs)).to(DEV)
    th = pos.float()[:, None] * inv_freq[None]
    rope_cs = torch.cat([th.cos().bfloat16().float(), th.sin().bfloat16().float()], 1).contiguous()
    res = {}
    for fused in (False, True):
        kc = torch.zeros(B, K, S, hd, dtype=torch.int8, device=DEV)
        vc = torch.zeros_like(kc)
        ks = torch.zeros(B, K, S, dtype=torch.float16, device=DEV)
        vs = torch.zeros_like(ks)
        oob = torch.zeros(1, dtype=torch.int32, device=DEV)
        gates = torch.zeros(B, H, device=DEV)
        qkv = torch.zeros(B, (H + 2 * K) * hd, device=DEV, dtype=torch.bfloat16)
        qa = L.QkvArgs()
        qa.qkv, qa.xn, qa.tok, qa.value_embed, qa.ve_gate = qkv.data_ptr(), xn.data_ptr(), tok.data_ptr(), \
            ve.data_ptr(), ve_gate.data_ptr()
        qa.inv_freq, qa.pos, qa.rope_cs = inv_freq.data_ptr(), pos.data_ptr(), rope_cs.data_ptr()
        qa.k_cache, qa.v_cache, qa.k_scale, qa.v_scale = kc.data_ptr(), vc.data_ptr(), ks.data_ptr(), vs.data_ptr()
        qa.oob_count, qa.dtype, qa.vocab = oob.data_ptr(), 2, vocab
        qa.B, qa.H, qa.K, qa.hd, qa.d, qa.S, qa.S_alloc, qa.ring, qa.ve_ch, qa.n_pairs = B, H, K, hd, d, S, S, 1, \
            ve_ch, n_pairs
        qa.gate_w, qa.gate_out, qa.gate_ch = gate_w.data_ptr(), gates.data_ptr(), gate_ch
        if fused:
            ss = _ss_parts(x)
            L.check(lib.uv_gemm_sw_qkv(x.data_ptr(), d, w.data_ptr(), C.byref(qa), ss.data_ptr(), 5, B, 0, 0, None,
                                       _sp()), "uv_gemm_sw_qkv")
        else:
            torch.mm(xn, w.t(), out=qkv)
            L.check(lib.uv_qkv_post_args(C.byref(qa), _sp()), "uv_qkv_post_args")
        torch.cuda.synchronize()
        assert int(oob.item()) == 0
        res[fused] = (qkv.float(), kc.clone(), vc.clone(), ks.float(), vs.float(), gates.clone())
    a, b = res[False], res[True]
    assert (a[0] - b[0]).abs().max().item() <= a[0].abs().max().item() * 2.0 ** -6
    for i in (1, 2):   # int8 cache bytes: a step on a small fraction (the deferred norm moves the projection by one
        dq = (a[i].int() - b[i].int()).abs()   # bf16 rounding, which the per-head norm and RoPE can double)
        assert int(dq.max()) <= 2 and (dq > 0).float().mean().item() < 0.05 and (dq > 1).float().mean().item() < 1e-3
    for i in (3, 4):
        torch.testing.assert_close(a[i], b[i], rtol=2e-2, atol=1e-6)
    torch.testing.assert_close(a[5], b[5], rtol=2e-2, atol=2e-2)
    assert b[1].any() and b[2].any() and b[5].abs().sum() > 0


def test_gemm_sw_rejects_bad_arguments():
    L, lib = _lib()
    a = torch.zeros(128, 96, device=DEV, dtype=torch.bfloat16)
    c = torch.zeros(128, 128, device=DEV, dtype=torch.bfloat16)
    assert lib.uv_gemm_sw(a.data_ptr(), 96, a.data_ptr(), c.data_ptr(), 128, 2, 128, 128, 96, None, 0, 0, 0, 0, None,
                          None) == -3                       # K % 64
    assert lib.uv_gemm_sw(a.data_ptr(), 64, a.data_ptr(), c.data_ptr(), 128, 1, 128, 128, 64, None, 0, 0, 0, 0, None,
                          None) != 0                        # fp16 is not built
    assert lib.uv_gemm_sw(a.data_ptr(), 64, a.data_ptr(), c.data_ptr(), 128, 2, 128, 96, 64, None, 0, 0, 0, 0, None,
                          None) == -3                       # N % 128


def _steps(m, B, steps, seed):
    st = m.new_state(B, 64)
    g = torch.Generator(device=DEV).manual_seed(seed)
    out = []
    for _ in range(steps):
        tok = torch.randint(1, m.cfg.vocab_size, (B,), device=DEV, generator=g)
        out.append(m.decode_step(tok, st, 64).float().cpu().numpy())
    return np.stack(out), st


@pytest.mark.parametrize("B", [5, 256])
def test_three_step_paths_agree(B):
    """One model, three ways (and one hybrid) to run the step: the reference's literal op order (library GEMMs + separate residual /
    norm kernels), the folded residual stream with deferred norms (the default), and the tcgen05 GEMMs with fused
    epilogues.  Logits agree within the path's 2e-2 tolerance; first-layer cache bytes within a step."""
    from tests import golden_inputs as gi
    from tests.helpers import build_model
    spec = gi.model_specs()["uv50m"]
    m = build_model(spec).to(DEV).to(torch.bfloat16).fuse_for_inference(torch.bfloat16)
    eng = m.engine
    assert eng.fold and eng.tc_gemm_ok
    res = {}
    # (fold_sw: the folded step with QKV GEMM + uv_qkv_post as one launch of the own tcgen05 kernel)
    for name, fold, tc, sw in (("fold", True, False, "0"), ("literal", False, False, "0"), ("tc", False, True, "0"),
                               ("fold_sw", True, False, "1")):
        eng.fold, eng.tc_gemm, eng.sw_qkv = fold, tc, sw
        eng.load_from(m)
        res[name] = _steps(m, B, 5, 3)
        assert eng.device_status() == {"attn_status": 0, "kv_oob": 0}
    eng.fold, eng.tc_gemm, eng.sw_qkv = True, False, "0"
    eng.load_from(m)
    ref, sref = res["literal"]
    for name in ("fold", "tc", "fold_sw"):
        lg, st = res[name]
        assert np.isfinite(lg).all()
        err = np.abs(lg - ref)
        assert err.max() <= 2e-2 * np.abs(ref).max(), (name, err.max(), np.abs(ref).max())
        assert (lg.argmax(-1) == ref.argmax(-1)).mean() > 0.9
        d = (st.k[0].int() - sref.k[0].int()).abs()
        assert int(d.max()) <= 2 and (d > 0).float().mean().item() < 0.05, (name, int(d.max()))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,d,f", [(256, 640, 1664), (7, 64, 128), (33, 1280, 4096)])
def test_swiglu_with_deferred_norm(M, d, f, dtype):
    """uv_swiglu_rs(gu, h) = silu(g * rs) * (u * rs), rs = rsqrt(mean(h^2) + eps), with the reference's rounding
    points (the scaled projection and silu(g) are rounded to the activation dtype)."""
    L, lib = _lib()
    code = {torch.float16: 1, torch.bfloat16: 2}[dtype]
    g = torch.Generator(device=DEV).manual_seed(M + f)
    h = (torch.randn(M, d, device=DEV, generator=g) * 3).to(dtype)
    gu = torch.randn(M, 2 * f, device=DEV, generator=g).to(dtype)
    act = torch.full((M, f), 7.0, device=DEV, dtype=dtype)
    L.check(lib.uv_swiglu_rs(gu.data_ptr(), h.data_ptr(), code, d, f, act.data_ptr(), M, _sp()), "uv_swiglu_rs")
    rs = torch.rsqrt(h.float().pow(2).mean(1, keepdim=True) + torch.finfo(torch.float32).eps)
    gs = (gu.float() * rs).to(dtype).float()
    ref = (torch.nn.functional.silu(gs[:, :f]).to(dtype).float() * gs[:, f:]).to(dtype)
    torch.cuda.synchronize()
    assert (act.float() - ref.float()).abs().max().item() <= ref.float().abs().max().item() * 2.0 ** -7
    assert (act == ref).float().mean().item() > 0.98


@pytest.mark.parametrize("H,K", [(8, 1), (28, 2), (6, 1), (3, 1)])   # 18 / 60 / 14 / 8 items per row: the row's sum
def test_qkv_post_on_unnormalised_rows_equals_normalise_first(H, K):  # of squares by 6 warps, 6, each warp alone, 4
    """uv_qkv_post_args with xn_raw: qkv holds the projection of the UN-normalised rows; the kernel scales it by the
    row's RMS factor and reads normalised gate inputs on the fly -- same q / k / v, cache bytes and gates as the
    projection of the normalised rows with xn_raw = 0, up to one bf16 rounding of the projection."""
    L, lib = _lib()
    g = torch.Generator(device=DEV).manual_seed(11)
    B, hd, d, S, vocab, n_pairs, ve_ch, gate_ch = 130, 64, 640, 264, 300, 16, 12, 128
    y = (torch.randn(B, d, device=DEV, generator=g) * 2.5).bfloat16()
    yn = torch.nn.functional.rms_norm(y.float(), (d,), eps=torch.finfo(torch.float32).eps).bfloat16()
    w = (torch.randn((H + 2 * K) * hd, d, device=DEV, generator=g) * 0.06).bfloat16()
    tok = torch.randint(0, vocab, (B,), device=DEV, generator=g)
    ve = torch.randn(vocab, K * hd, device=DEV, generator=g).bfloat16()
    ve_gate = (torch.randn(K, ve_ch, device=DEV, generator=g) * 0.3).bfloat16()
    gate_w = (torch.randn(H, gate_ch, device=DEV, generator=g) * 0.2).bfloat16()
    pos = torch.randint(0, 900, (B,), device=DEV, generator=g)
    inv_freq = ((1.0 / 1024) ** torch.linspace(0, 1, n_pairs)).to(DEV)
    th = pos.float()[:, None] * inv_freq[None]
    rope_cs = torch.cat([th.cos().bfloat16().float(), th.sin().bfloat16().float()], 1).contiguous()
    res = {}
    # 0: normalise first; 1: raw rows + xn_raw; 2..: ONE launch of uv_gemm_sw_qkv on the raw rows with no sums of
    # squares handed in (the kernel forms them from its own activation tiles), several tilings / cluster splits
    sw_hints = {2: (0, 0), 3: (32, 1), 4: (32, 4), 5: (64, 2), 6: (128, 4)} if (H + 2 * K) % 2 == 0 else {}
    for raw in (0, 1, *sw_hints):
        kc = torch.zeros(B, K, S, hd, dtype=torch.int8, device=DEV)
        vc = torch.zeros_like(kc)
        ks = torch.zeros(B, K, S, dtype=torch.float16, device=DEV)
        vs = torch.zeros_like(ks)
        oob = torch.zeros(1, dtype=torch.int32, device=DEV)
        gates = torch.zeros(B, H, device=DEV)
        src = y if raw else yn
        qkv = torch.mm(src, w.t()) if raw < 2 else torch.zeros(B, (H + 2 * K) * hd, dtype=torch.bfloat16, device=DEV)
        qa = L.QkvArgs()
        qa.qkv, qa.xn, qa.tok, qa.value_embed, qa.ve_gate = qkv.data_ptr(), src.data_ptr(), tok.data_ptr(), \
            ve.data_ptr(), ve_gate.data_ptr()
        qa.inv_freq, qa.pos, qa.rope_cs = inv_freq.data_ptr(), pos.data_ptr(), rope_cs.data_ptr()
        qa.k_cache, qa.v_cache, qa.k_scale, qa.v_scale = kc.data_ptr(), vc.data_ptr(), ks.data_ptr(), vs.data_ptr()
        qa.oob_count, qa.dtype, qa.vocab = oob.data_ptr(), 2, vocab
        qa.B, qa.H, qa.K, qa.hd, qa.d, qa.S, qa.S_alloc, qa.ring, qa.ve_ch, qa.n_pairs = B, H, K, hd, d, S, S, 1, \
            ve_ch, n_pairs
        qa.gate_w, qa.gate_out, qa.gate_ch, qa.xn_raw = gate_w.data_ptr(), gates.data_ptr(), gate_ch, min(raw, 1)
        if raw < 2:
            L.check(lib.uv_qkv_post_args(C.byref(qa), _sp()), "uv_qkv_post_args")
        else:
            status = torch.zeros(1, dtype=torch.int32, device=DEV)
            bn, ks_ = sw_hints[raw]
            L.check(lib.uv_gemm_sw_qkv(y.data_ptr(), d, w.data_ptr(), C.byref(qa), None, -1 if raw == 3 else 0, 0, bn,
                                       ks_, status.data_ptr(), _sp()), "uv_gemm_sw_qkv")
            torch.cuda.synchronize()
            assert int(status.item()) == 0
        torch.cuda.synchronize()
        assert int(oob.item()) == 0
        res[raw] = (qkv.float(), kc, vc, ks.float(), vs.float(), gates)
    a, b = res[0], res[1]
    assert (a[0] - b[0]).abs().max().item() <= a[0].abs().max().item() * 2.0 ** -6
    for i in (1, 2):
        dq = (a[i].int() - b[i].int()).abs()
        assert int(dq.max()) <= 3 and (dq > 0).float().mean().item() < 0.05 and (dq > 1).float().mean().item() < 1e-3
    torch.testing.assert_close(a[5], b[5], rtol=2e-2, atol=2e-2)
    assert b[1].any() and b[5].abs().sum() > 0
    for v in sw_hints:
        c = res[v]
        assert (c[0] - b[0]).abs().max().item() <= b[0].abs().max().item() * 2.0 ** -6, v
        for i in (1, 2):
            dq = (c[i].int() - b[i].int()).abs()
            assert int(dq.max()) <= 3 and (dq > 0).float().mean().item() < 0.05 and \
                (dq > 1).float().mean().item() < 1e-3, (v, i)
        torch.testing.assert_close(c[5], b[5], rtol=2e-2, atol=2e-2)
