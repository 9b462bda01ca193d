"""CUDA kernels (through the C ABI) against the oracle and the reference-generated golden files.

int8 bytes and fp16 scales: bit-exact.  Attention: atol = rtol = 2e-3 for fp16 queries (the reference's own kernel
tolerance, tests/test_math_kernels.py:52), 2e-2 relative for bf16 queries.
"""
import numpy as np
import pytest
import torch

from oracle import attn as oattn
from oracle import kv as okv
from oracle import model as om
from tests import golden_inputs as gi
from tests.helpers import golden

pytestmark = pytest.mark.gpu
DEV = "cuda"


def T(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    return t if dtype is None else t.to(dtype)


def u16(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


# ------------------------------------------------------------------------------------------------ quantiser
@pytest.mark.parametrize("name", sorted(gi.quant_cases()))
def test_quantize_bit_exact_vs_reference_golden(name):
    from ultraviolet_b200.kernels import quantize_kv
    g = golden("quant")
    x = gi.quant_cases()[name]
    q, s = quantize_kv(T(x))
    assert q.dtype == torch.int8 and s.dtype == torch.float16 and q.shape == x.shape and s.shape == x.shape[:-1]
    assert np.array_equal(q.cpu().numpy(), g[name + ".q"])
    assert np.array_equal(u16(s), g[name + ".s"])


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("hd", [16, 32, 64, 128])
def test_quantize_half_inputs(dtype, hd):
    from ultraviolet_b200.kernels import quantize_kv
    r = np.random.default_rng(hd)
    x = T(r.standard_normal((333, hd)).astype(np.float32) * 2, dtype)
    q, s = quantize_kv(x)
    qr, sr = okv.quantize_kv(x.float().cpu().numpy())
    assert np.array_equal(q.cpu().numpy(), qr) and np.array_equal(u16(s), sr.view(np.uint16))


def test_kv_write_scatter_golden():
    from ultraviolet_b200.kernels import kv_write
    g = golden("quant")
    x, idx = gi.kv_write_case()
    cache = torch.zeros(4, 2, 16, 64, dtype=torch.int8, device=DEV)
    sc = torch.zeros(4, 2, 16, dtype=torch.float16, device=DEV)
    kv_write(cache, sc, T(idx), T(x))
    assert np.array_equal(cache.cpu().numpy(), g["kv_write.cache"])
    assert np.array_equal(u16(sc), g["kv_write.scale"])


@pytest.mark.parametrize("ring,S", [(False, 40), (True, 8), (True, 256)])
def test_kv_append_matches_oracle(ring, S):
    from ultraviolet_b200.kernels import kv_append
    r = np.random.default_rng(5)
    B, KH, hd = 7, 2, 64
    k = T(r.standard_normal((B, KH, hd)).astype(np.float32), torch.bfloat16)
    v = T(r.standard_normal((B, KH, hd)).astype(np.float32), torch.bfloat16)
    pos = r.integers(0, 1000 if ring else S, B)
    kc = torch.zeros(B, KH, S, hd, dtype=torch.int8, device=DEV)
    vc, ks, vs = torch.zeros_like(kc), torch.zeros(B, KH, S, dtype=torch.float16, device=DEV), None
    vs = torch.zeros_like(ks)
    kv_append(kc, vc, ks, vs, T(pos), k, v, ring)
    rk, rv = np.zeros((B, KH, S, hd), np.int8), np.zeros((B, KH, S, hd), np.int8)
    rks, rvs = np.zeros((B, KH, S), np.float16), np.zeros((B, KH, S), np.float16)
    slot = pos % S if ring else pos
    idx = ((np.arange(B)[:, None] * KH + np.arange(KH)[None]) * S + slot[:, None]).reshape(-1)
    okv.kv_write(rk, rks, idx, k.float().cpu().numpy())
    okv.kv_write(rv, rvs, idx, v.float().cpu().numpy())
    assert np.array_equal(kc.cpu().numpy(), rk) and np.array_equal(vc.cpu().numpy(), rv)
    assert np.array_equal(u16(ks), rks.view(np.uint16)) and np.array_equal(u16(vs), rvs.view(np.uint16))


# ------------------------------------------------------------------------------------------------ attention
def _quant(c):
    kq, ks = okv.quantize_kv(c["k"])
    vq, vs = okv.quantize_kv(c["v"])
    return T(kq), T(ks), T(vq), T(vs)


def _close(out, ref, rel):
    out, ref = out.float().cpu().numpy(), np.asarray(ref, np.float32)
    assert np.isfinite(out).all()
    err = np.abs(out - ref)
    assert err.max() <= rel * max(np.abs(ref).max(), 1e-6), (err.max(), np.abs(ref).max())
    np.testing.assert_allclose(out, ref, rtol=rel, atol=rel * 0.25)


def test_config1_bytes_and_attention():
    from ultraviolet_b200.kernels import decode_attention, quantize_kv
    g = golden("attn")
    c = gi.config1()
    kq, ks = quantize_kv(T(c["k"]))
    vq, vs = quantize_kv(T(c["v"]))
    for n, a in (("kq", kq.cpu().numpy()), ("ks", ks.cpu().numpy()), ("vq", vq.cpu().numpy()),
                 ("vs", vs.cpu().numpy())):
        assert gi.sha(a) == str(g[f"config1.{n}_sha"]), n        # int8 bytes and fp16 scales bit-exact
    pos, starts = T(c["lens"] - 1), torch.zeros(16, dtype=torch.long, device=DEV)
    for dtype, rel in ((torch.float16, 2e-3), (torch.bfloat16, 2e-2)):
        q = T(c["q"], dtype)
        for splits in (1, 2, None):
            out = decode_attention(q, kq, vq, pos, starts, 0.14125, k_scale=ks, v_scale=vs, num_splits=splits)
            assert out.dtype == dtype and out.shape == (16, 8, 64)
            _close(out, g["config1.global"], 2e-2 if dtype == torch.bfloat16 else 4e-3)  # vs fp32-query reference
            ref = oattn.decode_attention_ref(q.float().cpu().numpy(), kq.cpu().numpy(), vq.cpu().numpy(),
                                             c["lens"] - 1, np.zeros(16, np.int64), 0.14125,
                                             k_scale=ks.cpu().numpy(), v_scale=vs.cpu().numpy())
            _close(out, ref, 8e-3 if dtype == torch.bfloat16 else rel)           # vs oracle on the same rounded q
        out = decode_attention(q, kq[:, :, :256].contiguous(), vq[:, :, :256].contiguous(), pos, starts, 0.14125,
                               window=256, k_scale=ks[:, :, :256].contiguous(), v_scale=vs[:, :, :256].contiguous())
        _close(out, g["config1.local"], 2e-2 if dtype == torch.bfloat16 else 4e-3)


GRID = [n for n, c in gi.attn_cases().items() if c["int8"]]


# 2..8 splits merge inside a thread-block cluster (short rows leave some of its CTAs without tiles), more than 8
# through the workspace and the arrival counters
@pytest.mark.parametrize("splits", [1, 3, 8, 12, None])
@pytest.mark.parametrize("name", sorted(GRID))
def test_attention_grid_int8(name, splits):
    from ultraviolet_b200.kernels import decode_attention
    g = golden("attn")
    c = gi.attn_cases()[name]
    kq, ks, vq, vs = _quant(c)
    q = T(c["q"], torch.float16)
    pos, starts = T(c["pos"]), T(c["starts"])
    if name == "slice.i8":  # cache[:, :, :g_len] views keep the parent strides
        kq, vq, ks, vs = kq[:, :, :256], vq[:, :, :256], ks[:, :, :256], vs[:, :, :256]
    out = decode_attention(q, kq, vq, pos, starts, c["scale"], window=c["window"], ring=c["ring"], k_scale=ks,
                           v_scale=vs, num_splits=splits)
    np.testing.assert_allclose(out.float().cpu().numpy(), g[name], atol=2e-3, rtol=2e-3)


# Ring lengths that are not a multiple of the 128-key tile: multiples of 8 stay on the bulk-copy path (the tile that
# crosses slot S - 1 arrives in two pieces), the others take the two-stage cp.async path.  Positions wrap the ring
# several times (reference grid: tests/test_math_kernels.py:55-70).
@pytest.mark.parametrize("splits", [1, 2, None])
@pytest.mark.parametrize("S,bulk", [(136, 1), (192, 1), (200, 1), (104, 1), (8, 1), (100, 0), (189, 0), (255, 0)])
def test_attention_ring_lengths(S, bulk, splits):
    import ctypes as C
    from ultraviolet_b200 import _lib
    from ultraviolet_b200.kernels import decode_attention
    from ultraviolet_b200.kernels.decode_attn import attn_args
    r = np.random.default_rng(S)
    B, H, hd = 12, 8, 64
    k = r.standard_normal((B, 1, S, hd)).astype(np.float32)
    v = r.standard_normal((B, 1, S, hd)).astype(np.float32)
    kq, ks = okv.quantize_kv(k)
    vq, vs = okv.quantize_kv(v)
    pos = np.concatenate([[0, S - 1, S, S + 1, 2 * S - 1, 2 * S, 5 * S + 3], r.integers(0, 6 * S, B - 7)]).astype(np.int64)
    starts = np.where(r.random(B) < 0.5, 0, np.maximum(pos - r.integers(0, S, B), 0)).astype(np.int64)
    window = S - 3 if S > 16 else S
    q = T(r.standard_normal((B, H, hd)).astype(np.float32), torch.float16)
    tk, tv, tks, tvs = T(kq), T(vq), T(ks), T(vs)
    out = decode_attention(q, tk, tv, T(pos), T(starts), 0.14125, window=window, ring=True, k_scale=tks, v_scale=tvs,
                           num_splits=splits)
    ref = oattn.decode_attention_ref(q.float().cpu().numpy(), kq, vq, pos, starts, 0.14125, window=window, ring=True,
                                     k_scale=ks, v_scale=vs)
    np.testing.assert_allclose(out.float().cpu().numpy(), ref, atol=2e-3, rtol=2e-3)
    a = attn_args(q, tk, tv, T(pos), T(starts), 0.14125, window, True, tks, tvs, 1, out)
    assert _lib.lib().uv_decode_attn_uses_bulk(C.byref(a)) == bulk


def test_attention_q_view_and_bf16():
    from ultraviolet_b200.kernels import decode_attention
    c = gi.attn_cases()["uv.global"]
    kq, ks, vq, vs = _quant(c)
    q4 = T(c["q"], torch.bfloat16).view(c["B"], 1, 8, 64)
    out = decode_attention(q4, kq, vq, T(c["pos"]), T(c["starts"]), c["scale"], k_scale=ks, v_scale=vs)
    ref = oattn.decode_attention_ref(q4.float().cpu().numpy(), kq.cpu().numpy(), vq.cpu().numpy(), c["pos"],
                                     c["starts"], c["scale"], k_scale=ks.cpu().numpy(), v_scale=vs.cpu().numpy())
    _close(out, ref, 8e-3)


def test_attention_errors_are_loud():
    from ultraviolet_b200 import _lib
    from ultraviolet_b200.kernels import decode_attention
    q = torch.zeros(2, 8, 64, dtype=torch.float16)
    with pytest.raises(RuntimeError):
        decode_attention(q, q, q, q, q, 1.0)                       # CPU tensors: no fallback
    qc = q.to(DEV)
    kc = torch.zeros(2, 1, 64, 48, dtype=torch.int8, device=DEV)   # head_dim 48 is not compiled
    sc = torch.zeros(2, 1, 64, dtype=torch.float16, device=DEV)
    z = torch.zeros(2, dtype=torch.long, device=DEV)
    with pytest.raises(_lib.UvError):
        decode_attention(qc[:, :, :48].contiguous(), kc, kc, z, z, 1.0, k_scale=sc, v_scale=sc)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("splits", [1, 4, 7, 10])
def test_fused_xsa_gate_epilogue(dtype, splits):
    """Attention + XSA + head gate in one launch == oracle attention followed by Attention.post's elementwise part."""
    from ultraviolet_b200.kernels.decode_attn import attn_launch, workspace_for
    c = gi.attn_cases()["uv.global"]
    B, H, hd = c["B"], 8, 64
    kq, ks, vq, vs = _quant(c)
    r = np.random.default_rng(9)
    q = T(c["q"], dtype)
    v_cur = T(r.standard_normal((B, 1, hd)).astype(np.float32), dtype)
    xn = T(r.standard_normal((B, 640)).astype(np.float32), dtype)
    gate_w = T(r.standard_normal((H, 128)).astype(np.float32) * 0.3, dtype)
    alpha = T(np.tanh(r.standard_normal(H).astype(np.float32) * 0.3))
    out = torch.empty_like(q)
    ws = workspace_for(B, 1, H, hd, splits, DEV)
    cnt = torch.zeros(B, dtype=torch.int32, device=DEV)  # last-arriving split merges in the same launch
    attn_launch(q, kq, vq, T(c["pos"]), T(c["starts"]), c["scale"], 0, False, ks, vs, splits, out, ws,
                v_cur=v_cur, xsa_alpha=alpha, xsa_eps=1e-4, gate_x=xn, gate_w=gate_w, counters=cnt)
    assert int(cnt.abs().sum()) == 0  # counters are left zeroed for the next launch
    f = lambda t: t.float().cpu().numpy()
    z = oattn.decode_attention_ref(f(q), f(kq).astype(np.int8), f(vq).astype(np.int8), c["pos"], c["starts"],
                                   c["scale"], k_scale=ks.cpu().numpy(), v_scale=vs.cpu().numpy())
    v = f(v_cur)
    vd = v / np.maximum(np.sqrt((v * v).sum(-1, keepdims=True)), 1e-4)
    z = z - f(alpha)[None, :, None] * (z * vd).sum(-1, keepdims=True) * vd
    gate = 2.0 / (1.0 + np.exp(-(f(xn)[:, :128] @ f(gate_w).T)))
    _close(out, z * gate[..., None], 2.5e-2 if dtype == torch.bfloat16 else 6e-3)


# ------------------------------------------------------------------------------------------------ sampler
def _sample(x, **kw):
    """uv_sample through the engine-independent raw binding."""
    import ctypes as C
    from ultraviolet_b200 import _lib
    from ultraviolet_b200.kernels._util import DTYPE_CODE, stream_ptr
    B, V = x.shape
    tok = torch.empty(B, dtype=torch.int64, device=DEV)
    lp = torch.empty(B, dtype=torch.float32, device=DEV)
    p = lambda t: None if t is None else t.data_ptr()
    cap = kw.get("cap", (23.0, 5.0, 7.5))
    if "top_k" in kw:
        rc = _lib.lib().uv_sample_topk(x.data_ptr(), DTYPE_CODE[x.dtype], x.stride(0), B, V,
                                       int(kw.get("precapped", False)), cap[0], cap[1], cap[2], kw.get("T", 1.0),
                                       int(kw["top_k"]), kw.get("top_p", 1.0), p(kw.get("u")),
                                       C.c_uint64(kw.get("seed", 0)), p(kw.get("row_keys")), p(kw.get("steps")),
                                       tok.data_ptr(), lp.data_ptr(), None, None, stream_ptr(torch.device(DEV)))
    else:
        rc = _lib.lib().uv_sample(x.data_ptr(), DTYPE_CODE[x.dtype], x.stride(0), B, V,
                                  int(kw.get("precapped", False)), cap[0], cap[1], cap[2], kw.get("T", 1.0),
                                  kw.get("top_p", 1.0), p(kw.get("u")), C.c_uint64(kw.get("seed", 0)),
                                  p(kw.get("row_keys")), p(kw.get("steps")), tok.data_ptr(), lp.data_ptr(), None,
                                  None, stream_ptr(torch.device(DEV)))
    _lib.check(rc, "uv_sample")
    return tok.cpu().numpy(), lp.cpu().numpy()


def _cdf64(x, cap, T):
    a, b, c = cap
    z = a / (1.0 + np.exp(-(x.astype(np.float64) + b) / c))
    e = np.exp((z - a) / T)
    return z, e, np.cumsum(e, -1)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_fused_sample_matches_reference_golden_and_cdf(dtype):
    g = golden("sampler")
    x, u, cap, temps = gi.fused_sample_case()
    xt = T(x, dtype)
    xr = xt.float().cpu().numpy()
    for t in temps:
        tok, lp = _sample(xt, u=T(u), T=t)
        z, e, cs = _cdf64(xr, cap, t)
        S = cs[:, -1]
        target = (1.0 - u.astype(np.float64)) * S
        lo = np.where(tok > 0, cs[np.arange(len(tok)), np.maximum(tok - 1, 0)], 0.0)
        hi = cs[np.arange(len(tok)), tok]
        # the drawn token's CDF interval contains the target up to fp32 summation error (tests/test_perf_fz.py:95-119)
        assert (target >= lo - 1e-5 * S).all() and (target <= hi + 1e-5 * S).all()
        ref_lp = (z[np.arange(len(tok)), tok] - cap[0]) / t - np.log(S)
        np.testing.assert_allclose(lp, ref_lp, atol=3e-5)
        if dtype == torch.float16:  # the golden inputs are fp16 values: compare with the reference's own tokens
            # row 0 has u = 0: the target is the total itself and the winner is whichever index first reaches it
            # in each implementation's own fp32 summation order (the interval test above still holds for it)
            assert (np.abs(tok - g[f"fused.tok.T{t}"])[1:] <= 1).all()


def test_greedy_argmax_and_logp():
    r = np.random.default_rng(3)
    x = T(r.standard_normal((9, 16384)).astype(np.float32) * 3, torch.bfloat16)
    x[2, 100] = x[2].max() + 1
    x[2, 7000] = x[2, 100]          # a tie: the first index wins
    tok, lp = _sample(x, T=0.0)
    xr = x.float().cpu().numpy()
    z, e, cs = _cdf64(xr, (23.0, 5.0, 7.5), 1.0)
    assert np.array_equal(tok, z.astype(np.float32).argmax(-1)) and tok[2] == 100
    np.testing.assert_allclose(lp, z[np.arange(9), tok] - 23.0 - np.log(cs[:, -1]), atol=3e-5)


def test_sampler_distribution_and_top_p():
    """Chi-square of 2^16 draws against softmax(z / T) (tests/test_perf_fz.py:122-134) and nucleus support."""
    from scipy import stats
    r = np.random.default_rng(4)
    V, N = 256, 1 << 16
    row = (r.standard_normal(V) * 2).astype(np.float32)
    x = T(np.tile(row, (N, 1)))
    u = torch.rand(N, device=DEV, generator=torch.Generator(DEV).manual_seed(5))
    tok, _ = _sample(x, u=u, T=0.9, precapped=True)
    p = np.exp(row.astype(np.float64) / 0.9)
    p /= p.sum()
    cnt = np.bincount(tok, minlength=V)
    keep = p * N >= 5
    chi = (((cnt - p * N) ** 2 / (p * N))[keep]).sum()
    assert stats.chi2.sf(chi, keep.sum() - 1) > 1e-3
    tok, lp = _sample(x, u=u, T=0.9, top_p=0.7, precapped=True)
    nucleus = om.top_p_keep(row[None], 0.9, 0.7)[0]
    assert nucleus[np.unique(tok)].all()                       # never outside the reference's nucleus
    assert set(np.flatnonzero(nucleus & (p > 1e-3))) <= set(np.unique(tok))
    np.testing.assert_allclose(lp, np.log(p[tok]), atol=3e-5)  # log-prob stays untruncated


def test_top_k_support_and_renormalised_nucleus():
    """top_k of sample() (ultraviolet/model.py:1201-1203): only the k largest logits, ties with the k-th kept, can be
    drawn; top_p then acts on the renormalised top-k set; the log-prob stays untruncated."""
    r = np.random.default_rng(8)
    V, N, k, temp = 256, 1 << 14, 5, 0.9
    row = (r.standard_normal(V) * 2).astype(np.float32)
    order = np.argsort(-row)
    row[order[5]] = row[order[4]]            # a tie at the k-th rank: both stay
    x = T(np.tile(row, (N, 1)))
    u = torch.rand(N, device=DEV, generator=torch.Generator(DEV).manual_seed(9))
    tok, lp = _sample(x, u=u, T=temp, precapped=True, top_k=k)
    kth = np.sort(row)[-k]
    keep = row >= kth
    assert keep.sum() == 6 and set(np.unique(tok)) == set(np.flatnonzero(keep))
    p = np.exp(row.astype(np.float64) / temp)
    p /= p.sum()
    np.testing.assert_allclose(lp, np.log(p[tok]), atol=3e-5)
    pk = np.where(keep, p, 0) / p[keep].sum()
    cnt = np.bincount(tok, minlength=V)
    from scipy import stats
    chi = (((cnt - pk * N) ** 2 / np.maximum(pk * N, 1e-30))[keep]).sum()
    assert stats.chi2.sf(chi, keep.sum() - 1) > 1e-3
    # top_k then top_p: the nucleus of the renormalised top-k distribution (reference order of the two filters)
    tok2, _ = _sample(x, u=u, T=temp, precapped=True, top_k=k, top_p=0.6)
    masked = np.where(keep, row, -np.inf)[None]
    nucleus = om.top_p_keep(masked, temp, 0.6)[0]
    assert nucleus[np.unique(tok2)].all() and nucleus.sum() < keep.sum()
    # k >= V and k = 0 are no-ops
    a, _ = _sample(x[:64], u=u[:64], T=temp, precapped=True, top_k=0)
    b, _ = _sample(x[:64], u=u[:64], T=temp, precapped=True, top_k=V)
    assert np.array_equal(a, b)


def test_philox_keyed_draws_match_oracle():
    from oracle import philox
    r = np.random.default_rng(6)
    x = T(r.standard_normal((16, 4096)).astype(np.float32) * 3, torch.bfloat16)
    keys = torch.arange(100, 116, device=DEV)
    steps = torch.arange(16, device=DEV) * 3
    tok, lp = _sample(x, T=1.0, seed=1234567, row_keys=keys, steps=steps)
    u = np.array([philox.uniform(1234567, 100 + i, 3 * i) for i in range(16)], np.float32)
    tok_u, lp_u = _sample(x, T=1.0, u=T(u))
    assert np.array_equal(tok, tok_u) and np.array_equal(lp, lp_u)
    tok2, _ = _sample(x.flip(0).contiguous(), T=1.0, seed=1234567, row_keys=keys.flip(0).contiguous(),
                      steps=steps.flip(0).contiguous())
    assert np.array_equal(tok2[::-1], tok)   # a sequence's draw does not depend on the row it sits in


# ------------------------------------------------------------------------------------------------ fused QKV + attention
def _qkv_attn_case(dtype, ring, splits, rope, ve, fused, G=8, hd=64, seed=0, gate_pre=False):
    """One layer's uv_qkv_post + uv_decode_attn (fused=False) or uv_qkv_attn (fused=True) on identical inputs.
    Returns (attention output, k cache, v cache, k scales, v scales)."""
    import ctypes as C
    from ultraviolet_b200 import _lib
    from ultraviolet_b200.kernels._util import DTYPE_CODE
    from ultraviolet_b200.kernels.decode_attn import attn_launch, workspace_for
    r = np.random.default_rng(seed)
    B, H, K, d, vocab = 12, G, 1, 640, 512
    S = 256 if ring else 1024
    window = 256 if ring else 0
    slots = H + 2 * K
    # positions that sit on, just before and just after 128-key tile edges; row 0 is a fresh sequence
    pos_np = np.array([0, 5, 127, 128, 129, 255, 256, 383, 384, 600, 777, 1000], np.int64)
    starts_np = np.array([0, 2, 0, 100, 0, 130, 0, 0, 300, 0, 512, 0], np.int64)
    rows_np = r.permutation(16)[:B].astype(np.int64)  # batch entries live in arbitrary rows of a 16-row cache
    kc = T(r.integers(-127, 128, (16, K, S, hd)).astype(np.int8))
    vc = T(r.integers(-127, 128, (16, K, S, hd)).astype(np.int8))
    ks = T((r.random((16, K, S)) * 0.02 + 0.005).astype(np.float16))
    vs = T((r.random((16, K, S)) * 0.02 + 0.005).astype(np.float16))
    qkv = T(r.standard_normal((B, slots * hd)).astype(np.float32), dtype)
    xn = T(r.standard_normal((B, d)).astype(np.float32), dtype)
    tok = T(r.integers(0, vocab, B).astype(np.int64))
    vemb = T(r.standard_normal((vocab, K * hd)).astype(np.float32), dtype)
    vgate = T(r.standard_normal((K, 12)).astype(np.float32) * 0.3, dtype)
    inv_freq = T((1024.0 ** (-np.arange(16) / 16.0)).astype(np.float32))
    gate_w = T(r.standard_normal((H, 128)).astype(np.float32) * 0.3, dtype)
    alpha = T(np.tanh(r.standard_normal(H).astype(np.float32) * 0.3))
    pos, starts, rows = T(pos_np), T(starts_np), T(rows_np)
    oob = torch.zeros(1, dtype=torch.int32, device=DEV)
    post = (tok.data_ptr(), vemb.data_ptr() if ve else None, vgate.data_ptr() if ve else None,
            inv_freq.data_ptr() if rope else None, pos.data_ptr(), kc.data_ptr(), vc.data_ptr(), ks.data_ptr(),
            vs.data_ptr(), rows.data_ptr(), oob.data_ptr(), DTYPE_CODE[dtype], vocab, B, H, K, hd, d, S, S,
            int(ring), 12, 16)
    q3 = qkv.view(B, slots, hd)
    out = torch.empty(B, H, hd, dtype=dtype, device=DEV)
    ws = workspace_for(B, K, G, hd, splits, DEV)
    cnt = torch.zeros(B * K, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    pre = None
    raw = qkv.clone()
    if fused:
        pre = _lib.QkvArgs()
        (pre.qkv, pre.xn, pre.tok, pre.value_embed, pre.ve_gate, pre.inv_freq, pre.pos, pre.k_cache, pre.v_cache,
         pre.k_scale, pre.v_scale, pre.row_map, pre.oob_count, pre.dtype, pre.vocab, pre.B, pre.H, pre.K, pre.hd,
         pre.d, pre.S, pre.S_alloc, pre.ring, pre.ve_ch, pre.n_pairs) = (qkv.data_ptr(), xn.data_ptr(), *post)
        if rope:  # the step's cos / sin table, as the engine gets it from the kernel that opens the step
            emb = torch.zeros(vocab, d, dtype=dtype, device=DEV)
            x0, x1 = torch.empty(B, d, dtype=dtype, device=DEV), torch.empty(B, d, dtype=dtype, device=DEV)
            cs = torch.zeros(B, 32, dtype=torch.float32, device=DEV)
            _lib.check(_lib.lib().uv_embed_norm_rope(tok.data_ptr(), emb.data_ptr(), DTYPE_CODE[dtype], vocab, d,
                                                     x0.data_ptr(), x1.data_ptr(), B, pos.data_ptr(),
                                                     inv_freq.data_ptr(), 16, cs.data_ptr(),
                                                     torch.cuda.current_stream().cuda_stream), "uv_embed_norm_rope")
            pre.rope_cs = cs.data_ptr()
    elif gate_pre:  # parameters by name; the kernel also leaves the head gates for the attention launch
        qa = _lib.QkvArgs()
        (qa.qkv, qa.xn, qa.tok, qa.value_embed, qa.ve_gate, qa.inv_freq, qa.pos, qa.k_cache, qa.v_cache, qa.k_scale,
         qa.v_scale, qa.row_map, qa.oob_count, qa.dtype, qa.vocab, qa.B, qa.H, qa.K, qa.hd, qa.d, qa.S, qa.S_alloc,
         qa.ring, qa.ve_ch, qa.n_pairs) = (qkv.data_ptr(), xn.data_ptr(), *post)
        gates = torch.zeros(B, H, dtype=torch.float32, device=DEV)
        qa.gate_w, qa.gate_out, qa.gate_ch = gate_w.data_ptr(), gates.data_ptr(), 128
        _lib.check(_lib.lib().uv_qkv_post_args(C.byref(qa), torch.cuda.current_stream().cuda_stream),
                   "uv_qkv_post_args")
    else:
        _lib.check(_lib.lib().uv_qkv_post(qkv.data_ptr(), xn.data_ptr(), *post,
                                          torch.cuda.current_stream().cuda_stream), "uv_qkv_post")
    attn_launch(q3[:, :H], kc, vc, pos, starts, 0.14125, window, ring, ks, vs, splits, out, ws,
                v_cur=q3[:, H + K:], xsa_alpha=alpha, xsa_eps=1e-4, gate_x=xn, gate_w=gate_w, counters=cnt,
                status=status, row_map=rows, pre=pre, gate_vals=gates if gate_pre and not fused else None)
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and int(cnt.abs().sum()) == 0
    # the one-launch form reads the projection and leaves it alone; the two-launch form rewrites it in place
    assert torch.equal(raw, qkv) == fused
    return out, kc, vc, ks, vs, int(oob.item())


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("ring,rope,ve", [(True, True, True), (True, True, False), (False, False, True),
                                          (False, False, False)])
@pytest.mark.parametrize("splits", [1, 3, 8, 11])
def test_qkv_attn_one_launch_equals_two(dtype, ring, rope, ve, splits):
    """uv_qkv_attn == uv_qkv_post then uv_decode_attn: cache bytes and scales bit-identical, outputs identical."""
    a = _qkv_attn_case(dtype, ring, splits, rope, ve, fused=False)
    b = _qkv_attn_case(dtype, ring, splits, rope, ve, fused=True)
    for x, y, name in zip(a[1:5], b[1:5], ("k", "v", "k_scale", "v_scale")):
        assert torch.equal(x, y), name
    assert a[5] == b[5]  # rows past the end of a linear cache are counted, not written, either way
    assert torch.equal(a[0], b[0])


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_head_gates_from_qkv_post_equal_epilogue_gates(dtype):
    a = _qkv_attn_case(dtype, True, 1, True, True, fused=False)
    b = _qkv_attn_case(dtype, True, 1, True, True, fused=False, gate_pre=True)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]) and torch.equal(a[2], b[2])


def test_qkv_attn_group16_and_small_heads():
    for G, hd in ((16, 64), (8, 32), (4, 128)):
        a = _qkv_attn_case(torch.bfloat16, True, 2, True, True, fused=False, G=G, hd=hd, seed=G + hd)
        b = _qkv_attn_case(torch.bfloat16, True, 2, True, True, fused=True, G=G, hd=hd, seed=G + hd)
        assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]) and torch.equal(a[2], b[2])


# ------------------------------------------------------------------------------------------------ prefill-time writes
def test_kv_write_rows_all_index_forms():
    """kv_write_rows (kv_quant.py:39-54): whole batch, a row subset with a slice of slots, a row subset with a
    tensor of slots (the local-ring write of the last 256 positions) -- against the oracle's restatement."""
    from ultraviolet_b200.kernels import kv_write_rows
    r = np.random.default_rng(11)
    B, K, S, hd = 6, 2, 40, 64
    base_c = r.integers(-127, 128, (B, K, S, hd)).astype(np.int8)
    base_s = (r.random((B, K, S)) * 0.02).astype(np.float16)
    cases = [
        (None, slice(3, 19), r.standard_normal((B, K, 16, hd)).astype(np.float32)),
        (np.array([4, 1, 5]), slice(0, 7), r.standard_normal((3, K, 7, hd)).astype(np.float32) * 3),
        (np.array([2, 0]), np.array([39, 0, 1, 17, 5]), r.standard_normal((2, K, 5, hd)).astype(np.float32)),
    ]
    for rows, slots, new in cases:
        c_ref, s_ref = base_c.copy(), base_s.copy()
        okv.kv_write_rows(c_ref, s_ref, new, slots, rows)
        c, s = T(base_c), T(base_s)
        kv_write_rows(c, s, T(new), slots if isinstance(slots, slice) else T(slots),
                      None if rows is None else T(rows))
        assert np.array_equal(c.cpu().numpy(), c_ref)
        assert np.array_equal(u16(s), s_ref.view(np.uint16))


def test_decode_attention_is_a_registered_custom_op():
    """The reference registers its launch as a custom op with a fake implementation so that graph capture and
    tracing keep working (decode_attn.py:174-190); the same holds here."""
    from ultraviolet_b200.kernels import decode_attention
    assert hasattr(torch.ops.uvb200, "decode_attn")
    c = gi.attn_cases()["uv.global"]
    kq, ks, vq, vs = _quant(c)
    q = T(c["q"], torch.float16)
    args = (q, kq, vq, T(c["pos"]), T(c["starts"]), c["scale"], 0, False, ks, vs, 2)
    torch.library.opcheck(torch.ops.uvb200.decode_attn.default, args,
                          test_utils=("test_schema", "test_faketensor"))
    # and the launch is capturable: a replay reproduces the eager result
    eager = decode_attention(q, kq, vq, T(c["pos"]), T(c["starts"]), c["scale"], k_scale=ks, v_scale=vs, num_splits=2)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        decode_attention(q, kq, vq, T(c["pos"]), T(c["starts"]), c["scale"], k_scale=ks, v_scale=vs, num_splits=2)
    torch.cuda.current_stream().wait_stream(side)
    g = torch.cuda.CUDAGraph()
    pos, starts = T(c["pos"]), T(c["starts"])
    with torch.cuda.graph(g):
        out = decode_attention(q, kq, vq, pos, starts, c["scale"], k_scale=ks, v_scale=vs, num_splits=2)
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager)


# ------------------------------------------------------------------------------------------------ full-size properties
def _long_context_inputs(B=64, ctx=8192, seed=1):
    """The long-context stress shape: B sequences with int8 KV filled to ctx tokens from N(0, 1)."""
    from ultraviolet_b200.kernels import quantize_kv
    g = torch.Generator(device=DEV).manual_seed(seed)
    S = ctx + 256
    k = torch.randn(B, 1, S, 64, device=DEV, generator=g)
    v = torch.randn(B, 1, S, 64, device=DEV, generator=g)
    kq, ks = quantize_kv(k)
    vq, vs = quantize_kv(v)
    q = torch.randn(B, 8, 64, device=DEV, generator=g).half()
    pos = torch.full((B,), ctx - 1, device=DEV, dtype=torch.long)
    pos[::7] -= torch.arange(0, B, 7, device=DEV) * 37          # ragged: some rows are shorter
    starts = torch.zeros(B, dtype=torch.long, device=DEV)
    starts[::5] = 1000
    return q, kq, ks, vq, vs, pos, starts


def test_long_context_full_size_properties():
    """64 sequences x 8192 keys, where the oracle is too slow for every row: (1) the result does not depend on the
    split count (1, the 8-split cluster merge, the 12-split workspace merge); (2) three rows against the oracle;
    (3) linearity in V: doubling every V scale doubles the output; (4) a window equal to the whole context changes
    nothing."""
    from ultraviolet_b200.kernels import decode_attention
    q, kq, ks, vq, vs, pos, starts = _long_context_inputs()
    outs = {s: decode_attention(q, kq, vq, pos, starts, 0.14125, k_scale=ks, v_scale=vs, num_splits=s)
            for s in (1, 8, 12)}
    for s in (8, 12):
        torch.testing.assert_close(outs[s].float(), outs[1].float(), atol=2e-3, rtol=2e-3)
    rows = [0, 7, 35]  # a full row, two ragged ones (row 35 also starts at 1000)
    ref = oattn.decode_attention_ref(q[rows].float().cpu().numpy(), kq[rows].cpu().numpy(), vq[rows].cpu().numpy(),
                                     pos[rows].cpu().numpy(), starts[rows].cpu().numpy(), 0.14125,
                                     k_scale=ks[rows].cpu().numpy(), v_scale=vs[rows].cpu().numpy())
    np.testing.assert_allclose(outs[8][rows].float().cpu().numpy(), ref, atol=2e-3, rtol=2e-3)
    dbl = decode_attention(q, kq, vq, pos, starts, 0.14125, k_scale=ks, v_scale=vs * 2, num_splits=8)
    torch.testing.assert_close(dbl.float(), 2 * outs[8].float(), atol=4e-3, rtol=2e-3)
    win = decode_attention(q, kq, vq, pos, starts, 0.14125, window=8192, k_scale=ks, v_scale=vs, num_splits=8)
    assert torch.equal(win, outs[8])


def test_appended_key_changes_only_its_row():
    """kv_append of one new key per row followed by attention at pos + 1 equals attention over a cache that was
    quantised with that key in place from the start (the append is the quantiser, bit for bit)."""
    from ultraviolet_b200.kernels import decode_attention, kv_append, quantize_kv
    g = torch.Generator(device=DEV).manual_seed(5)
    B, S = 32, 2048
    k = torch.randn(B, 1, S, 64, device=DEV, generator=g)
    v = torch.randn(B, 1, S, 64, device=DEV, generator=g)
    q = torch.randn(B, 8, 64, device=DEV, generator=g).half()
    pos = torch.randint(100, S - 1, (B,), device=DEV, generator=g)
    starts = torch.zeros(B, dtype=torch.long, device=DEV)
    kq, ks = quantize_kv(k)
    vq, vs = quantize_kv(v)
    full = decode_attention(q, kq, vq, pos, starts, 0.14125, k_scale=ks, v_scale=vs)
    # wipe the entry at pos, then append it again from the unquantised vectors
    idx = pos.view(B, 1, 1, 1).expand(B, 1, 1, 64)
    kq2, vq2, ks2, vs2 = kq.clone(), vq.clone(), ks.clone(), vs.clone()
    kq2.scatter_(2, idx, 0), vq2.scatter_(2, idx, 0)
    ks2.scatter_(2, pos.view(B, 1, 1), 0), vs2.scatter_(2, pos.view(B, 1, 1), 0)
    knew = k.gather(2, idx).squeeze(2)
    vnew = v.gather(2, idx).squeeze(2)
    kv_append(kq2, vq2, ks2, vs2, pos, knew, vnew, ring=False)
    assert torch.equal(kq2, kq) and torch.equal(vq2, vq) and torch.equal(ks2, ks) and torch.equal(vs2, vs)
    again = decode_attention(q, kq2, vq2, pos, starts, 0.14125, k_scale=ks2, v_scale=vs2)
    assert torch.equal(again, full)


def test_default_splits_with_the_references_knobs():
    """default_splits without min_chunk / waves is the library's heuristic; with either of them it is the reference's
    rule (decode_attn.py:121-129) on those values."""
    from ultraviolet_b200.kernels import default_splits
    n_sm = torch.cuda.get_device_properties(0).multi_processor_count
    ref = lambda n_bk, ctx, mc, w: max(1, min(-(-w * n_sm // max(n_bk, 1)), max(1, ctx // mc), 64))
    for n_bk, ctx, mc, w in ((64, 8192, 128, 8), (256, 256, 64, 4), (1, 100000, 128, 8), (4096, 512, 128, 8)):
        assert default_splits(n_bk, ctx, "cuda", min_chunk=mc, waves=w) == ref(n_bk, ctx, mc, w)
    assert default_splits(64, 8192, "cuda", waves=4) == ref(64, 8192, 128, 4)
    assert default_splits(64, 8192, "cuda") == 8 if n_sm == 148 else default_splits(64, 8192, "cuda") >= 1


@pytest.mark.parametrize("splits", [1, 3])
def test_rows_without_a_valid_key_give_zeros_and_leave_the_others_alone(splits):
    """Edge case of the ragged batch: rows whose key range is empty (starts > pos) produce zeros, with or without a
    split merge, and every other row of the launch equals the launch without them."""
    from ultraviolet_b200.kernels import decode_attention, quantize_kv
    g = torch.Generator(device=DEV).manual_seed(9)
    B, S = 12, 640
    k = torch.randn(B, 1, S, 64, device=DEV, generator=g)
    v = torch.randn(B, 1, S, 64, device=DEV, generator=g)
    q = torch.randn(B, 8, 64, device=DEV, generator=g).half()
    kq, ks = quantize_kv(k)
    vq, vs = quantize_kv(v)
    pos = torch.randint(50, S, (B,), device=DEV, generator=g)
    starts = torch.zeros(B, dtype=torch.long, device=DEV)
    full = decode_attention(q, kq, vq, pos, starts, 0.14125, k_scale=ks, v_scale=vs, num_splits=splits)
    empty = [1, 6, 11]
    starts2 = starts.clone()
    starts2[empty] = pos[empty] + 1
    out = decode_attention(q, kq, vq, pos, starts2, 0.14125, k_scale=ks, v_scale=vs, num_splits=splits)
    keep = [b for b in range(B) if b not in empty]
    assert torch.equal(out[keep], full[keep])
    assert torch.isfinite(out).all() and (out[empty] == 0).all()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_sampler_edges_of_the_uniform(dtype):
    """The reference sampler's edge cases (tests/test_perf_fz.py:66-71): with (almost) all of the mass on one token,
    u -> 1 (target -> 0) and u = 0 (target = the whole sum) still give valid ids with finite log-probs -- the softcap
    leaves every other token a mass of about 1e-9 of the total, so the extreme targets may land on those -- and any
    u away from the ends draws the token that holds the mass, wherever it sits in the vocabulary."""
    from ultraviolet_b200.kernels import fused_sample
    V = 4096
    for hot in (0, 40, 2047, 2048, V - 1):
        x = torch.full((5, V), -1e4, device=DEV, dtype=dtype)
        x[:, hot] = 10.0
        u = torch.tensor([0.0, 1.0 - 2.0 ** -24, 0.5, 1e-3, 0.999], device=DEV)
        tok, lp = fused_sample(x, u, (23.0, 5.0, 7.5), 1.0)
        assert int(tok.min()) >= 0 and int(tok.max()) < V
        assert tok[2:].tolist() == [hot] * 3
        assert torch.isfinite(lp).all() and (lp <= 0).all() and (lp[2:] > -1e-3).all()
        if hot == 0:
            assert int(tok[1]) == 0          # target -> 0: the first token that has any mass
