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


@pytest.mark.parametrize("splits", [1, 3, None])
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
@pytest.mark.parametrize("splits", [1, 4])
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
