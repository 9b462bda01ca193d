"""Packed varlen prefill: the attention kernel (uv_prefill_attn, through the C ABI) against the oracle's restatement
of the reference's varlen reference, and the whole packed prefill path (prefill_fast) against the oracle's
left-padded prefill: last-position logits, dequantised cache contents and int8 bytes.

Tolerances: attention 2e-2 relative in bf16 / 4e-3 in fp16 (probabilities are rounded to the activation dtype for the
P V product); the reference's own bounds for its packed prefill are dequantised cache within 0.05 and logits within
5e-2 (tests/test_perf_opt.py:153-190)."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import attn as oattn
from oracle import kv as okv
from oracle import model as om
from tests import golden_inputs as gi
from tests.helpers import build_model, golden, oracle_weights

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _run_attn(qkv, lens, H, K, hd, window, scale, dtype, xsa=None, gates=None):
    from ultraviolet_b200 import _lib
    from ultraviolet_b200.kernels._util import DTYPE_CODE, stream_ptr
    M = qkv.shape[0]
    lens = np.asarray(lens, np.int64)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    tcu = np.concatenate([[0], np.cumsum((lens + 15) // 16)]).astype(np.int32)
    t_qkv = torch.from_numpy(qkv).to(DEV, dtype)
    out = torch.full((M, H * hd), float("nan"), device=DEV, dtype=dtype)
    t_cu, t_tcu = torch.from_numpy(cu).to(DEV), torch.from_numpy(tcu).to(DEV)
    a = _lib.PrefillAttnArgs()
    a.qkv, a.dtype, a.ld = t_qkv.data_ptr(), DTYPE_CODE[dtype], t_qkv.stride(0)
    a.cu_seqlens, a.tile_cu, a.n_seq = t_cu.data_ptr(), t_tcu.data_ptr(), len(lens)
    a.max_tiles = int(tcu[-1]) + 3          # a grid larger than needed: surplus blocks exit
    a.out, a.ldo, a.H, a.K, a.hd, a.window, a.scale = out.data_ptr(), out.stride(0), H, K, hd, window, scale
    keep = [t_qkv, t_cu, t_tcu]
    if xsa is not None:
        t_x = torch.from_numpy(xsa).to(DEV)
        a.xsa_alpha, a.xsa_eps = t_x.data_ptr(), 1e-4
        keep.append(t_x)
    if gates is not None:
        t_g = torch.from_numpy(gates).to(DEV)
        a.gate_vals = t_g.data_ptr()
        keep.append(t_g)
    _lib.check(_lib.lib().uv_prefill_attn(C.byref(a), stream_ptr(torch.device(DEV))), "uv_prefill_attn")
    torch.cuda.synchronize()
    return out.float().cpu().numpy(), t_qkv.float().cpu().numpy()


@pytest.mark.parametrize("dtype,rel", [(torch.bfloat16, 2e-2), (torch.float16, 4e-3)])
@pytest.mark.parametrize("H,K,hd", [(8, 1, 64), (4, 2, 16), (4, 4, 32), (8, 2, 128)])
@pytest.mark.parametrize("window", [0, 24, 256])
def test_prefill_attention_vs_oracle(H, K, hd, window, dtype, rel):
    r = np.random.default_rng(H * 1000 + hd + window)
    lens = [1, 15, 16, 17, 0, 63, 64, 65, 130, 300, 2]     # ragged, an empty prompt, several key tiles
    M = sum(lens)
    qkv = r.standard_normal((M, (H + 2 * K) * hd)).astype(np.float32)
    out, qr = _run_attn(qkv, lens, H, K, hd, window, 0.2, dtype)
    q = qr[:, :H * hd].reshape(M, H, hd)
    k = qr[:, H * hd:(H + K) * hd].reshape(M, K, hd)
    v = qr[:, (H + K) * hd:].reshape(M, K, hd)
    cu = np.concatenate([[0], np.cumsum(lens)])
    ref = oattn.varlen_attention_ref(q, k, v, cu, 0.2, window or None).reshape(M, H * hd)
    assert np.isfinite(out).all()
    assert np.abs(out - ref).max() <= rel * np.abs(ref).max(), np.abs(out - ref).max()


def test_prefill_attention_epilogue_xsa_and_gates():
    r = np.random.default_rng(5)
    H, K, hd, lens = 8, 1, 64, [40, 7, 100]
    M = sum(lens)
    qkv = r.standard_normal((M, (H + 2 * K) * hd)).astype(np.float32)
    alpha = np.tanh(r.standard_normal(H) * 0.5).astype(np.float32)
    gates = (r.random((M, H)) * 2).astype(np.float32)
    out, qr = _run_attn(qkv, lens, H, K, hd, 32, 0.14125, torch.bfloat16, xsa=alpha, gates=gates)
    q = qr[:, :H * hd].reshape(M, H, hd)
    k = qr[:, H * hd:(H + K) * hd].reshape(M, K, hd)
    v = qr[:, (H + K) * hd:].reshape(M, K, hd)
    z = oattn.varlen_attention_ref(q, k, v, np.concatenate([[0], np.cumsum(lens)]), 0.14125, 32)
    vh = v / np.maximum(np.linalg.norm(v, axis=-1, keepdims=True), 1e-4)        # (M, 1, hd): K == 1
    z = z - alpha[None, :, None] * (z * vh).sum(-1, keepdims=True) * vh           # Attention.post, model.py:324-329
    z = z * gates[..., None]
    ref = z.reshape(M, H * hd)
    assert np.abs(out - ref).max() <= 2.5e-2 * np.abs(ref).max()


@pytest.mark.parametrize("name", ["tiny", "tiny_hd64", "uv50m"])
def test_packed_prefill_vs_oracle_prefill(name):
    """prefill_fast on ragged prompts: logits and cache against the oracle's left-padded prefill on the same bf16
    weights; the ring of local layers holds the newest positions only; subsets of rows leave the others alone."""
    spec = gi.model_specs()[name]
    m = build_model(spec).to(DEV).to(torch.bfloat16).fuse_for_inference(torch.bfloat16)
    cfg = m.cfg
    r = np.random.default_rng(17)
    n = 5
    T = 70 if name != "uv50m" else 300          # uv50m: longer than the 256-slot ring of its local layers
    lens = np.array([T, 1, T // 2, 3, T - 1])
    idx = np.zeros((n, T), np.int64)
    for i, L in enumerate(lens):
        idx[i, T - L:] = r.integers(1, cfg.vocab_size, L)
    starts = (T - lens).astype(np.int64)
    max_len = T + 4
    st = m.new_state(n, max_len)
    lg = m.prefill(torch.from_numpy(idx).to(DEV), torch.from_numpy(starts).to(DEV), st).float().cpu().numpy()
    W = oracle_weights(build_model(spec), "bf16")
    ost = om.State(cfg, n, max_len)
    ref = om.prefill(W, cfg, idx, starts, ost)
    assert np.abs(lg - ref).max() <= 5e-2 * np.abs(ref).max(), np.abs(lg - ref).max()
    assert (lg.argmax(-1) == ref.argmax(-1)).mean() >= 0.8
    assert np.array_equal(st.pos.cpu().numpy(), ost.pos) and np.array_equal(st.starts.cpu().numpy(), ost.starts)
    for l in range(cfg.n_layers):
        S = st.k[l].shape[2]
        for got_q, got_s, want_q, want_s in ((st.k[l], st.k_scale[l], ost.k[l], ost.k_scale[l]),
                                             (st.v[l], st.v_scale[l], ost.v[l], ost.v_scale[l])):
            gq, gs = got_q.cpu().numpy(), got_s.cpu().numpy()
            for i in range(n):
                t = np.arange(max(starts[i], T - S) if not cfg.is_global(l) else starts[i], T)
                sl = t % S if not cfg.is_global(l) else t
                a = okv.dequantize_kv(gq[i][:, sl], gs[i][:, sl])
                b = okv.dequantize_kv(want_q[i][:, sl], want_s[i][:, sl])
                assert np.abs(a - b).max() <= 0.05 * max(1.0, np.abs(b).max()), (l, i)
                if l == 0:   # first layer: a bf16 run against the fp32 oracle -> a step or two on a fraction of the
                    dq = np.abs(gq[i][:, sl].astype(np.int32) - want_q[i][:, sl].astype(np.int32))   # bytes (the
                    assert dq.max() <= 3 and (dq > 0).mean() < 0.35, (dq.max(), (dq > 0).mean())   # bf16 goldens
                    #                               of test_model_gpu pin the same bytes exactly)
    # a subset of rows: the other rows' cache and positions stay as they were
    st2 = m.new_state(n, max_len)
    rows = torch.tensor([3, 1], device=DEV)
    sub = [0, 2]
    lg2 = m.prefill(torch.from_numpy(idx[sub]).to(DEV), torch.from_numpy(starts[sub]).to(DEV), st2, rows=rows)
    np.testing.assert_allclose(lg2.float().cpu().numpy(), lg[sub], atol=2e-2 * np.abs(lg).max())
    assert st2.pos.cpu().tolist() == [0, T, 0, T, 0]
    dk = (st2.k[0][3].int() - st.k[0][0].int()).abs()   # same prompt in another batch: GEMM rounding at most
    assert int(dk.max()) <= 1 and not st2.k[0][0].any()
