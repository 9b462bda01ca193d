"""GEMMs with fused epilogues (uv_gemm_qkv / uv_gemm_swiglu / uv_gemm_resid_norm) against the same step computed
with library GEMMs + the separate row kernels, and against the oracle."""
import numpy as np
import pytest
import torch

from oracle import model as om
from tests import golden_inputs as gi
from tests.helpers import build_model, oracle_weights

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _run(eng, m, fused, B, steps, seed):
    eng.fused_gemm = fused
    st = m.new_state(B, 64)
    g = torch.Generator(device=DEV).manual_seed(seed)
    hs = []
    for _ in range(steps):
        tok = torch.randint(1, m.cfg.vocab_size, (B,), device=DEV, generator=g)
        hs.append(m.decode_step(tok, st, 64, ).clone())
    return torch.stack(hs), st


@pytest.mark.parametrize("B", [7, 256, 300])
def test_fused_gemm_step_matches_unfused_step(B):
    spec = gi.model_specs()["uv50m"]
    m = build_model(spec).to(DEV).to(torch.bfloat16).fuse_for_inference(torch.bfloat16)
    eng = m.engine
    assert eng.fused_gemm_ok
    eng.fold = False          # both sides on the reference's literal op order (the arena then holds unfolded weights)
    eng.load_from(m)
    a, sa = _run(eng, m, True, B, 6, 1)
    b, sb = _run(eng, m, False, B, 6, 1)
    eng.fused_gemm = True
    a, b = a.float().cpu().numpy(), b.float().cpu().numpy()
    assert np.isfinite(a).all()
    err = np.abs(a - b)
    assert err.max() <= 1e-2 * np.abs(b).max() and err.mean() < 2e-3, (err.max(), err.mean())
    assert (a.argmax(-1) == b.argmax(-1)).mean() > 0.97
    for l in (0, 4, 9):
        ka, kb = sa.k[l].cpu().numpy().astype(np.int16), sb.k[l].cpu().numpy().astype(np.int16)
        d = np.abs(ka - kb)
        lim = 0.01 if l == 0 else 0.2      # the first layer's keys depend on one GEMM only
        assert d.max() <= (2 if l == 0 else 8) and (d != 0).mean() < lim, (l, d.max(), (d != 0).mean())


def test_fused_gemm_step_matches_oracle():
    spec = gi.model_specs()["uv50m"]
    mc = build_model(spec)
    W = oracle_weights(mc, "bf16")
    m = build_model(spec).to(DEV).to(torch.bfloat16).fuse_for_inference(torch.bfloat16)
    assert m.engine.fused_gemm_ok
    m.engine.fold = False     # the fused-epilogue kernels apply the residual lambdas themselves: unfolded weights
    m.engine.load_from(m)
    m.engine.fused_gemm = True
    B, steps = 5, 4
    r = np.random.default_rng(2)
    toks = r.integers(1, mc.cfg.vocab_size, (steps, B))
    st, ost = m.new_state(B, 16), om.State(mc.cfg, B, 16)
    for i in range(steps):
        lg = m.decode_step(torch.from_numpy(toks[i]).to(DEV), st, 16).float().cpu().numpy()
        olg = om.decode_step(W, mc.cfg, toks[i], ost)
        err = np.abs(lg - olg)
        assert err.max() <= 2e-2 * np.abs(olg).max(), (i, err.max())
