"""Host-side logic that needs no GPU: configuration, parameter container, state layout, loud failures."""
import numpy as np
import pytest
import torch

from tests import golden_inputs as gi
from tests.helpers import build_model, golden


def test_preset_geometry():
    from ultraviolet_b200.config import make_config
    c = make_config("uv-50m-alpha", vocab_size=16384)
    assert (c.d_model, c.n_layers, c.n_heads, c.n_kv_heads, c.head_dim, c.d_ff, c.window) == (640, 10, 8, 1, 64,
                                                                                             1664, 256)
    assert [l for l in range(10) if c.is_global(l)] == [4, 9]
    assert [l for l in range(10) if c.has_ve(l)] == [1, 4, 7]
    assert c.rope_pairs == 16 and abs(c.attn_scale - 0.14125) < 1e-9 and c.gate_channels == 128
    p = c.param_counts()
    assert p["non_embedding"] == 39_321_600 and p["embedding_tied"] == 10_485_760 and p["value_embedding"] == 1_048_576
    c.check_decode_supported()
    with pytest.raises(NotImplementedError):
        make_config("uv-50m-alpha", mudd=True).check_decode_supported()


@pytest.mark.parametrize("name", sorted(gi.model_specs()))
def test_parameter_container_matches_reference_init(name):
    """Same names, shapes, creation order and RNG consumption as the reference's MathLM: the digest stored by
    make_golden.py is the reference's own state dict."""
    spec = gi.model_specs()[name]
    m = build_model(spec)
    assert gi.state_sha(m.state_dict()) == str(golden("model")[name + ".weights_sha"])
    if name == "uv50m":
        assert sum(p.numel() for p in m.parameters()) == 50_866_352


def test_state_layout_and_bytes():
    from ultraviolet_b200.config import make_config
    from ultraviolet_b200.fast_decode import KernelDecodeState, kv_bytes_per_seq
    c = make_config("uv-50m-alpha", vocab_size=16384)
    st = KernelDecodeState(c, 4, 1000, torch.bfloat16, "cpu")
    assert st.k[0].shape == (4, 1, 256, 64) and st.k[4].shape == (4, 1, 1000, 64) and st.k[0].dtype == torch.int8
    assert st.k_scale[4].shape == (4, 1, 1000) and st.k_scale[4].dtype == torch.float16
    assert st.nbytes() == 4 * kv_bytes_per_seq(c, 1000)
    assert kv_bytes_per_seq(c, 4096) == 132 * (2 * 4096 + 8 * 256)   # 132 B per token per layer
    with pytest.raises(NotImplementedError):
        KernelDecodeState(c, 1, 8, torch.bfloat16, "cpu", kv_dtype="fp16")


def test_no_cpu_fallback():
    from ultraviolet_b200.kernels import decode_attention, quantize_kv
    spec = gi.model_specs()["tiny"]
    m = build_model(spec)
    with pytest.raises(RuntimeError):
        m.fuse_for_inference(torch.bfloat16)          # CPU model: the engine refuses
    with pytest.raises(RuntimeError):
        quantize_kv(torch.zeros(2, 64))
    with pytest.raises(RuntimeError):
        m.decode_step(torch.zeros(1, dtype=torch.long), None, 8)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from ultraviolet_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "libuvdecode.so"))
    with pytest.raises(_lib.UvError):
        _lib.lib()


def test_device_handoff_layout_matches_reference_micro_batches():
    """handoff.build_packed_device lays finished rollouts out exactly as the reference's host-side build_packed does
    (golden: tests/golden/packing.npz, produced by ultraviolet/perf.py:55-95 itself).  Pure index arithmetic on
    tensors, so the layout logic is checked here on CPU tensors; the GPU tests feed it real harvests."""
    import numpy as np
    import torch
    from tests.helpers import golden
    from ultraviolet_b200.handoff import build_packed_device, pack_bins
    g = golden("packing")
    items, budget, pad_id, seg_max = gi.packing_case()
    p = dict(tokens=torch.from_numpy(np.concatenate([t[s:] for t, s, _, _ in items]).astype(np.int32)),
             logp=torch.from_numpy(np.concatenate([b for *_, b in items])),
             offsets=torch.from_numpy(np.concatenate([[0], np.cumsum([len(t) - s for t, s, _, _ in items])])),
             prompt_tokens=torch.from_numpy(np.concatenate([t[:s] for t, s, _, _ in items]).astype(np.int32)),
             prompt_offsets=torch.from_numpy(np.concatenate([[0], np.cumsum([s for _, s, _, _ in items])])),
             metas=list(range(len(items))))
    mbs = build_packed_device(p, [a for _, _, a, _ in items], budget, pad_id, seg_max)
    assert len(mbs) == int(g["n"])
    for i, mb in enumerate(mbs):
        for k in ("x", "y", "pos", "cu", "tgt"):
            assert np.array_equal(mb[k].numpy(), g[f"mb{i}.{k}"]), (i, k)
        for k in ("A", "OL"):
            np.testing.assert_allclose(mb[k].numpy(), g[f"mb{i}.{k}"], rtol=0, atol=0)
        assert mb["max_seqlen"] == int(g[f"mb{i}.max_seqlen"])
    bins = pack_bins([5, 900, 200, 100, 1024], 1024)
    assert sorted(sum(bins, [])) == [0, 1, 2, 3, 4] and all(sum([5, 900, 200, 100, 1024][i] for i in b) <= 1024
                                                           for b in bins)


def test_admission_pass_capacities():
    """Capacities an admission pass is captured at: ascending multiples of 64 from 256 to the limit, never more than
    a quarter above the one before, powers of two included."""
    from ultraviolet_b200.scheduler import _pass_caps
    for limit in (256, 1024, 16384):
        caps = _pass_caps(limit)
        assert caps[0] == 256 and caps[-1] == limit and caps == sorted(set(caps))
        assert all(c % 64 == 0 for c in caps)
        assert all(b <= a * 1.25 + 1e-9 for a, b in zip(caps, caps[1:]))
        p = 256
        while p <= limit:
            assert p in caps
            p *= 2


def test_bench_workload_definitions_are_deterministic_and_match_their_configurations():
    """bench.py's synthetic workloads: the same requests every time (both benchmark arms and every rank build them
    independently), with the shapes the configurations name; the algorithmic-bytes formula of an attention launch."""
    import importlib.util
    import os
    spec = importlib.util.spec_from_file_location(
        "uv_bench", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    p3, stops, max_prompt, max_new = bench.config3_requests()
    q3, stops2, _, _ = bench.config3_requests()
    assert p3 == q3 and (stops == stops2).all()
    assert len(p3) == 4096 and (max_prompt, max_new) == (256, 2048)
    lens = np.array([len(p) for p in p3])
    assert lens.min() >= 16 and lens.max() <= 256 and stops.min() >= 1 and stops.max() == 2048
    assert 500 < stops.mean() < 620                       # Geometric(mean 600) capped at 2048
    assert all(0 < t < bench.VOCAB for p in p3[:50] for t in p)          # EOS (0) never inside a prompt
    p5, mp5, mn5 = bench.config5_requests()
    assert len(p5) == 2048 and (mp5, mn5) == (256, 2048)
    assert all(p5[8 * g + c] == p5[8 * g] for g in range(256) for c in range(8))   # groups of 8 identical prompts
    assert len({tuple(p5[8 * g]) for g in range(256)}) == 256
    assert min(len(p) for p in p5) >= 64 and max(len(p) for p in p5) <= 256
    a = bench.make_prompts(256, 32, 128, 100)
    assert a == bench.make_prompts(256, 32, 128, 100) and 32 <= min(map(len, a)) and max(map(len, a)) <= 128
    # 132 bytes per attended key (64 + 64 int8 + two fp16 scales) + q and out of 8 heads x 64 x 2 bytes per row
    pos, starts = np.array([9, 300, 5]), np.array([0, 0, 3])
    assert bench.attn_bytes(pos, starts, 0) == (10 + 301 + 3) * 132 + 2 * 3 * 8 * 64 * 2
    assert bench.attn_bytes(pos, starts, 256, S=256, ring=True) == (10 + 256 + 3) * 132 + 2 * 3 * 8 * 64 * 2
    cfg = bench.workload_config(20)
    assert cfg == bench.workload_config(20) and "workload" in cfg
