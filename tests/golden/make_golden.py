"""Generate the golden fixtures in this directory from the reference implementation itself.

Run where the reference checkout is available, with ``REFERENCE_ROOT`` pointing at it:

    REFERENCE_ROOT=/path/to/ultraviolet python tests/golden/make_golden.py

It imports the reference's own CPU-runnable code for the rollout-decode path (ultraviolet.kernels.quantize_kv,
kv_write, decode_attention_ref, fused_sample_ref; fast_decode.decode_step_fast / prefill_fast with the attention
call rebound to decode_attention_ref; model.generate / generate_continuous / sample) and stores its outputs on
seeded inputs.  Inputs are NOT stored: ``tests/golden_inputs.py`` rebuilds them from the same seeds, and the
fixtures carry SHA-256 digests of the inputs so a drift in input generation is detected rather than silently
compared.  The tests never import the reference.
"""
from __future__ import annotations

import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
if "REFERENCE_ROOT" not in os.environ:
    sys.exit("set REFERENCE_ROOT to the reference checkout (hliuson/ultraviolet)")
sys.path.insert(0, os.environ["REFERENCE_ROOT"])

from tests import golden_inputs as gi  # noqa: E402
import ultraviolet.kernels.fast_decode as ref_fd  # noqa: E402
from ultraviolet.kernels import decode_attention_ref, kv_write, quantize_kv  # noqa: E402
from ultraviolet.kernels.fused_sample import fused_sample_ref  # noqa: E402
from ultraviolet.model import MathLM, generate, generate_continuous, make_config, sample  # noqa: E402


def _ref_attn(q, k, v, pos, starts, scale, *, window=0, ring=None, k_scale=None, v_scale=None, **_):
    return decode_attention_ref(q, k, v, pos, starts, scale, window=window, ring=ring, k_scale=k_scale,
                                v_scale=v_scale)


ref_fd.decode_attention = _ref_attn  # the reference's CPU route for the kernel path: same step, fp32 torch attention
T = torch.from_numpy


def save(name, **arrs):
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **arrs)
    print(f"{name}.npz  {os.path.getsize(path) / 1024:.1f} KiB  {sorted(arrs)}")


# ------------------------------------------------------------------------------------------------ quantiser
def make_quant():
    out = {}
    for name, x in gi.quant_cases().items():
        q, s = quantize_kv(T(x))
        out[name + ".q"] = q.numpy()
        out[name + ".s"] = s.numpy().view(np.uint16)
        out[name + ".in_sha"] = np.array(gi.sha(x))
    # kv_write scatter (kv_quant.py:26-36) into a small cache
    x, idx = gi.kv_write_case()
    cache = torch.zeros(4, 2, 16, 64, dtype=torch.int8)
    sc = torch.zeros(4, 2, 16, dtype=torch.float16)
    kv_write(cache, sc, T(idx), T(x))
    out["kv_write.cache"] = cache.numpy()
    out["kv_write.scale"] = sc.numpy().view(np.uint16)
    save("quant", **out)


# ------------------------------------------------------------------------------------------------ attention
def make_attn():
    out = {}
    c1 = gi.config1()
    out["config1.lens"] = c1["lens"]
    kq, ks = quantize_kv(T(c1["k"]))
    vq, vs = quantize_kv(T(c1["v"]))
    for n, a in (("kq", kq), ("ks", ks), ("vq", vq), ("vs", vs)):
        out[f"config1.{n}_sha"] = np.array(gi.sha(a.numpy()))
    pos, starts = T(c1["lens"] - 1), torch.zeros(16, dtype=torch.long)
    out["config1.global"] = decode_attention_ref(T(c1["q"]), kq, vq, pos, starts, 0.14125, k_scale=ks,
                                                 v_scale=vs).numpy()
    out["config1.local"] = decode_attention_ref(T(c1["q"]), kq[:, :, :256].contiguous(),
                                                vq[:, :, :256].contiguous(), pos, starts, 0.14125, window=256,
                                                ring=True, k_scale=ks[:, :, :256].contiguous(),
                                                v_scale=vs[:, :, :256].contiguous()).numpy()
    for name, c in gi.attn_cases().items():
        q, k, v = T(c["q"]), T(c["k"]), T(c["v"])
        if c["int8"]:
            kq, ks = quantize_kv(k)
            vq, vs = quantize_kv(v)
        else:
            kq, ks, vq, vs = k, None, v, None
        ref = decode_attention_ref(q, kq, vq, T(c["pos"]), T(c["starts"]), c["scale"], window=c["window"],
                                   ring=c["ring"], k_scale=ks, v_scale=vs)
        out[name] = ref.numpy()
        out[name + ".in_sha"] = np.array(gi.sha(c["q"], c["k"], c["v"], c["pos"], c["starts"]))
    # packed varlen attention of the prefill (varlen_attn.py:94-114)
    from ultraviolet.kernels.varlen_attn import varlen_attention_ref
    c = gi.varlen_case()
    for name, window in (("varlen.window", c["window"]), ("varlen.full", None)):
        out[name] = varlen_attention_ref(T(c["q"])[None], T(c["k"])[None], T(c["v"])[None], T(c["cu"]), c["scale"],
                                         window)[0].numpy()
    out["varlen.in_sha"] = np.array(gi.sha(c["q"], c["k"], c["v"], c["cu"]))
    save("attn", **out)


# ------------------------------------------------------------------------------------------------ model
def _ref_model(spec):
    torch.manual_seed(spec["seed"])
    m = MathLM(make_config(spec["preset"], **spec["over"]))
    gi.perturb_(m, spec)
    m.decode_impl = "kernel-int8"
    return m.float().fuse_for_inference(torch.float32)


def _teacher_forced(m, idx, starts, cont, max_len):
    st = m.new_state(idx.size(0), max_len, torch.float32, "cpu")
    outs = [m.prefill(idx, starts, st)]
    for t in range(cont.size(1)):
        outs.append(m.decode_step(cont[:, t], st, max_len))
    return torch.stack(outs, 1).float(), st


def make_model():
    out = {}
    for name, spec in gi.model_specs().items():
        m = _ref_model(spec)
        out[name + ".weights_sha"] = np.array(gi.state_sha(m.state_dict()))
        idx, starts, cont, max_len = gi.teacher_inputs(spec)
        lg, st = _teacher_forced(m, T(idx), T(starts), T(cont), max_len)
        lg = lg.numpy()
        cols = gi.logit_columns(spec, lg.shape[-1])
        out[name + ".logits"] = lg[..., cols]
        out[name + ".argmax"] = lg.argmax(-1)
        out[name + ".max"] = lg.max(-1)
        for l in spec["cache_layers"]:
            out[f"{name}.k{l}"] = st.k[l].numpy()
            out[f"{name}.ks{l}"] = st.k_scale[l].numpy().view(np.uint16)
            out[f"{name}.v{l}"] = st.v[l].numpy()
            out[f"{name}.vs{l}"] = st.v_scale[l].numpy().view(np.uint16)
        out[name + ".pos"] = st.pos.numpy()
        if spec.get("generate"):
            g = spec["generate"]
            res = generate(m, g["prompts"], g["max_new"], temperature=0.0, use_graph=False, compile=False,
                           eos_id=g["eos_id"], dtype=torch.float32)
            out[name + ".generate"] = gi.pack_lists(res)
            c = spec["continuous"]
            res = generate_continuous(m, c["prompts"], c["max_new"], batch=c["batch"], temperature=0.0,
                                      eos_id=c["eos_id"], check_every=c["check_every"], use_graph=False,
                                      compile=False, dtype=torch.float32, target_lens=c["target_lens"])
            out[name + ".continuous"] = gi.pack_lists(res)
    save("model", **out)


def make_model_bf16():
    """The same teacher-forced run with the reference itself in bfloat16 on the CPU (weights, activations and the
    int8 cache path as a bf16 deployment computes them): the GPU path is compared against these bytes much more
    tightly than against the fp32 run, because both sides round where bf16 rounds."""
    out = {}
    for name in ("uv50m", "tiny_hd64"):
        spec = gi.model_specs()[name]
        torch.manual_seed(spec["seed"])
        m = MathLM(make_config(spec["preset"], **spec["over"]))
        gi.perturb_(m, spec)
        m.decode_impl = "kernel-int8"
        m = m.bfloat16().fuse_for_inference(torch.bfloat16)
        idx, starts, cont, max_len = gi.teacher_inputs(spec)
        st = m.new_state(idx.shape[0], max_len, torch.bfloat16, "cpu")
        outs = [m.prefill(T(idx), T(starts), st)]
        for t in range(cont.shape[1]):
            outs.append(m.decode_step(T(cont)[:, t], st, max_len))
        lg = torch.stack(outs, 1).float().numpy()
        cols = gi.logit_columns(spec, lg.shape[-1])
        out[name + ".logits"] = lg[..., cols]
        out[name + ".argmax"] = lg.argmax(-1)
        for l in spec["cache_layers"]:
            out[f"{name}.k{l}"] = st.k[l].numpy()
            out[f"{name}.ks{l}"] = st.k_scale[l].numpy().view(np.uint16)
            out[f"{name}.v{l}"] = st.v[l].numpy()
            out[f"{name}.vs{l}"] = st.v_scale[l].numpy().view(np.uint16)
        out[name + ".pos"] = st.pos.numpy()
    save("model_bf16", **out)


# ------------------------------------------------------------------------------------------------ samplers
def make_sampler():
    out = {}
    x, u, cap, temps = gi.fused_sample_case()
    for t in temps:
        tok, lp = fused_sample_ref(T(x), T(u), cap, t)
        out[f"fused.tok.T{t}"] = tok.numpy()
        out[f"fused.lp.T{t}"] = lp.numpy()
    out["fused.in_sha"] = np.array(gi.sha(x, u))
    # nucleus support: empirical support of the reference's sample(top_p) over many draws
    lg, temp, top_p, draws = gi.top_p_case()
    torch.manual_seed(1234)
    rows = T(lg)
    seen = np.zeros(lg.shape, dtype=bool)
    for _ in range(draws):
        tok = sample(rows, temp, 0, top_p).numpy()
        seen[np.arange(lg.shape[0]), tok] = True
    out["top_p.support"] = seen
    save("sampler", **out)


def make_packing():
    """The trainer-side micro-batch layout (ultraviolet/perf.py:55-95) on seeded rollouts."""
    from ultraviolet.perf import build_packed
    items, budget, pad_id, seg_max = gi.packing_case()
    out = {"n": np.array(0)}
    mbs = build_packed(items, budget, pad_id, seg_max=seg_max)
    out["n"] = np.array(len(mbs))
    for i, mb in enumerate(mbs):
        for k in ("x", "y", "A", "OL", "pos", "cu", "tgt"):
            out[f"mb{i}.{k}"] = np.asarray(mb[k])
        out[f"mb{i}.max_seqlen"] = np.array(mb["max_seqlen"])
    save("packing", **out)


if __name__ == "__main__":
    torch.set_grad_enabled(False)
    make_quant()
    make_attn()
    make_model()
    make_model_bf16()
    make_sampler()
    make_packing()
