"""Kernel decode state and the decode / prefill entry points, API of ultraviolet/kernels/fast_decode.py.

``KernelDecodeState`` keeps the reference's fields and cache layout (fast_decode.py:21-57): per layer ``k[l], v[l]``
int8 ``(B, K, S, hd)`` with S = max_len (global layers) or min(window, max_len) (local ring), ``k_scale[l],
v_scale[l]`` fp16 ``(B, K, S)``, ``pos`` / ``starts`` int64 ``(B,)``, ``host_pos``.

``decode_step_fast`` is one call of ``DecodeEngine.trunk`` (+ head).  ``prefill_fast`` feeds the left-padded prompt
through the SAME decode kernels one position at a time ("prefill as decode"): row i starts consuming at position
starts[i], so positions, ring slots, ``st.pos`` / ``st.starts`` and the int8 cache layout are those of the reference's
padded prefill; prompt tokens attend to the int8-quantised keys of their prefix instead of the unquantised ones the
reference's SDPA prefill sees (same model, int8 rounding noise only).  A packed varlen prefill kernel is the next
step of this path and is not built yet.
"""
from __future__ import annotations

import types

import numpy as np
import torch
from torch import Tensor

from .config import MathConfig, config_from


class KernelDecodeState:
    def __init__(self, cfg: MathConfig, B: int, max_len: int, dtype, device, kv_dtype: str = "int8"):
        cfg = config_from(cfg)
        if kv_dtype != "int8":
            raise NotImplementedError("ultraviolet_b200 keeps the KV cache in int8 (kv_dtype='int8')")
        self.cfg, self.B, self.max_len, self.dtype = cfg, B, max_len, dtype
        self.kv_dtype = kv_dtype
        self.local_len = min(cfg.window, max_len)
        self.k, self.v, self.k_scale, self.v_scale = [], [], [], []
        self.mix: dict[int, dict] = {}
        for l in range(cfg.n_layers):
            S = max_len if cfg.is_global(l) else self.local_len
            # linear (global) rows are allocated to a multiple of 8 slots so the attention kernel's bulk copies can
            # fetch whole 16-byte groups of scales; the tensors exposed are the reference's (B, K, S, hd) / (B, K, S)
            Sa = S if not cfg.is_global(l) else (S + 7) // 8 * 8
            shp = (B, cfg.n_kv_heads, Sa, cfg.head_dim)
            self.k.append(torch.zeros(shp, dtype=torch.int8, device=device)[:, :, :S])
            self.v.append(torch.zeros(shp, dtype=torch.int8, device=device)[:, :, :S])
            self.k_scale.append(torch.zeros(shp[:3], dtype=torch.float16, device=device)[:, :, :S])
            self.v_scale.append(torch.zeros(shp[:3], dtype=torch.float16, device=device)[:, :, :S])
        self.pos = torch.zeros(B, dtype=torch.long, device=device)
        self.starts = torch.zeros(B, dtype=torch.long, device=device)
        self.host_pos = np.zeros(B, dtype=np.int64)
        self.prev = None

    def set_pos(self, p: int):
        self.pos.fill_(p)
        self.host_pos[:] = p

    def nbytes(self) -> int:
        ts = self.k + self.v + self.k_scale + self.v_scale
        return sum(t.numel() * t.element_size() for t in ts)


def kv_bytes_per_seq(cfg: MathConfig, ctx: int, kv_dtype: str = "int8") -> int:
    """fast_decode.py:64-67."""
    per_pos = 2 * cfg.n_kv_heads * (cfg.head_dim * 2 if kv_dtype == "fp16" else cfg.head_dim + 2)
    return sum(per_pos * (ctx if cfg.is_global(l) else min(ctx, cfg.window)) for l in range(cfg.n_layers))


def _engine(model):
    eng = getattr(model, "_uvb200_engine", None) or getattr(model, "_engine", None)
    if eng is None:
        raise RuntimeError("no decode engine on this model: call patch_model(model) / fuse_for_inference(dtype) first")
    return eng


@torch.no_grad()
def decode_step_fast(self, tok: Tensor, st: KernelDecodeState, g_len: int, skip_attn: bool = False,
                     num_splits: dict | None = None, backend: str = "auto", return_hidden: bool = False) -> Tensor:
    """One token for every cache row at its own position st.pos (fast_decode.py:272-334); advances st.pos.  Returns
    (B, V) fp32 softcapped logits, or the final normed hidden (B, d) when return_hidden."""
    eng = _engine(self)
    h = eng.trunk(tok, st, st.pos, st.starts, g_len=g_len, num_splits=num_splits, skip_attn=skip_attn)
    st.pos.add_(1)
    return h if return_hidden else eng.logits(h)


@torch.no_grad()
def prefill_fast(self, idx: Tensor, starts: Tensor, st: KernelDecodeState, rows: Tensor | None = None) -> Tensor:
    """idx (n, T) left-padded; writes the cache rows `rows` (default all) from position starts[i] on, sets their
    pos = T / starts, returns the last-position logits (n, V) (contract of fast_decode.py:70-114)."""
    eng = _engine(self)
    n, T = idx.shape
    if T > st.max_len:
        raise AssertionError("prompt longer than the cache")
    full = rows is None
    if full:
        if n != st.B:
            raise AssertionError("prefill without rows needs one prompt per cache row")
        rows = torch.arange(n, device=idx.device)
    rows = rows.to(torch.int64)
    starts = starts.to(torch.int64).contiguous()
    idx_t = idx.t().contiguous()  # (T, n): one contiguous token vector per position
    h = _prefill_positions(eng, st, idx_t, starts, None if full else rows, T)
    st.starts[rows] = starts
    st.pos[rows] = T
    st.host_pos[rows.cpu().numpy()] = T
    return eng.logits(h)


def _prefill_positions(eng, st, idx_t: Tensor, starts: Tensor, rows, T: int) -> Tensor:
    """Feed positions 0..T-1 of a left-padded sub-batch through the decode kernels.  The step for one position is
    captured once as a CUDA graph reading a static token / position pair and replayed T times (positions differ
    only through those two device tensors); short prompts run eagerly."""
    n = idx_t.size(1)
    dev = idx_t.device
    pos = torch.zeros(n, dtype=torch.int64, device=dev)
    if T < 8:
        h = None
        for t in range(T):
            pos.fill_(t)
            h = eng.trunk(idx_t[t], st, pos, starts, g_len=T, row_map=rows)
        return h
    tok = torch.zeros(n, dtype=torch.int64, device=dev)
    out = {}

    def body():
        out["h"] = eng.trunk(tok, st, pos, starts, g_len=T, row_map=rows)
        pos.add_(1)

    tok.copy_(idx_t[0])
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):   # warm-up run of position 0 (allocates scratch); it is simply redone below
        body()
        pos.zero_()
    torch.cuda.current_stream(dev).wait_stream(side)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, capture_error_mode="thread_local"):
        body()
    for t in range(T):
        tok.copy_(idx_t[t])
        g.replay()
    return out["h"].clone()  # the graph's private pool goes away with the graph


def patch_model(model, kv_dtype: str = "int8", num_splits: dict | None = None, backend: str = "auto",
                dtype: torch.dtype | None = None):
    """Bind the B200 decode path onto a MathLM instance (the reference's or ours), as fast_decode.patch_model does
    (fast_decode.py:341-358): instance attributes new_state / prefill / decode_step / logits.  The fused weights are
    copied into a DecodeEngine arena; call ``refresh_weights(model)`` (or sync_weights_inplace) after a parameter
    update."""
    from .engine import DecodeEngine
    if kv_dtype != "int8":
        raise NotImplementedError("only the int8 KV cache is built")
    p0 = model.embed.weight
    dt = dtype or (p0.dtype if p0.dtype in (torch.float16, torch.bfloat16) else torch.bfloat16)
    eng = DecodeEngine.from_model(model, dt)
    model.__dict__["_uvb200_engine"] = eng

    def new_state(self, batch, max_len, dtype=None, device=None):
        return KernelDecodeState(eng.cfg, batch, max_len, dtype or eng.dtype, device or eng.device, kv_dtype)

    def decode_step(self, tok, st, g_len, skip_attn=False):
        return decode_step_fast(self, tok, st, g_len, skip_attn, num_splits, backend)

    def logits(self, h):
        return eng.logits(h)

    model.new_state = types.MethodType(new_state, model)
    model.prefill = types.MethodType(prefill_fast, model)
    model.decode_step = types.MethodType(decode_step, model)
    model.logits = types.MethodType(logits, model)
    return model


def unpatch_model(model):
    for n in ("new_state", "prefill", "decode_step", "logits", "_uvb200_engine"):
        model.__dict__.pop(n, None)
    return model


def refresh_weights(model) -> None:
    """In-place weight refresh of a patched model's engine (pointer-stable; captured graphs stay valid)."""
    _engine(model).load_from(model)
