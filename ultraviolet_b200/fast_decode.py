"""Kernel decode state and the decode / prefill entry points, API of ultraviolet/kernels/fast_decode.py.

``KernelDecodeState`` keeps the reference's fields and cache layout (fast_decode.py:21-57): per layer ``k[l], v[l]``
int8 ``(B, K, S, hd)`` with S = max_len (global layers) or min(window, max_len) (local ring), ``k_scale[l],
v_scale[l]`` fp16 ``(B, K, S)``, ``pos`` / ``starts`` int64 ``(B,)``, ``host_pos``.

``decode_step_fast`` is one call of ``DecodeEngine.trunk`` (+ head).  ``prefill_fast`` packs the prompts of a batch
back to back and runs them through the same GEMMs and row kernels as ONE batch of sum(len) rows, with a packed
varlen attention kernel (uv_prefill_attn) over the unquantised keys / values and the int8 cache written by the same
fused quantise + append as in decode; positions, ring slots, ``st.pos`` / ``st.starts`` and the cache layout are those
of the reference's left-padded prefill.
"""
from __future__ import annotations

import types

import numpy as np
import torch
from torch import Tensor

from .config import MathConfig, config_from


class KernelDecodeState:
    def __init__(self, cfg: MathConfig, B: int, max_len: int, dtype, device, kv_dtype: str = "int8",
                 ring_extra: int = 0):
        """ring_extra > 0 (not in the reference): local-layer rings get window + ring_extra slots (rounded up to a
        multiple of 8) instead of window.  A step that writes up to ring_extra + 1 consecutive positions of one
        sequence (prefill lanes) then never overwrites a key that another row of the same step still attends to,
        for prompts of any length."""
        cfg = config_from(cfg)
        if kv_dtype != "int8":
            raise NotImplementedError("ultraviolet_b200 keeps the KV cache in int8 (kv_dtype='int8')")
        self.cfg, self.B, self.max_len, self.dtype = cfg, B, max_len, dtype
        self.kv_dtype = kv_dtype
        self.local_len = min(cfg.window, max_len)
        if ring_extra > 0:
            self.local_len = min((cfg.window + int(ring_extra) + 7) // 8 * 8, max(max_len, cfg.window))
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


PREFILL_CHUNK_TOKENS = 32768   # packed rows per pass (activations of one pass: ~19 KB per row)


@torch.no_grad()
def prefill_fast(self, idx: Tensor, starts: Tensor, st: KernelDecodeState, rows: Tensor | None = None) -> Tensor:
    """idx (n, T) left-padded; writes the cache rows `rows` (default all) from position starts[i] on, sets their
    pos = T / starts, returns the last-position logits (n, V) (contract of fast_decode.py:70-114).

    The prompts are packed back to back (pad columns are never computed) and go through the step's kernels as one
    batch of sum(len) rows per pass, with attention by the packed varlen kernel over the unquantised keys / values
    (the packed route of the reference, fast_decode.py:117-163, :210-269); positions are those of the left-padded
    frame (token j of row i sits at starts[i] + j), so ring slots and the int8 cache layout are the reference's."""
    eng = _engine(self)
    n, T = idx.shape
    if T > st.max_len:
        raise AssertionError("prompt longer than the cache")
    dev = idx.device
    full = rows is None
    if full:
        if n != st.B:
            raise AssertionError("prefill without rows needs one prompt per cache row")
        rows = torch.arange(n, device=dev)
    rows = rows.to(torch.int64)
    starts = starts.to(torch.int64).contiguous()
    lens_h = (T - starts).clamp_(min=0).cpu().numpy()   # the one host round trip (the reference has one too, :111)
    hfin = torch.zeros(n, eng.cfg.d_model, dtype=eng.dtype, device=dev)
    # passes over whole prompts, at most PREFILL_CHUNK_TOKENS packed rows each (one prompt alone may exceed it)
    a = 0
    while a < n:
        b, tot = a, 0
        while b < n and (b == a or tot + int(lens_h[b]) <= PREFILL_CHUNK_TOKENS):
            tot += int(lens_h[b])
            b += 1
        if tot > 0:
            hfin[a:b] = prefill_packed(eng, st, idx[a:b], starts[a:b], rows[a:b], lens_h[a:b])
        a = b
    st.starts[rows] = starts
    st.pos[rows] = T
    st.host_pos[rows.cpu().numpy()] = T
    return eng.logits(hfin)


def pack_prompts(idx: Tensor, starts: Tensor, rows: Tensor, lens_h) -> dict:
    """Packed description of a left-padded (n, T) prompt batch: per packed row its token, position and cache row,
    plus the prefix sums the varlen attention kernel walks.  lens_h: host array of prompt lengths (T - starts)."""
    n, T = idx.shape
    dev = idx.device
    t = torch.arange(T, device=dev)
    keep = t[None, :] >= starts[:, None]                      # row-major selection = prompt after prompt
    tok = idx[keep].contiguous()
    pos = t.expand(n, T)[keep].contiguous()
    cache_row = rows[:, None].expand(n, T)[keep].contiguous()
    lens = np.asarray(lens_h, dtype=np.int64)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    tile_cu = np.concatenate([[0], np.cumsum((lens + 15) // 16)]).astype(np.int32)
    M = int(cu[-1])
    return dict(tok=tok, pos=pos, rows=cache_row, M=M, n_seq=n, max_tiles=int(tile_cu[-1]),
                cu=torch.from_numpy(cu).to(dev), tile_cu=torch.from_numpy(tile_cu).to(dev),
                last_pos=torch.full((M,), T - 1, dtype=torch.int64, device=dev),
                last_row=torch.from_numpy(np.maximum(cu[1:].astype(np.int64) - 1, 0)).to(dev),
                empty=torch.from_numpy(lens == 0).to(dev))


def prefill_packed(eng, st, idx: Tensor, starts: Tensor, rows: Tensor, lens_h) -> Tensor:
    """One packed pass: returns the final normed hidden state of every prompt's last token (n, d) (zeros for an
    empty prompt)."""
    pk = pack_prompts(idx, starts, rows, lens_h)
    zero = torch.zeros(pk["M"], dtype=torch.int64, device=idx.device)
    h = eng.trunk(pk["tok"], st, pk["pos"], zero, g_len=idx.size(1), row_map=pk["rows"], packed=pk)
    out = h[pk["last_row"]]
    return out.masked_fill(pk["empty"][:, None], 0)


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

    def new_state(self, batch, max_len, dtype=None, device=None, ring_extra=0):
        return KernelDecodeState(eng.cfg, batch, max_len, dtype or eng.dtype, device or eng.device, kv_dtype,
                                 ring_extra=ring_extra)

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
