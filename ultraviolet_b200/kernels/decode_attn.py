"""Split-K decode attention (API of ultraviolet/kernels/decode_attn.py:193-230) on the sm_100a kernel."""
from __future__ import annotations

import ctypes as C

import torch
from torch import Tensor

from .. import _lib
from ._util import DTYPE_CODE, need_cuda, ptr, stream_ptr

_N_SM: dict = {}


def _n_sm(dev: torch.device) -> int:
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    if idx not in _N_SM:
        _N_SM[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _N_SM[idx]


def default_splits(n_bk: int, ctx: int, device=None, min_chunk: int | None = None, waves: int | None = None) -> int:
    """Splits per (row, kv head) (role of decode_attn.py:121-129).  Without min_chunk / waves the heuristic is the
    library's own (uv_default_splits: 128-key tiles, every CTA resident in one wave, a split only when it takes at
    least four tiles off every CTA).  A caller that passes either one gets the reference's rule with those values
    (about `waves` programs per SM, chunks of at least min_chunk keys, at most 64 splits; defaults 8 and 128)."""
    dev = torch.device(device or "cuda")
    if min_chunk is None and waves is None:
        return int(_lib.lib().uv_default_splits(int(n_bk), int(ctx), _n_sm(dev)))
    waves, min_chunk = 8 if waves is None else int(waves), 128 if min_chunk is None else int(min_chunk)
    want = -(-waves * _n_sm(dev) // max(int(n_bk), 1))
    return int(max(1, min(want, max(1, int(ctx) // max(min_chunk, 1)), 64)))


def _row_alloc(k_cache: Tensor, v_cache: Tensor, k_scale: Tensor, v_scale: Tensor, S: int) -> int:
    """Slots really allocated per cache row when the tensors are [:, :, :S] views of a longer allocation (all four
    must agree and the padded rows must lie inside their storages); else S."""
    hd = k_cache.size(-1)
    if k_cache.stride(2) != hd or k_cache.stride(1) % hd:
        return S
    alloc = k_cache.stride(1) // hd
    if alloc <= S or v_cache.stride(1) != alloc * hd or k_scale.stride(1) != alloc or v_scale.stride(1) != alloc:
        return S
    for t, row in ((k_cache, alloc * hd), (v_cache, alloc * hd), (k_scale, alloc), (v_scale, alloc)):
        last = t.storage_offset() + (t.size(0) - 1) * t.stride(0) + (t.size(1) - 1) * t.stride(1) + row
        if last * t.element_size() > t.untyped_storage().nbytes():
            return S
    return alloc


def attn_args(q: Tensor, k_cache: Tensor, v_cache: Tensor, pos: Tensor, starts: Tensor, scale: float, window: int,
              ring: bool, k_scale: Tensor, v_scale: Tensor, num_splits: int, out: Tensor,
              workspace: Tensor | None = None, v_cur: Tensor | None = None, xsa_alpha: Tensor | None = None,
              xsa_eps: float = 1e-4, gate_x: Tensor | None = None, gate_w: Tensor | None = None,
              counters: Tensor | None = None, status: Tensor | None = None,
              row_map: Tensor | None = None, gate_vals: Tensor | None = None) -> "_lib.AttnArgs":
    """uv_attn_args filled from tensor metadata.  q / out (B, H, hd) with unit inner stride."""
    B, H, hd = q.shape
    KH, S = k_cache.shape[1], k_cache.shape[2]
    a = _lib.AttnArgs()
    a.q, a.q_dtype, a.sqb, a.sqh = q.data_ptr(), DTYPE_CODE[q.dtype], q.stride(0), q.stride(1)
    a.k_cache, a.v_cache, a.kv_dtype = k_cache.data_ptr(), v_cache.data_ptr(), DTYPE_CODE[k_cache.dtype]
    a.skb, a.skh, a.sks = k_cache.stride(0), k_cache.stride(1), k_cache.stride(2)
    a.svb, a.svh, a.svs = v_cache.stride(0), v_cache.stride(1), v_cache.stride(2)
    a.k_scale, a.v_scale = k_scale.data_ptr(), v_scale.data_ptr()
    a.ssb, a.ssh, a.stb, a.sth = k_scale.stride(0), k_scale.stride(1), v_scale.stride(0), v_scale.stride(1)
    a.pos, a.starts = pos.data_ptr(), starts.data_ptr()
    a.out, a.sob, a.soh = out.data_ptr(), out.stride(0), out.stride(1)
    a.B, a.H, a.KH, a.hd, a.S = B, H, KH, hd, S
    a.S_alloc = _row_alloc(k_cache, v_cache, k_scale, v_scale, S)
    a.window, a.ring, a.scale, a.num_splits = int(window), int(bool(ring)), float(scale), int(num_splits)
    if num_splits > 1:
        if workspace is not None:
            a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel() * workspace.element_size()
        if counters is not None:
            if counters.numel() < B * KH or counters.dtype != torch.int32:
                raise ValueError("counters must hold B*KH int32 zeros")
            a.counters = counters.data_ptr()
    if status is not None:
        a.status = status.data_ptr()
    if row_map is not None:
        a.row_map = row_map.data_ptr()
    if xsa_alpha is not None:
        a.v_cur, a.v_cur_sb, a.v_cur_sh = v_cur.data_ptr(), v_cur.stride(0), v_cur.stride(1)
        a.xsa_alpha, a.xsa_eps = xsa_alpha.data_ptr(), float(xsa_eps)
    if gate_vals is not None:  # (B, H) fp32 gates computed by uv_qkv_post_args
        a.gate_vals = gate_vals.data_ptr()
    elif gate_w is not None:
        a.gate_x, a.gate_x_stride = gate_x.data_ptr(), gate_x.stride(0)
        a.gate_w, a.gate_ch = gate_w.data_ptr(), gate_w.size(-1)
    return a


def attn_launch(q: Tensor, k_cache: Tensor, v_cache: Tensor, pos: Tensor, starts: Tensor, scale: float, window: int,
                ring: bool, k_scale: Tensor, v_scale: Tensor, num_splits: int, out: Tensor,
                workspace: Tensor | None = None, pre=None, **epilogue) -> Tensor:
    """Raw launch of uv_decode_attn (arguments as ``attn_args``).
    pre: a filled _lib.QkvArgs -> uv_qkv_attn (uv_qkv_post's work done inside the attention launch)."""
    a = attn_args(q, k_cache, v_cache, pos, starts, scale, window, ring, k_scale, v_scale, num_splits, out,
                  workspace, **epilogue)
    with torch.cuda.device(q.device):
        if pre is not None:
            rc = _lib.lib().uv_qkv_attn(C.byref(pre), C.byref(a), stream_ptr(q.device))
        else:
            rc = _lib.lib().uv_decode_attn(C.byref(a), stream_ptr(q.device))
    _lib.check(rc, "uv_qkv_attn" if pre is not None else "uv_decode_attn")
    return out


def workspace_for(B: int, KH: int, G: int, hd: int, num_splits: int, device) -> Tensor | None:
    n = _lib.lib().uv_decode_attn_workspace_bytes(B, KH, G, hd, num_splits)
    return torch.empty(n // 4, dtype=torch.float32, device=device) if n else None


@torch.library.custom_op("uvb200::decode_attn", mutates_args=())
def _decode_attn_op(q: Tensor, k_cache: Tensor, v_cache: Tensor, pos: Tensor, starts: Tensor, scale: float,
                    window: int, ring: bool, k_scale: Tensor, v_scale: Tensor, num_splits: int) -> Tensor:
    out = torch.empty(q.shape, device=q.device, dtype=q.dtype)
    B, H, hd = q.shape
    KH = k_cache.shape[1]
    ws = workspace_for(B, KH, H // KH, hd, num_splits, q.device)
    return attn_launch(q, k_cache, v_cache, pos, starts, scale, window, ring, k_scale, v_scale, num_splits, out, ws)


@_decode_attn_op.register_fake
def _(q, k_cache, v_cache, pos, starts, scale, window, ring, k_scale, v_scale, num_splits):
    return torch.empty_like(q)


def decode_attention(q: Tensor, k_cache: Tensor, v_cache: Tensor, pos: Tensor, starts: Tensor, scale: float, *,
                     window: int = 0, ring: bool | None = None, k_scale: Tensor | None = None,
                     v_scale: Tensor | None = None, ctx_hint: int | None = None, num_splits: int | None = None,
                     block_n: int | None = None, num_warps: int = 1, backend: str = "auto") -> Tensor:
    """Single-query attention for every row of a static KV cache; same contract as decode_attn.py:193-230.

    q (B, H, hd) fp16 / bf16 (a (B, 1, H, hd) view is accepted); k_cache, v_cache (B, K, S, hd) int8 with
    k_scale / v_scale (B, K, S) fp16; pos (B,) = position of the newest key (already written); keys attended are
    positions max(starts[b], pos[b] - window + 1, 0) .. pos[b]; ring: slot of position t is t % S (default:
    window > 0).  block_n / num_warps / backend are accepted and ignored (one kernel, fixed 128-key tiles).
    Registered as the torch custom op ``uvb200::decode_attn`` (opaque to torch.compile, graph-capturable).
    """
    if q.dim() == 4:
        q = q.reshape(q.size(0), q.size(-2), q.size(-1))
    need_cuda(q, k_cache, v_cache, pos, starts, k_scale, v_scale)
    if k_cache.dtype != torch.int8:
        raise NotImplementedError("ultraviolet_b200.decode_attention reads int8 KV caches (kv_dtype='int8')")
    if k_scale is None or v_scale is None:
        raise ValueError("int8 caches need k_scale and v_scale")
    B, H, hd = q.shape
    KH, S = k_cache.shape[1], k_cache.shape[2]
    if ring is None:
        ring = window > 0
    if num_splits is None:
        ctx = ctx_hint or S
        if window > 0:
            ctx = min(ctx, window)
        num_splits = default_splits(B * KH, ctx, q.device)
    if q.stride(-1) != 1:
        q = q.contiguous()
    pos = pos if pos.dtype == torch.int64 else pos.long()
    starts = starts if starts.dtype == torch.int64 else starts.long()
    return _decode_attn_op(q, k_cache, v_cache, pos, starts, float(scale), int(window), bool(ring), k_scale, v_scale,
                           int(num_splits))
