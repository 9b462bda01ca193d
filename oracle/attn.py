"""Oracle (test infrastructure): single-query decode attention over the slot-indexed KV cache, numpy restatement of
``decode_attention_ref`` (ultraviolet/kernels/decode_attn.py:233-263).
"""
from __future__ import annotations

import numpy as np


def _valid_mask(pos, starts, S, window, ring):
    """(B, S) bool: which cache slots hold a key the row attends to (decode_attn.py:249-258)."""
    p = np.asarray(pos, dtype=np.int64)[:, None]
    slot = np.arange(S, dtype=np.int64)[None, :]
    if ring:
        tpos = p - np.remainder(p - slot, S)  # absolute position currently held by each ring slot
    else:
        tpos = np.broadcast_to(slot, (p.shape[0], S))
    lo = np.maximum(np.asarray(starts, dtype=np.int64)[:, None], 0)
    if window > 0:
        lo = np.maximum(lo, p - window + 1)
    return (tpos >= lo) & (tpos <= p)


def attention_key_counts(pos, starts, window: int = 0) -> np.ndarray:
    """n_b = pos_b - max(starts_b, pos_b - window + 1, 0) + 1: keys each row reads (decode_attn.py:38-41)."""
    p = np.asarray(pos, dtype=np.int64)
    lo = np.maximum(np.asarray(starts, dtype=np.int64), 0)
    if window > 0:
        lo = np.maximum(lo, p - window + 1)
    return p + 1 - lo


def decode_attention_ref(q, k_cache, v_cache, pos, starts, scale, *, window: int = 0, ring=None,
                         k_scale=None, v_scale=None) -> np.ndarray:
    """decode_attn.py:233-263 in fp32.  q (B, H, hd); caches (B, K, S, hd) int8 (+ (B, K, S) fp16 scales) or float;
    pos = position of the newest key (already in the cache); returns (B, H, hd) fp32."""
    q = np.asarray(q, dtype=np.float32)
    if q.ndim == 4:
        q = q.reshape(q.shape[0], q.shape[-2], q.shape[-1])
    B, H, hd = q.shape
    KH, S = k_cache.shape[1], k_cache.shape[2]
    G = H // KH
    if ring is None:
        ring = window > 0
    kf = k_cache.astype(np.float32)
    vf = v_cache.astype(np.float32)
    if k_cache.dtype == np.int8:
        kf = kf * k_scale.astype(np.float32)[..., None]
        vf = vf * v_scale.astype(np.float32)[..., None]
    valid = _valid_mask(pos, starts, S, window, ring)
    qf = q.reshape(B, KH, G, hd)
    s = np.einsum("bkgd,bksd->bkgs", qf, kf, optimize=True) * np.float32(scale)
    s = np.where(valid[:, None, None, :], s, -np.inf).astype(np.float32)
    m = s.max(-1, keepdims=True)
    e = np.exp(s - m)
    w = e / e.sum(-1, keepdims=True)
    return np.einsum("bkgs,bksd->bkgd", w.astype(np.float32), vf, optimize=True).reshape(B, H, hd)


def varlen_attention_ref(q, k, v, cu_seqlens, scale, window=None) -> np.ndarray:
    """fp32 packed causal attention, restating ``varlen_attention_ref`` (ultraviolet/kernels/varlen_attn.py:94-114):
    q (N, H, hd), k / v (N, K, hd) packed along N, cu_seqlens (S + 1,) segment boundaries; query i of a segment sees
    keys j of the same segment with 0 <= i - j < window (window None / 0: all j <= i).  Returns (N, H, hd)."""
    q, k, v = (np.asarray(a, dtype=np.float32) for a in (q, k, v))
    H, K = q.shape[1], k.shape[1]
    G = H // K
    out = np.zeros_like(q)
    cu = [int(c) for c in cu_seqlens]
    for a, b in zip(cu[:-1], cu[1:]):
        L = b - a
        if L == 0:
            continue
        kk = np.repeat(k[a:b], G, axis=1)          # (L, H, hd): kv head h serves query heads h*G .. h*G + G - 1
        vv = np.repeat(v[a:b], G, axis=1)
        s = np.einsum("ihd,jhd->hij", q[a:b], kk, optimize=True) * np.float32(scale)
        i = np.arange(L)
        d = i[:, None] - i[None, :]
        m = d >= 0
        if window:
            m = m & (d < window)
        s = np.where(m[None], s, -np.inf).astype(np.float32)
        e = np.exp(s - s.max(-1, keepdims=True))
        w = e / e.sum(-1, keepdims=True)
        out[a:b] = np.einsum("hij,jhd->ihd", w.astype(np.float32), vv, optimize=True)
    return out
