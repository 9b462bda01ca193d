"""Oracle (test infrastructure): int8 KV quantiser and cache writes, numpy restatement of
ultraviolet/kernels/kv_quant.py.

Cache layout: values (B, K, S, hd) int8, scales (B, K, S) fp16; flat row index of (row b, kv head h, slot s) is
(b*K + h)*S + s for both (kv_quant.py:3-4).
"""
from __future__ import annotations

import numpy as np

_F127 = np.float32(127.0)
_TINY = np.float32(1e-30)


def quantize_kv(x: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """kv_quant.py:12-19.  x (..., hd) -> (int8 (..., hd), fp16 scale (...)).

    scale16 = fp16_rne(max|x| / 127) with the division in fp32; values are divided (true fp32 division) by the
    fp16-rounded scale, rounded half-to-even and clamped to [-127, 127].  All-zero rows give q = 0, scale = 0.
    """
    xf = np.asarray(x, dtype=np.float32)
    s16 = (np.abs(xf).max(axis=-1) / _F127).astype(np.float16)
    sf = np.maximum(s16.astype(np.float32), _TINY)
    with np.errstate(over="ignore", invalid="ignore"):
        q = np.rint(xf / sf[..., None])
    q = np.clip(q, -127.0, 127.0).astype(np.int8)
    return q, s16


def dequantize_kv(q: np.ndarray, s: np.ndarray) -> np.ndarray:
    """kv_quant.py:22-23 (returned in fp32)."""
    return q.astype(np.float32) * s.astype(np.float32)[..., None]


def kv_write(cache: np.ndarray, scale: np.ndarray | None, flat_idx: np.ndarray, x: np.ndarray) -> None:
    """kv_quant.py:26-36.  One token per (row, kv head): rows of the flat (B*K*S, hd) view at flat_idx."""
    hd = cache.shape[-1]
    x = np.asarray(x).reshape(-1, hd)
    flat = cache.reshape(-1, hd)
    assert flat.base is not None or flat is cache  # must be a view
    if scale is None:
        flat[flat_idx] = x.astype(cache.dtype)
    else:
        q, s = quantize_kv(x)
        flat[flat_idx] = q
        scale.reshape(-1)[flat_idx] = s


def kv_write_rows(cache: np.ndarray, scale: np.ndarray | None, new: np.ndarray, slots, rows=None) -> None:
    """kv_quant.py:39-54.  Prefill-time write of new (n, K, T', hd) into cache[rows][:, :, slots]."""
    if scale is None:
        vals = [(cache, new.astype(cache.dtype))]
    else:
        q, s = quantize_kv(new)
        vals = [(cache, q), (scale, s)]
    for dst, src in vals:
        if rows is None:
            dst[:, :, slots] = src
        else:
            for j, r in enumerate(np.asarray(rows).tolist()):
                dst[r][:, slots] = src[j]
