"""int8 KV cache quantiser and writes (API of ultraviolet/kernels/kv_quant.py) on the fused sm_100a kernel."""
from __future__ import annotations

import torch
from torch import Tensor

from .. import _lib
from ._util import DTYPE_CODE, need_cuda, ptr, stream_ptr


def _rows(x: Tensor, hd: int) -> Tensor:
    """(…, hd) -> 2-D (n, hd) view with unit inner stride (copy only if the layout forces one)."""
    x2 = x.reshape(-1, hd)
    if x2.stride(-1) != 1 or x2.dtype not in DTYPE_CODE or x2.dtype == torch.int8:
        x2 = x2.contiguous() if x2.dtype in (torch.float32, torch.float16, torch.bfloat16) else x2.float().contiguous()
    return x2


def quantize_kv(x: Tensor) -> tuple[Tensor, Tensor]:
    """x (..., hd) float -> (int8 (..., hd), fp16 scale (...)); bit-exact with kv_quant.py:12-19."""
    need_cuda(x)
    hd = x.size(-1)
    x2 = _rows(x, hd)
    q = torch.empty(x2.shape, dtype=torch.int8, device=x.device)
    s = torch.empty(x2.size(0), dtype=torch.float16, device=x.device)
    with torch.cuda.device(x.device):
        rc = _lib.lib().uv_kv_quant_scatter(x2.data_ptr(), DTYPE_CODE[x2.dtype], x2.stride(0), x2.size(0), hd,
                                            q.data_ptr(), s.data_ptr(), None, x2.size(0), None, stream_ptr(x.device))
    _lib.check(rc, "uv_kv_quant_scatter")
    return q.view(x.shape), s.view(x.shape[:-1])


def dequantize_kv(q: Tensor, s: Tensor, dtype=torch.float16) -> Tensor:
    """kv_quant.py:22-23 (plain elementwise torch; not on the decode path)."""
    return (q.float() * s.float().unsqueeze(-1)).to(dtype)


def kv_write(cache: Tensor, scale: Tensor | None, flat_idx: Tensor, x: Tensor) -> None:
    """kv_quant.py:26-36: one token per (row, kv head); cache (B, K, S, hd), scale (B, K, S) fp16 or None,
    flat_idx (B*K,) = (b*K + h)*S + slot."""
    need_cuda(cache, scale, flat_idx, x)
    hd = cache.size(-1)
    if scale is None:  # 16-bit cache: a plain row scatter
        cache.view(-1, hd).index_copy_(0, flat_idx, x.reshape(-1, hd).to(cache.dtype))
        return
    if not cache.is_contiguous() or not scale.is_contiguous():
        raise RuntimeError("kv_write needs contiguous cache / scale tensors")
    x2 = _rows(x, hd)
    idx = flat_idx.to(torch.int64).contiguous()
    with torch.cuda.device(cache.device):
        rc = _lib.lib().uv_kv_quant_scatter(x2.data_ptr(), DTYPE_CODE[x2.dtype], x2.stride(0), x2.size(0), hd,
                                            cache.data_ptr(), scale.data_ptr(), idx.data_ptr(),
                                            cache.numel() // hd, None, stream_ptr(cache.device))
    _lib.check(rc, "uv_kv_quant_scatter")


def kv_append(k_cache: Tensor, v_cache: Tensor, k_scale: Tensor, v_scale: Tensor, pos: Tensor, k: Tensor, v: Tensor,
              ring: bool) -> None:
    """Decode-time append of one token per cache row: both kv_write calls of a layer (fast_decode.py:316-317) in one
    launch, slot computed on the device from pos (ring: pos % S)."""
    need_cuda(k_cache, v_cache, k_scale, v_scale, pos, k, v)
    B, KH, S, hd = k_cache.shape
    if not (k_cache.is_contiguous() and v_cache.is_contiguous() and k_scale.is_contiguous()
            and v_scale.is_contiguous()):
        raise RuntimeError("kv_append needs contiguous caches and scales")
    k2, v2 = _rows(k, hd), _rows(v, hd)
    if k2.dtype != v2.dtype:
        v2 = v2.to(k2.dtype)
    with torch.cuda.device(k_cache.device):
        rc = _lib.lib().uv_kv_append(k2.data_ptr(), v2.data_ptr(), DTYPE_CODE[k2.dtype], k2.stride(0), v2.stride(0),
                                     k_cache.data_ptr(), v_cache.data_ptr(), k_scale.data_ptr(), v_scale.data_ptr(),
                                     pos.data_ptr(), B, KH, hd, S, int(ring), None, stream_ptr(k_cache.device))
    _lib.check(rc, "uv_kv_append")


def kv_write_rows(cache: Tensor, scale: Tensor | None, new: Tensor, slots, rows: Tensor | None = None) -> None:
    """kv_quant.py:39-54: prefill-time write of new (n, K, T', hd) into cache[rows][:, :, slots]."""
    need_cuda(cache, scale, new)
    if scale is not None and _write_rows_fused(cache, scale, new, slots, rows):
        return
    if scale is None:
        vals = [(cache, new.to(cache.dtype))]
    else:
        q, s = quantize_kv(new)
        vals = [(cache, q), (scale, s)]
    for dst, src in vals:
        if rows is None:
            dst[:, :, slots] = src
        elif isinstance(slots, slice):
            dst[rows, :, slots] = src
        else:
            dst[rows[:, None], :, slots[None, :]] = src.transpose(1, 2)


def _write_rows_fused(cache: Tensor, scale: Tensor, new: Tensor, slots, rows: Tensor | None) -> bool:
    """kv_write_rows as ONE launch of the fused quantise + scatter kernel: the destination of every (row, head,
    token) vector is computed as a flat cache-row index (integer arithmetic on a few small tensors) and handed to
    uv_kv_quant_scatter, so the payload is read once and written once.  Returns False when the layout is not the
    (B, K, S_alloc, hd) / (B, K, S_alloc) pair of a decode state (the caller then scatters with torch indexing)."""
    Bc, K, S, hd = cache.shape
    n, Kn, T, hdn = new.shape
    pitch = cache.stride(1) // hd if hd else 0
    if (Kn != K or hdn != hd or cache.stride(3) != 1 or cache.stride(2) != hd or cache.stride(1) != pitch * hd
            or cache.stride(0) != K * pitch * hd or scale.stride(2) != 1 or scale.stride(1) != pitch
            or scale.stride(0) != K * pitch or pitch < S or T == 0 or n == 0):
        return False
    dev = cache.device
    if isinstance(slots, slice):
        sl = torch.arange(S, device=dev)[slots]
    else:
        sl = torch.as_tensor(slots, device=dev).to(torch.int64).reshape(-1)
        sl = torch.where(sl < 0, sl + S, sl)
    if sl.numel() != T:
        return False
    r = torch.arange(Bc, device=dev) if rows is None else rows.to(dev, torch.int64).reshape(-1)
    if r.numel() != n:
        return False
    idx = ((r[:, None, None] * K + torch.arange(K, device=dev)[None, :, None]) * pitch + sl[None, None, :]).reshape(-1)
    x2 = _rows(new, hd)
    with torch.cuda.device(dev):
        rc = _lib.lib().uv_kv_quant_scatter(x2.data_ptr(), DTYPE_CODE[x2.dtype], x2.stride(0), x2.size(0), hd,
                                            cache.data_ptr(), scale.data_ptr(), idx.contiguous().data_ptr(),
                                            Bc * K * pitch, None, stream_ptr(dev))
    _lib.check(rc, "uv_kv_quant_scatter")
    return True
