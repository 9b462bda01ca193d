"""fused_sample / fused_sample_ok with the reference's signatures (ultraviolet/kernels/fused_sample.py:61-78) on
uv_sample."""
from __future__ import annotations

import ctypes as C

import torch
from torch import Tensor

from .. import _lib
from ._util import DTYPE_CODE, need_cuda, stream_ptr


def fused_sample_ok(x_or_dev, V: int, softcap, temperature: float, block: int = 1024) -> bool:
    """fused_sample.py:61-65: CUDA device, vocabulary a multiple of 256 (<= 49152), T > 0 and a / T <= 80."""
    dev = x_or_dev.device if isinstance(x_or_dev, Tensor) else torch.device(x_or_dev)
    return dev.type == "cuda" and V % 256 == 0 and 256 <= V <= 49152 and temperature > 0 \
        and float(softcap[0]) / temperature <= 80.0


def fused_sample(x: Tensor, u: Tensor, softcap, temperature: float = 1.0, block: int = 1024,
                 top_p: float = 1.0) -> tuple[Tensor, Tensor]:
    """x (B, V) raw head output (before the softcap), u (B,) fp32 uniforms in [0, 1) -> (tokens int64 (B,),
    log softmax(softcap(x) / T)[token] fp32 (B,)).  Graph-capturable; `block` is accepted and ignored."""
    need_cuda(x, u)
    B, V = x.shape
    if x.stride(1) != 1:
        raise ValueError("fused_sample needs unit stride along the vocabulary")
    out = torch.empty(B, dtype=torch.int64, device=x.device)
    lp = torch.empty(B, dtype=torch.float32, device=x.device)
    a, b, c = (float(v) for v in softcap)
    u = u.to(torch.float32).contiguous()
    with torch.cuda.device(x.device):
        rc = _lib.lib().uv_sample(x.data_ptr(), DTYPE_CODE[x.dtype], x.stride(0), B, V, 0, a, b, c,
                                  float(temperature), float(top_p), u.data_ptr(), C.c_uint64(0), None, None,
                                  out.data_ptr(), lp.data_ptr(), None, None, stream_ptr(x.device))
    _lib.check(rc, "uv_sample")
    return out, lp
