from __future__ import annotations

import torch

from .. import _lib

DTYPE_CODE = {torch.float32: _lib.UV_F32, torch.float16: _lib.UV_F16, torch.bfloat16: _lib.UV_BF16,
              torch.int8: _lib.UV_I8}


def need_cuda(*tensors) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("ultraviolet_b200 kernels run on CUDA tensors only (no CPU fallback); got a "
                               f"{t.device} tensor")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"tensors on different devices: {dev} and {t.device}")
    return dev


def stream_ptr(dev: torch.device) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()
