"""sm_100a decode kernels behind the reference's ``ultraviolet.kernels`` names (ultraviolet/kernels/__init__.py:9-10).

``decode_attention`` / ``default_splits`` / ``quantize_kv`` / ``dequantize_kv`` / ``kv_write`` / ``kv_write_rows`` keep
the reference signatures; every one of them launches a kernel of libuvdecode.so on the tensors' CUDA device and raises
on CPU tensors (there is no eager fallback).
"""
from .decode_attn import decode_attention, default_splits  # noqa: F401
from .kv_quant import dequantize_kv, kv_append, kv_write, kv_write_rows, quantize_kv  # noqa: F401
from .sampling import fused_sample, fused_sample_ok  # noqa: E402,F401
