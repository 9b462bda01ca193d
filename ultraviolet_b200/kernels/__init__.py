"""sm_100a decode kernels behind the reference's ``ultraviolet.kernels`` names (ultraviolet/kernels/__init__.py:9-10).

``decode_attention`` / ``default_splits`` / ``quantize_kv`` / ``dequantize_kv`` / ``kv_write`` / ``kv_write_rows`` keep
the reference signatures; every one of them launches a kernel of libuvdecode.so on the tensors' CUDA device and raises
on CPU tensors (there is no eager fallback).
"""
from .decode_attn import decode_attention, default_splits  # noqa: F401
from .kv_quant import dequantize_kv, kv_append, kv_write, kv_write_rows, quantize_kv  # noqa: F401
from .sampling import fused_sample, fused_sample_ok  # noqa: E402,F401


def decode_attention_ref(q, k_cache, v_cache, pos, starts, scale, *, window: int = 0, ring=None, k_scale=None,
                         v_scale=None):
    """Name kept from ultraviolet/kernels/decode_attn.py:233-263 for callers that import it.  The reference's
    function is its dense fp32 torch cross-check; this package has no torch or CPU path, so the name runs the same
    CUDA kernel in its plainest form (one split: no partials, no merge) on CUDA tensors and int8 caches.  For an
    independent check keep using the reference's own function (it runs on any device)."""
    return decode_attention(q, k_cache, v_cache, pos, starts, scale, window=window, ring=ring, k_scale=k_scale,
                            v_scale=v_scale, num_splits=1)


def fused_sample_ref(x, u, softcap, temperature: float = 1.0):
    """Name kept from ultraviolet/kernels/fused_sample.py:81-91: same inputs and outputs as ``fused_sample``, which it
    calls (the reference's version is the eager-torch restatement of its Triton kernel; there is no eager path here)."""
    return fused_sample(x, u, softcap, temperature)
