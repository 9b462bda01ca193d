"""ctypes binding of libuvdecode.so (declared in include/uvdecode.h).

The library is the product: there is no Python or torch fallback for any entry point.  ``lib()`` raises if the
shared object is missing instead of degrading silently.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("UVDECODE_LIB") or os.path.join(HERE, "libuvdecode.so")

UV_F32, UV_F16, UV_BF16, UV_I8 = 0, 1, 2, 3
UV_ABI_VERSION = 2

_lock = threading.Lock()
_lib = None


class UvError(RuntimeError):
    pass


class AttnArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("q_dtype", C.c_int), ("sqb", C.c_int64), ("sqh", C.c_int64),
        ("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("kv_dtype", C.c_int),
        ("skb", C.c_int64), ("skh", C.c_int64), ("sks", C.c_int64),
        ("svb", C.c_int64), ("svh", C.c_int64), ("svs", C.c_int64),
        ("k_scale", C.c_void_p), ("v_scale", C.c_void_p),
        ("ssb", C.c_int64), ("ssh", C.c_int64), ("stb", C.c_int64), ("sth", C.c_int64),
        ("pos", C.c_void_p), ("starts", C.c_void_p), ("row_map", C.c_void_p),
        ("out", C.c_void_p), ("sob", C.c_int64), ("soh", C.c_int64),
        ("B", C.c_int), ("H", C.c_int), ("KH", C.c_int), ("hd", C.c_int), ("S", C.c_int), ("S_alloc", C.c_int),
        ("window", C.c_int), ("ring", C.c_int), ("scale", C.c_float), ("num_splits", C.c_int),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("counters", C.c_void_p), ("status", C.c_void_p),
        ("v_cur", C.c_void_p), ("v_cur_sb", C.c_int64), ("v_cur_sh", C.c_int64), ("xsa_alpha", C.c_void_p), ("xsa_eps", C.c_float),
        ("gate_x", C.c_void_p), ("gate_x_stride", C.c_int64), ("gate_w", C.c_void_p), ("gate_ch", C.c_int),
        ("gate_vals", C.c_void_p),
    ]


class QkvArgs(C.Structure):
    """uv_qkv_args (include/uvdecode.h): the parameters of uv_qkv_post, by name."""
    _fields_ = [
        ("qkv", C.c_void_p), ("xn", C.c_void_p), ("tok", C.c_void_p), ("value_embed", C.c_void_p),
        ("ve_gate", C.c_void_p), ("inv_freq", C.c_void_p), ("pos", C.c_void_p),
        ("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("k_scale", C.c_void_p), ("v_scale", C.c_void_p),
        ("row_map", C.c_void_p), ("oob_count", C.c_void_p), ("dtype", C.c_int), ("vocab", C.c_int64),
        ("B", C.c_int), ("H", C.c_int), ("K", C.c_int), ("hd", C.c_int), ("d", C.c_int), ("S", C.c_int),
        ("S_alloc", C.c_int), ("ring", C.c_int), ("ve_ch", C.c_int), ("n_pairs", C.c_int),
        ("rope_cs", C.c_void_p), ("gate_w", C.c_void_p), ("gate_out", C.c_void_p), ("gate_ch", C.c_int),
        ("last_pos", C.c_void_p), ("xn_raw", C.c_int),
    ]


class PrefillAttnArgs(C.Structure):
    """uv_prefill_attn_args (include/uvdecode.h)."""
    _fields_ = [
        ("qkv", C.c_void_p), ("dtype", C.c_int), ("ld", C.c_int64), ("cu_seqlens", C.c_void_p),
        ("tile_cu", C.c_void_p), ("n_seq", C.c_int), ("max_tiles", C.c_int), ("out", C.c_void_p), ("ldo", C.c_int64),
        ("H", C.c_int), ("K", C.c_int), ("hd", C.c_int), ("window", C.c_int), ("scale", C.c_float),
        ("xsa_alpha", C.c_void_p), ("xsa_eps", C.c_float), ("gate_vals", C.c_void_p),
    ]


class SchedArgs(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in (
        "req", "fed", "gen", "cur_tok", "pos", "starts", "row_key", "step_ctr", "samp_tok", "samp_lp", "prompt_off",
        "prompt_len", "limit", "key", "out_off", "out_len", "start_version", "tokens", "out_tok", "out_lp",
        "fin_ring", "ctl")] + [("B", C.c_int), ("q_cap", C.c_int), ("tok_cap", C.c_int64), ("out_cap", C.c_int64),
                               ("eos", C.c_int), ("pad", C.c_int), ("force_eos", C.c_int), ("max_len", C.c_int64),
                               ("row_map", C.c_void_p), ("lanes", C.c_int), ("lane_chunk", C.c_int),
                               ("ring_len", C.c_int64), ("no_admit", C.c_int), ("compact", C.c_int),
                               ("step_row", C.c_void_p), ("pend_req", C.c_void_p), ("pend_fed", C.c_void_p),
                               ("pend_tok", C.c_void_p), ("pend_pos", C.c_void_p), ("pend_key", C.c_void_p)]


class SchedAdmitArgs(C.Structure):
    """uv_sched_admit_args (include/uvdecode.h)."""
    _fields_ = [("tok", C.c_void_p), ("pos", C.c_void_p), ("row", C.c_void_p), ("last_pos", C.c_void_p),
                ("cu", C.c_void_p), ("tile_cu", C.c_void_p), ("cap", C.c_int), ("reserved_", C.c_int)]


# name -> (restype, argtypes); every symbol include/uvdecode.h declares
SIGNATURES = {
    "uv_abi_version": (C.c_int, []),
    "uv_error_string": (C.c_char_p, [C.c_int]),
    "uv_last_cuda_error": (C.c_int, []),
    "uv_kv_quant_scatter": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_int, C.c_void_p, C.c_void_p,
                                      C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]),
    "uv_kv_append": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p,
                               C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                               C.c_void_p, C.c_void_p]),
    "uv_decode_attn_workspace_bytes": (C.c_size_t, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "uv_default_splits": (C.c_int, [C.c_int, C.c_int, C.c_int]),
    "uv_decode_attn": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p]),
    "uv_decode_attn_uses_bulk": (C.c_int, [C.POINTER(AttnArgs)]),
    "uv_decode_attn_static": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p]),
    "uv_embed_norm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_void_p, C.c_void_p, C.c_int,
                                C.c_void_p]),
    "uv_embed_norm_rope": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_void_p, C.c_void_p,
                                     C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
    "uv_embed_norm_ss": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_void_p, C.c_void_p,
                                   C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                   C.c_void_p]),
    "uv_qkv_post": (C.c_int, [C.c_void_p] * 13 + [C.c_int, C.c_int64] + [C.c_int] * 10 + [C.c_void_p]),
    "uv_qkv_post_args": (C.c_int, [C.POINTER(QkvArgs), C.c_void_p]),
    "uv_prefill_attn": (C.c_int, [C.POINTER(PrefillAttnArgs), C.c_void_p]),
    "uv_qkv_attn": (C.c_int, [C.POINTER(QkvArgs), C.POINTER(AttnArgs), C.c_void_p]),
    "uv_resid_norm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_int,
                                C.c_void_p]),
    "uv_swiglu": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p]),
    "uv_swiglu_rs": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p]),
    "uv_gemm_qkv": (C.c_int, [C.c_void_p, C.c_int64] + [C.c_void_p] * 13 + [C.c_int, C.c_int64] + [C.c_int] * 10
                    + [C.c_void_p]),
    "uv_gemm_tc": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int, C.c_int,
                             C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "uv_gemm_tc_swiglu": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                    C.c_void_p, C.c_void_p]),
    "uv_gemm_sw": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_int,
                             C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "uv_gemm_sw_qkv": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.POINTER(QkvArgs), C.c_void_p, C.c_int, C.c_int,
                                 C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "uv_gemm_sw_swiglu": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                    C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]),
    "uv_gemm_sw_resid": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                   C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                   C.c_void_p, C.c_void_p]),
    "uv_gemm_swiglu": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                 C.c_void_p]),
    "uv_gemm_resid_norm": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                     C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "uv_sched_step": (C.c_int, [C.POINTER(SchedArgs), C.c_void_p]),
    "uv_sched_admit": (C.c_int, [C.POINTER(SchedArgs), C.POINTER(SchedAdmitArgs), C.c_void_p]),
    "uv_sched_enqueue": (C.c_int, [C.POINTER(SchedArgs), C.c_int, C.c_void_p]),
    "uv_sched_commit": (C.c_int, [C.POINTER(SchedArgs), C.c_void_p]),
    "uv_sample_topk": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_float, C.c_float,
                                 C.c_float, C.c_float, C.c_int, C.c_float, C.c_void_p, C.c_uint64, C.c_void_p,
                                 C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "uv_sample": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_float, C.c_float,
                            C.c_float, C.c_float, C.c_float, C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p,
                            C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
}


def lib() -> C.CDLL:
    """Load libuvdecode.so once; raise loudly if it has not been built (python -m ultraviolet_b200.build)."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise UvError(f"{LIB_PATH} is missing: build it with `python -m ultraviolet_b200.build` "
                              "(nvcc, sm_100a). There is no fallback path.")
            h = C.CDLL(LIB_PATH)
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(h, name)  # AttributeError if the library does not export a declared symbol
                fn.restype, fn.argtypes = res, args
            if h.uv_abi_version() != UV_ABI_VERSION:
                raise UvError(f"libuvdecode ABI {h.uv_abi_version()} != binding {UV_ABI_VERSION}: rebuild")
            _lib = h
    return _lib


def check(code: int, what: str) -> None:
    if code != 0:
        h = lib()
        msg = h.uv_error_string(code).decode()
        if code == -6:
            msg += f" [cudaError {h.uv_last_cuda_error()}]"
        raise UvError(f"{what}: {msg} (code {code})")
