"""The C-ABI library loads and exports every symbol include/uvdecode.h declares; argument validation returns the
documented codes without launching anything (no GPU needed)."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from ultraviolet_b200 import _lib
    if not os.path.exists(_lib.LIB_PATH):
        from ultraviolet_b200.build import build
        build()
    return _lib.lib()


def _declared():
    src = open(os.path.join(ROOT, "include", "uvdecode.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(uv_[a-z0-9_]+)\s*\(", src)))


def test_every_declared_symbol_is_exported_and_bound(lib):
    from ultraviolet_b200 import _lib
    names = _declared()
    assert len(names) >= 14
    for n in names:
        assert hasattr(lib, n), n
    assert set(names) == set(_lib.SIGNATURES), set(names) ^ set(_lib.SIGNATURES)


def test_version_and_error_strings(lib):
    from ultraviolet_b200 import _lib
    assert lib.uv_abi_version() == _lib.UV_ABI_VERSION == 2
    for code in range(0, -7, -1):
        assert lib.uv_error_string(code)
    assert b"unknown" in lib.uv_error_string(-99)


def test_argument_errors_return_codes_without_launching(lib):
    from ultraviolet_b200 import _lib
    assert lib.uv_decode_attn(None, None) == -1
    a = _lib.AttnArgs()
    a.B = 0
    assert lib.uv_decode_attn(C.byref(a), None) == 0            # empty batch: nothing to do
    a.B, a.H, a.KH, a.hd, a.S, a.num_splits = 2, 8, 1, 64, 128, 1
    assert lib.uv_decode_attn(C.byref(a), None) == -1           # null pointers
    assert lib.uv_kv_quant_scatter(None, 0, 64, 4, 64, None, None, None, 4, None, None) == -1
    assert lib.uv_kv_quant_scatter(None, 0, 64, 0, 64, None, None, None, 0, None, None) == 0
    assert lib.uv_sample(None, 2, 0, 4, 16384, 0, 23.0, 5.0, 7.5, 1.0, 1.0, None, 0, None, None, None, None,
                         None, None, None) == -1
    assert lib.uv_sched_step(None, None) == -1
    assert lib.uv_embed_norm(None, None, 2, 10, 640, None, None, 0, None) == 0


def test_split_heuristic_and_workspace(lib):
    # one resident wave (4 CTAs per SM): 512 rows leave room for one split each, 64 rows for 9 -> 8 (cluster merge)
    assert lib.uv_default_splits(512, 2320, 148) == 1
    assert lib.uv_default_splits(64, 8192, 148) == 8
    assert lib.uv_default_splits(128, 4096, 148) == 4
    assert lib.uv_default_splits(8, 32768, 148) == 16  # a batch too small to fill the SMs with 8 splits per row
    for n_bk, ctx in ((16, 8192), (64, 2048), (256, 2048), (3, 70000)):
        s = lib.uv_default_splits(n_bk, ctx, 148)
        assert 1 <= s <= 64 and n_bk * s <= 4 * 148 + n_bk
    assert lib.uv_default_splits(4096, 256, 148) == 1
    assert lib.uv_default_splits(1, 100, 148) == 1
    assert lib.uv_decode_attn_workspace_bytes(64, 1, 8, 64, 1) == 0
    assert lib.uv_decode_attn_workspace_bytes(64, 1, 8, 64, 10) == 64 * 10 * 8 * 66 * 4
