"""uv_decode_attn_static: the allocation-free entry point (split partials and counters in a device array built into
the library) against the regular entry point, through the C ABI, twice in a row.

Collected last on purpose (file name): a run that stops at the first failure has then already run everything else.
The test builds its own inputs, so it passes alone in a fresh process as well as after the other tests -- including
after tests that left other data in the shared array."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _args(q, k, v, ks, vs, pos, starts, out, splits, scale):
    from ultraviolet_b200 import _lib
    from ultraviolet_b200.kernels._util import DTYPE_CODE
    a = _lib.AttnArgs()
    B, H, hd = q.shape
    a.q, a.q_dtype, a.sqb, a.sqh = q.data_ptr(), DTYPE_CODE[q.dtype], q.stride(0), q.stride(1)
    a.k_cache, a.v_cache, a.kv_dtype = k.data_ptr(), v.data_ptr(), DTYPE_CODE[k.dtype]
    a.skb, a.skh, a.sks = k.stride(0), k.stride(1), k.stride(2)
    a.svb, a.svh, a.svs = v.stride(0), v.stride(1), v.stride(2)
    a.k_scale, a.v_scale = ks.data_ptr(), vs.data_ptr()
    a.ssb, a.ssh, a.stb, a.sth = ks.stride(0), ks.stride(1), vs.stride(0), vs.stride(1)
    a.pos, a.starts, a.out, a.sob, a.soh = pos.data_ptr(), starts.data_ptr(), out.data_ptr(), out.stride(0), out.stride(1)
    a.B, a.H, a.KH, a.hd, a.S = B, H, k.shape[1], hd, k.shape[2]
    a.window, a.ring, a.scale, a.num_splits = 0, 0, scale, splits
    return a


def test_static_scratch_entry_matches_regular_entry_twice():
    from ultraviolet_b200 import _lib
    from ultraviolet_b200.kernels._util import stream_ptr
    lib = _lib.lib()
    g = torch.Generator(device=DEV).manual_seed(11)
    B, H, hd, S, splits = 24, 8, 64, 1536, 5
    sp = stream_ptr(torch.device(DEV))
    for call in range(2):  # second call: new data over the contents the first call left in the array
        q = torch.randn(B, H, hd, device=DEV, generator=g).to(torch.bfloat16)
        k = torch.randint(-127, 128, (B, 1, S, hd), device=DEV, dtype=torch.int8, generator=g)
        v = torch.randint(-127, 128, (B, 1, S, hd), device=DEV, dtype=torch.int8, generator=g)
        ks = (torch.rand(B, 1, S, device=DEV, generator=g) * 0.02 + 0.01).half()
        vs = (torch.rand(B, 1, S, device=DEV, generator=g) * 0.02 + 0.01).half()
        pos = torch.randint(200, S, (B,), device=DEV, generator=g)
        starts = torch.randint(0, 100, (B,), device=DEV, generator=g)
        # regular entry point: caller-owned workspace and counters
        ref = torch.empty_like(q)
        ws = torch.empty(lib.uv_decode_attn_workspace_bytes(B, 1, H, hd, splits) // 4, dtype=torch.float32, device=DEV)
        cnt = torch.zeros(B, dtype=torch.int32, device=DEV)
        a = _args(q, k, v, ks, vs, pos, starts, ref, splits, 0.14125)
        a.workspace, a.workspace_bytes, a.counters = ws.data_ptr(), ws.numel() * 4, cnt.data_ptr()
        _lib.check(lib.uv_decode_attn(C.byref(a), sp), "uv_decode_attn")
        # allocation-free entry point: no workspace, no counters
        out = torch.full_like(q, float("nan"))
        b = _args(q, k, v, ks, vs, pos, starts, out, splits, 0.14125)
        _lib.check(lib.uv_decode_attn_static(C.byref(b), sp), "uv_decode_attn_static")
        torch.cuda.synchronize()
        assert torch.isfinite(out.float()).all()
        torch.testing.assert_close(out.float(), ref.float(), atol=2e-3, rtol=2e-3)
        # and not only against the sibling entry point: three rows against the CPU oracle on the same bytes
        from oracle import attn as oattn
        rows = [0, B // 2, B - 1]
        want = oattn.decode_attention_ref(q[rows].float().cpu().numpy(), k[rows].cpu().numpy(), v[rows].cpu().numpy(),
                                          pos[rows].cpu().numpy(), starts[rows].cpu().numpy(), 0.14125,
                                          k_scale=ks[rows].cpu().numpy(), v_scale=vs[rows].cpu().numpy())
        got = out[rows].float().cpu().numpy()
        assert np.abs(got - want).max() <= 2e-2 * np.abs(want).max()   # bf16 queries and output


def test_static_scratch_rejects_oversized_problems():
    from ultraviolet_b200 import _lib
    lib = _lib.lib()
    z = torch.zeros(1, device=DEV)
    a = _lib.AttnArgs()
    a.q = a.k_cache = a.v_cache = a.k_scale = a.v_scale = a.pos = a.starts = a.out = z.data_ptr()
    a.B, a.H, a.KH, a.hd, a.S, a.num_splits = 512, 8, 1, 64, 4096, 16      # 512*16*8*66*4 B = 17 MiB of partials
    assert lib.uv_decode_attn_static(C.byref(a), None) == -7
    a.B, a.num_splits = 5000, 1                                             # more cache rows than counters
    assert lib.uv_decode_attn_static(C.byref(a), None) == -7
    assert b"built-in scratch" in lib.uv_error_string(-7)
