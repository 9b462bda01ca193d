"""tcgen05 / TMEM / TMA GEMM (csrc/gemm_tc.cu) against a plain fp32 PyTorch reference of the same product, and its
SwiGLU epilogue against library GEMM + uv_swiglu (same rounding points: bit-identical)."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _lib():
    from ultraviolet_b200 import _lib
    return _lib, _lib.lib()


@pytest.mark.parametrize("M,N,K", [(128, 64, 64), (256, 640, 640), (200, 3328, 640), (256, 640, 1664), (37, 128, 512),
                                   (640, 16384, 640)])
def test_gemm_tc_matches_fp32_reference(M, N, K):
    L, lib = _lib()
    g = torch.Generator(device=DEV).manual_seed(M + N + K)
    a = (torch.randn(M, K, device=DEV, generator=g) * 0.5).bfloat16()
    w = (torch.randn(N, K, device=DEV, generator=g) * 0.1).bfloat16()
    c = torch.full((M, N), 7.0, device=DEV, dtype=torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    L.check(lib.uv_gemm_tc(a.data_ptr(), K, w.data_ptr(), K, c.data_ptr(), N, 2, M, N, K, status.data_ptr(),
                           torch.cuda.current_stream().cuda_stream), "uv_gemm_tc")
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    ref = a.float() @ w.float().t()
    # one bf16 rounding of an fp32-accumulated product: half an ulp of the largest magnitude, plus summation order
    tol = ref.abs().max().item() * 2.0 ** -8
    assert (c.float() - ref).abs().max().item() <= tol
    assert torch.equal(c, torch.mm(a, w.t())) or (c.float() - torch.mm(a, w.t()).float()).abs().max().item() <= tol


@pytest.mark.parametrize("M,K,f", [(256, 640, 1664), (100, 128, 64), (512, 640, 1664)])
def test_gemm_tc_swiglu_equals_gemm_then_swiglu(M, K, f):
    L, lib = _lib()
    g = torch.Generator(device=DEV).manual_seed(M + f)
    a = (torch.randn(M, K, device=DEV, generator=g) * 0.5).bfloat16()
    w = (torch.randn(2 * f, K, device=DEV, generator=g) * 0.1).bfloat16()
    act = torch.full((M, f), 7.0, device=DEV, dtype=torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    sp = torch.cuda.current_stream().cuda_stream
    L.check(lib.uv_gemm_tc_swiglu(a.data_ptr(), K, w.data_ptr(), act.data_ptr(), 2, M, K, f, status.data_ptr(), sp),
            "uv_gemm_tc_swiglu")
    gu = torch.mm(a, w.t())
    ref = torch.empty_like(act)
    L.check(lib.uv_swiglu(gu.data_ptr(), 2, f, ref.data_ptr(), M, sp), "uv_swiglu")
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    # same products (fp32 accumulation of the same bf16 operands), same rounding points: equal up to the summation
    # order inside the two GEMMs
    diff = (act.float() - ref.float()).abs().max().item()
    assert diff <= ref.float().abs().max().item() * 2.0 ** -7, diff
    assert (act == ref).float().mean().item() > 0.99


def test_gemm_tc_rejects_bad_arguments():
    L, lib = _lib()
    a = torch.zeros(128, 96, device=DEV, dtype=torch.bfloat16)
    c = torch.zeros(128, 64, device=DEV, dtype=torch.bfloat16)
    assert lib.uv_gemm_tc(a.data_ptr(), 96, a.data_ptr(), 96, c.data_ptr(), 64, 2, 128, 64, 96, None, None) == -3  # K % 64
    assert lib.uv_gemm_tc(a.data_ptr(), 64, a.data_ptr(), 64, c.data_ptr(), 64, 1, 128, 64, 64, None, None) != 0  # fp16
