"""The tcgen05/TMEM/TMA dense contraction against a plain fp32/fp64 torch matmul of the same
(16-bit rounded) operands.  Covers both operand layouts the path uses, both 16-bit types, every
output type, the bias epilogue, sizes no tile divides, and both tile shapes: one CTA per 128 x BN
tile, and CTA pairs on 256 x 256 tiles (M >= 256 and N a multiple of 256)."""
import pytest
import torch

from flashlstm_poc_b200 import _lib

pytestmark = pytest.mark.gpu

DT = {"f16": (1, torch.float16), "bf16": (2, torch.bfloat16)}


@pytest.fixture(autouse=True, params=["rule", "pairs"])
def tile_shape(request, monkeypatch):
    """Every case runs twice: with the measured rule choosing the kernel, and with CTA pairs forced wherever the
    shape allows (FLSTM_GEMM_PAIR=2), so the pair kernel is checked on every layout and size."""
    if request.param == "pairs":
        monkeypatch.setenv("FLSTM_GEMM_PAIR", "2")
    else:
        monkeypatch.delenv("FLSTM_GEMM_PAIR", raising=False)


def _gemm(dtype, out, M, N, K, A, B, bias=None, mn=False):
    lib = _lib.load()
    code, td = DT[dtype]
    out_code, out_td = (0, torch.float32) if out == "f32" else DT[out]
    D = torch.full((M, N), float("nan"), dtype=out_td, device="cuda")
    st = lib.flstm_tc_gemm(code, out_code, M, N, K, A.data_ptr(), B.data_ptr(), D.data_ptr(), N,
                           None if bias is None else bias.data_ptr(), 1 if mn else 0,
                           torch.cuda.current_stream().cuda_stream)
    assert st == 0, lib.flstm_last_error()
    return D


def _rel(got, want):
    return float((got.double() - want).norm() / want.norm())


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 256, 128), (256, 512, 256), (384, 128, 1024),
                                   (200, 136, 72), (64, 64, 64), (1000, 520, 200), (4096, 1024, 512),
                                   (1000, 512, 200), (8192, 1024, 192),  # CTA-pair tiles: ragged M, many tiles per pair
                                   (300, 100, 64)])  # N=100: row pitch not a multiple of 16 B -> plain-store epilogue
def test_kmajor_gemm(dtype, M, N, K):
    torch.manual_seed(M + N + K)
    td = DT[dtype][1]
    A = torch.randn(M, K, device="cuda").to(td)
    B = torch.randn(N, K, device="cuda").to(td)
    want = A.double() @ B.double().t()
    got = _gemm(dtype, "f32", M, N, K, A, B)
    assert torch.isfinite(got).all()
    assert _rel(got, want) < 1e-5
    bias = torch.randn(N, device="cuda")
    got16 = _gemm(dtype, dtype, M, N, K, A, B, bias=bias)
    assert _rel(got16, want + bias.double()) < (2e-3 if dtype == "f16" else 1e-2)
    got16 = _gemm(dtype, dtype, M, N, K, A, B)
    assert _rel(got16, want) < (2e-3 if dtype == "f16" else 1e-2)


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 256, 128), (256, 128, 1024), (512, 512, 4096),
                                   (192, 320, 200), (64, 64, 64), (1024, 256, 8192), (4096, 2048, 512), (304, 256, 136)])
def test_mnmajor_gemm(dtype, M, N, K):
    """D = A^T-stored x B^T-stored: A is given as (K,M), B as (K,N); the reduction dim is outermost,
    which is how dG (T*B,4H) and [X|H] (T*B,I) lie in memory for dW = dG^T X."""
    torch.manual_seed(M * 3 + N + K)
    td = DT[dtype][1]
    At = torch.randn(K, M, device="cuda").to(td)
    Bt = torch.randn(K, N, device="cuda").to(td)
    want = At.double().t() @ Bt.double()
    got = _gemm(dtype, "f32", M, N, K, At, Bt, mn=True)
    assert torch.isfinite(got).all()
    assert _rel(got, want) < 1e-5


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (512, 256, 1024), (200, 192, 136), (2048, 1024, 4096)])
def test_mixed_major_gemm(dtype, M, N, K):
    """A K-major, B stored (K,N): the input-gradient form dX = dG W_ih with W_ih read as stored."""
    torch.manual_seed(M + 7 * N + K)
    td = DT[dtype][1]
    A = torch.randn(M, K, device="cuda").to(td)
    Bt = torch.randn(K, N, device="cuda").to(td)
    want = A.double() @ Bt.double()
    lib = _lib.load()
    for out, tol in (("f32", 1e-5), (dtype, 2e-3 if dtype == "f16" else 1e-2)):
        out_code, out_td = (0, torch.float32) if out == "f32" else DT[out]
        D = torch.full((M, N), float("nan"), dtype=out_td, device="cuda")
        st = lib.flstm_tc_gemm(DT[dtype][0], out_code, M, N, K, A.data_ptr(), Bt.data_ptr(), D.data_ptr(), N, None, 2,
                               torch.cuda.current_stream().cuda_stream)
        assert st == 0, lib.flstm_last_error()
        assert _rel(D, want) < tol


def test_gemm_rejects_unaligned():
    lib = _lib.load()
    A = torch.zeros(64, 60, dtype=torch.float16, device="cuda")
    D = torch.zeros(64, 64, device="cuda")
    st = lib.flstm_tc_gemm(1, 0, 64, 64, 60, A.data_ptr(), A.data_ptr(), D.data_ptr(), 64, None, 0, None)
    assert st == 4  # UNSUPPORTED: row pitch is not a multiple of 16 bytes
