"""The allocation-free bias-gradient entry point (for callers that must not allocate device memory
at call time: pre-reserved-memory serving loops, stream captures, embedders with strict memory
accounting) against the regular entry point, which allocates its scratch per call.

Collected last on purpose: a run that stops at the first failure has then already run every other
test.  It passes alone in a fresh process and after the rest of the suite: the shared scratch array
keeps the previous call's contents and needs no clearing, which the back-to-back calls check."""
import pytest
import torch

from flashlstm_poc_b200 import _lib

pytestmark = pytest.mark.gpu


def _run(fn, code, dg, H=0):
    rows, cols = dg.shape
    out = torch.full((cols,), float("nan"), device="cuda")
    st = fn(code, dg.data_ptr(), rows, cols, H, out.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return st, out


def test_static_bias_grad_matches_allocating_entry_point_twice_in_a_row():
    lib = _lib.load()
    torch.manual_seed(0)
    first = torch.randn(4096, 1024, device="cuda").half()
    second = torch.randn(777, 4096, device="cuda").bfloat16()  # wider, other dtype: reuses the scratch as left
    for code, dg in ((1, first), (2, second)):
        st_ref, want = _run(lib.flstm_bias_grad, code, dg)
        st, got = _run(lib.flstm_bias_grad_static, code, dg)
        assert st_ref == 0 and st == 0, lib.flstm_last_error()
        # same kernels, same fixed summation order: identical bits (tighter than the suite's 1e-5 relative bound)
        assert torch.equal(got, want)
        assert torch.allclose(got.double(), dg.double().sum(0), rtol=1e-5, atol=2e-3)
    # the first matrix again: nothing from the wider call leaks into a narrower one
    st, again = _run(lib.flstm_bias_grad_static, 1, first)
    _, want = _run(lib.flstm_bias_grad, 1, first)
    assert st == 0 and torch.equal(again, want)


def test_static_bias_grad_rejects_widths_beyond_its_fixed_scratch():
    lib = _lib.load()
    dg = torch.zeros(2, 16384 + 64, device="cuda", dtype=torch.float16)
    st, _ = _run(lib.flstm_bias_grad_static, 1, dg)
    assert st == 4  # FLSTM_ERR_UNSUPPORTED
    assert b"at most 16384 columns" in lib.flstm_last_error()
    st, out = _run(lib.flstm_bias_grad_static, 1, dg[:, :16384].contiguous())
    assert st == 0 and float(out.abs().max()) == 0.0


def test_static_bias_grad_allocates_nothing_and_runs_inside_a_stream_capture():
    """After one warm call (which looks the scratch array's address up) the entry point leaves the device's free
    memory untouched, and it can be captured into a CUDA graph and replayed -- the use its header names."""
    lib = _lib.load()
    torch.manual_seed(1)
    dg = torch.randn(2048, 2048, device="cuda").half()
    _, want = _run(lib.flstm_bias_grad, 1, dg)
    st, _ = _run(lib.flstm_bias_grad_static, 1, dg)  # warm call
    assert st == 0
    out = torch.zeros(2048, device="cuda")
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(5):
        st = lib.flstm_bias_grad_static(1, dg.data_ptr(), 2048, 2048, 0, out.data_ptr(), torch.cuda.current_stream().cuda_stream)
        assert st == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    assert torch.equal(out, want)

    graph = torch.cuda.CUDAGraph()
    out.zero_()
    with torch.cuda.graph(graph):
        st = lib.flstm_bias_grad_static(1, dg.data_ptr(), 2048, 2048, 0, out.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert st == 0, lib.flstm_last_error()
    for _ in range(2):
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, want)
