"""Stand-alone bias-gradient reduction (db = column sums of dG) against a float64 torch sum."""
import pytest
import torch

from flashlstm_poc_b200 import _lib

pytestmark = pytest.mark.gpu

DT = {"f32": (0, torch.float32), "f16": (1, torch.float16), "bf16": (2, torch.bfloat16)}


def interleave_columns(x, H):
    """torch gate order (g*H+u) -> tile-interleaved order ((u/16)*4+g)*16 + u%16."""
    R = x.shape[0]
    return x.view(R, 4, H // 16, 16).permute(0, 2, 1, 3).reshape(R, 4 * H).contiguous()


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("rows,cols", [(1, 64), (37, 40), (4096, 1024), (32768, 4096), (5, 3)])
def test_bias_grad_matches_torch(dtype, rows, cols):
    lib = _lib.load()
    code, td = DT[dtype]
    torch.manual_seed(rows + cols)
    dg = torch.randn(rows, cols, device="cuda").to(td)
    db = torch.full((cols,), float("nan"), device="cuda")
    assert lib.flstm_bias_grad(code, dg.data_ptr(), rows, cols, 0, db.data_ptr(), None) == 0, lib.flstm_last_error()
    want = dg.double().sum(0)
    assert torch.allclose(db.double(), want, rtol=1e-5, atol=1e-3 * max(1.0, rows ** 0.5) * 1e-2)
    again = torch.empty_like(db)
    assert lib.flstm_bias_grad(code, dg.data_ptr(), rows, cols, 0, again.data_ptr(), None) == 0
    assert torch.equal(db, again)  # fixed summation order


def test_bias_grad_interleaved_order():
    lib = _lib.load()
    H, rows = 128, 300
    dg = torch.randn(rows, 4 * H, device="cuda").half()
    db = torch.empty(4 * H, device="cuda")
    assert lib.flstm_bias_grad(1, interleave_columns(dg, H).data_ptr(), rows, 4 * H, H, db.data_ptr(), None) == 0
    assert torch.allclose(db.double(), dg.double().sum(0), rtol=1e-5, atol=1e-4)
    assert lib.flstm_bias_grad(1, dg.data_ptr(), rows, 4 * H, H + 16, db.data_ptr(), None) == 1  # H must be cols/4
