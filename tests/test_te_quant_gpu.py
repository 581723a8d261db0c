"""The text encoder's int8_rot linear with its outlier-row residual pass against the CPU oracle."""
import pytest
import torch

from oracle import inputs
from oracle import linear as ol
from oracle import quant as oq

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def te():
    from rapid_h3_b200 import _lib, kernels, te_quant
    assert torch.cuda.is_available()
    _lib.lib()
    return te_quant, kernels, _lib


def _case(m, k, n, seed):
    g = inputs.gen(seed)
    x = torch.randn(m, k, generator=g)
    # every 7th row carries a pattern that the rotation concentrates into ONE channel (a row of H256 itself):
    # these are the rows whose rotated abs-max towers over their rms, the ones the residual pass exists for
    x[::7, 256:512] += 6.0 * (ol.regular_hadamard(256)[5] * 16.0).float()
    w = (torch.randn(n, k, generator=g) / k ** 0.5).to(torch.bfloat16)
    return x, w


def test_residual_quantizer_bit_exact(te):
    te_quant, kernels, lib = te
    x, _ = _case(300, 1024, 8, 1)
    q1, s1 = oq.rot_quant_rows_i8(x.to(torch.bfloat16))
    rows = torch.tensor([0, 7, 14, 299, 5], dtype=torch.int64)
    q2, s2 = te_quant.rot_residual_quant_rows_i8(x.cuda(), q1.cuda(), s1.cuda(), rows.cuda())
    lib.check_status()
    q2r, s2r = oq.rot_residual_quant_rows_i8(x, q1, s1, rows)
    assert torch.equal(s2.cpu(), s2r) and torch.equal(q2.cpu(), q2r)


@pytest.mark.parametrize("mode", ["int8_rot", "int8_rot_plain"])
def test_te_linear_matches_oracle_and_helps_outlier_rows(te, mode):
    te_quant, kernels, lib = te
    m, k, n = 400, 2048, 512
    x, w = _case(m, k, n, 2)
    b = 0.1 * torch.randn(n, generator=inputs.gen(3))
    qw = kernels.quantize_weight(w.cuda(), "int8_rot")
    lin = te_quant._TELinear(qw, b.cuda(), mode, outlier_ratio=8.0)
    y = lin(x.cuda().reshape(4, 100, k))
    lib.check_status()
    assert y.shape == (4, 100, n) and y.dtype == torch.float32
    # oracle: the same two passes on CPU
    wq, ws = ol.quantize_weight(w, "int8_rot")
    q1, s1 = oq.rot_quant_rows_i8(x.to(torch.bfloat16))
    yr = ol.dequant(ol.int_mm(q1, wq), s1, ws).float()
    n_out = 0
    if mode == "int8_rot":
        ratio = 127.0 * s1[:, 0] / x.pow(2).mean(-1).sqrt().clamp_min(1e-12)
        rows = (ratio > 8.0).nonzero()[:, 0]
        n_out = rows.numel()
        assert 0 < n_out < m // 2
        q2, s2 = oq.rot_residual_quant_rows_i8(x, q1, s1, rows)
        yr[rows] += ol.dequant(ol.int_mm(q2, wq), s2, ws).float()
    yr = yr + b
    assert torch.allclose(y.cpu().reshape(m, n), yr, rtol=0, atol=1e-5 * yr.abs().max().item())
    ref = x.double() @ w.double().t() + b.double()
    err = ((y.cpu().reshape(m, n).double() - ref).norm(dim=1) / ref.norm(dim=1))
    print(mode, "rows with residual pass:", n_out, "median / max row error:", err.median().item(), err.max().item())
    if mode == "int8_rot":
        assert err.max().item() < 0.02
