"""Parity of the row quantizer kernels (through the C ABI) with the CPU oracle: bit-exact codes
and scales."""
import pytest
import torch

from oracle import inputs
from oracle import linear as ol
from oracle import quant as oq

pytestmark = pytest.mark.gpu


def _u8(t):
    return t.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t


@pytest.fixture(scope="module")
def ops():
    from rapid_h3_b200 import _lib, kernels, quantizers
    assert torch.cuda.is_available()
    _lib.lib()
    return quantizers, kernels, _lib


@pytest.mark.parametrize("shape", [(4096, 4096), (257, 5376), (64, 16384), (3, 8), (33, 1032), (5, 32768), (2, 65536)])
@pytest.mark.parametrize("mode", ["int8_rowwise", "fp8_rowwise"])
def test_quantize_rows_bit_exact(ops, shape, mode):
    tq, kernels, lib = ops
    m, k = shape
    x, _, _ = inputs.linear_case(m, k, 8, seed=m + k)
    if m > 2:
        x[1] = 0
    q, s = kernels.quantize_rows(x.cuda(), mode)
    lib.check_status()
    qr, sr = ol.quantize_rows(x, mode)
    assert torch.equal(s.cpu(), sr)
    assert torch.equal(_u8(q.cpu()), _u8(qr))


@pytest.mark.parametrize("case", ["a", "b"])
@pytest.mark.parametrize("mode", ["int8_rowwise", "fp8_rowwise"])
def test_quantizers_match_reference_golden(ops, golden_linear, case, mode):
    tq, kernels, lib = ops
    c = golden_linear[case]
    g = c[mode]
    q, s = kernels.quantize_rows(c["x"].cuda(), mode)
    qw = kernels.quantize_weight(c["w"].cuda(), mode)
    assert torch.equal(_u8(q.cpu()), g["xq"]) and torch.equal(s.cpu(), g["xs"])
    assert torch.equal(_u8(qw.q.cpu()), g["wq"]) and torch.equal(qw.scale.cpu(), g["ws"])


def test_strided_rows_and_empty(ops):
    tq, kernels, lib = ops
    x, _, _ = inputs.linear_case(100, 1024, 8, seed=5)
    xd = x.cuda()
    q, s = tq.quant_rows_i8(xd[:, 256:768])
    qr, sr = ol.quantize_rows(x[:, 256:768], "int8_rowwise")
    assert torch.equal(q.cpu(), qr) and torch.equal(s.cpu(), sr)
    q, s = tq.quant_rows_i8(xd[:0])
    assert q.shape == (0, 1024) and s.shape == (0, 1)
    with pytest.raises(RuntimeError):
        tq.quant_rows_i8(xd.float())
    with pytest.raises(RuntimeError):
        tq.quant_rows_i8(x)  # CPU tensor: no CPU path


@pytest.mark.parametrize("shape", [(1000, 4096), (77, 5376), (19, 16384), (40, 256)])
@pytest.mark.parametrize("has_w", [True, False])
def test_norm_mod_quant_bit_exact(ops, shape, has_w):
    tq, kernels, lib = ops
    m, k = shape
    g = inputs.gen(m)
    x = (torch.randn(m, k, generator=g) * (1 + torch.rand(m, 1, generator=g))).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(k, generator=g)).to(torch.bfloat16) if has_w else None
    tab = 0.1 * torch.randn(3, 6 * k, generator=g)
    shift, scale = tab[:, k:2 * k], tab[:, 3 * k:4 * k]
    idx = torch.randint(0, 3, (m,), generator=g, dtype=torch.int32)
    tabd = tab.cuda()
    q, s = tq.norm_mod_rot_quant_rows_i8(x.cuda(), None if w is None else w.cuda(), 1e-6, idx.cuda(),
                                         tabd[:, k:2 * k], tabd[:, 3 * k:4 * k])
    lib.check_status()
    qr, sr = oq.norm_mod_quant_rows_i8(x, w, 1e-6, idx, shift, scale)
    assert torch.equal(s.cpu(), sr)
    assert torch.equal(q.cpu(), qr)


def test_quant_heads_matches_transpose_then_rows(ops):
    # reference check: bench/fusion_test.py:21-36 (head-major read == transpose + row quantizer)
    tq, kernels, lib = ops
    g = inputs.gen(11)
    h, m = 32, 517
    o = torch.randn(h, m, 128, generator=g).to(torch.bfloat16)
    q, s = tq.rot_quant_heads_i8(o.cuda())
    qr, sr = oq.quant_heads_i8(o)
    assert torch.equal(q.cpu(), qr) and torch.equal(s.cpu(), sr)
    q2, s2 = tq.quant_rows_i8(o.cuda().permute(1, 0, 2).reshape(m, h * 128).contiguous())
    assert torch.equal(q, q2) and torch.equal(s, s2)


def test_swiglu_quant_close(ops):
    # silu uses exp: codes may differ by one step on a small fraction (reference: bench/rot_test.py:36-40)
    tq, kernels, lib = ops
    g = inputs.gen(12)
    m, f = 300, 2048
    x = torch.randn(m, 2 * f, generator=g).to(torch.bfloat16)
    q, s = tq.swiglu_rot_quant_rows_i8(x.cuda())
    qr, sr = oq.swiglu_quant_rows_i8(x)
    assert torch.allclose(s.cpu(), sr, rtol=1e-5)
    d = (q.cpu().int() - qr.int()).abs()
    assert d.max() <= 1 and (d > 0).float().mean() < 1e-3


def test_rotation_is_refused(ops):
    tq, kernels, lib = ops
    x = torch.zeros(4, 256, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(NotImplementedError):
        tq.rot_quant_rows_i8(x, rotate=True)
    with pytest.raises(NotImplementedError):
        kernels.quantize_weight(x, "int8_rot")
    with pytest.raises(ValueError):
        kernels.quantize_weight(x, "no_such_mode")
