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
                                         tabd[:, k:2 * k], tabd[:, 3 * k:4 * k], rotate=False)
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
    q, s = tq.rot_quant_heads_i8(o.cuda(), rotate=False)
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
    q, s = tq.swiglu_rot_quant_rows_i8(x.cuda(), rotate=False)
    qr, sr = oq.swiglu_quant_rows_i8(x)
    assert torch.allclose(s.cpu(), sr, rtol=1e-5)
    d = (q.cpu().int() - qr.int()).abs()
    assert d.max() <= 1 and (d > 0).float().mean() < 1e-3


def test_unknown_and_emulated_modes_raise(ops):
    tq, kernels, lib = ops
    x = torch.zeros(4, 256, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(NotImplementedError):
        kernels.quantize_weight(x, "nvfp4_fake")
    with pytest.raises(ValueError):
        kernels.quantize_weight(x, "no_such_mode")
    with pytest.raises(RuntimeError):  # the rotated width must be whole groups of 256 channels
        tq.rot_quant_rows_i8(torch.zeros(4, 384, dtype=torch.bfloat16, device="cuda"))


# ---- H256 ConvRot rotation (the `int8_rot` recipe) ------------------------------------------------------

@pytest.mark.parametrize("shape", [(4096, 4096), (257, 5376 - 256), (64, 16384), (3, 256), (33, 1024), (5, 32768),
                                   (2, 65536)])
def test_rot_quant_rows_bit_exact(ops, shape):
    tq, kernels, lib = ops
    m, k = shape
    x, _, _ = inputs.linear_case(m, k, 8, seed=m + k)
    if m > 2:
        x[1] = 0
    q, s = tq.rot_quant_rows_i8(x.cuda())
    lib.check_status()
    qr, sr = oq.rot_quant_rows_i8(x)
    assert torch.equal(s.cpu(), sr)
    assert torch.equal(q.cpu(), qr)
    q2, s2 = kernels.quantize_rows(x.cuda(), "int8_rot")
    assert torch.equal(q2, q) and torch.equal(s2, s)


def test_rot_quant_matches_matrix_product(ops):
    # the reference's own check (bench/rot_test.py:42-51): codes of the fused kernel against int8 of the
    # rotation written as one matrix product; they may differ by one step where the two roundings straddle .5
    tq, kernels, lib = ops
    x, _, _ = inputs.linear_case(512, 4096, 8, seed=21)
    q, s = tq.rot_quant_rows_i8(x.cuda())
    y = oq.convrot_matmul(x.float())
    sr = (y.abs().amax(dim=1, keepdim=True) / 127.0).clamp_min(1e-12)
    qr = (y / sr).round().clamp(-127, 127)
    assert torch.allclose(s.cpu().double(), sr, rtol=1e-6)
    d = (q.cpu().double() - qr).abs()
    assert d.max() <= 1 and (d > 0).double().mean() < 1e-3


@pytest.mark.parametrize("shape", [(1000, 4096), (77, 5376 - 256), (19, 16384), (40, 256)])
@pytest.mark.parametrize("has_w", [True, False])
def test_norm_mod_rot_quant_bit_exact(ops, shape, has_w):
    tq, kernels, lib = ops
    m, k = shape
    g = inputs.gen(m + 1)
    x = (torch.randn(m, k, generator=g) * (1 + torch.rand(m, 1, generator=g))).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(k, generator=g)).to(torch.bfloat16) if has_w else None
    tab = 0.1 * torch.randn(3, 6 * k, generator=g)
    shift, scale = tab[:, k:2 * k], tab[:, 3 * k:4 * k]
    idx = torch.randint(0, 3, (m,), generator=g, dtype=torch.int32)
    tabd = tab.cuda()
    q, s = tq.norm_mod_rot_quant_rows_i8(x.cuda(), None if w is None else w.cuda(), 1e-6, idx.cuda(),
                                         tabd[:, k:2 * k], tabd[:, 3 * k:4 * k])
    lib.check_status()
    qr, sr = oq.norm_mod_rot_quant_rows_i8(x, w, 1e-6, idx, shift, scale)
    assert torch.equal(s.cpu(), sr)
    assert torch.equal(q.cpu(), qr)


def test_rot_quant_heads_and_groups(ops):
    tq, kernels, lib = ops
    g = inputs.gen(13)
    h, m = 32, 517
    o = torch.randn(h, m, 128, generator=g).to(torch.bfloat16)
    q, s = tq.rot_quant_heads_i8(o.cuda())
    qr, sr = oq.rot_quant_heads_i8(o)
    assert torch.equal(q.cpu(), qr) and torch.equal(s.cpu(), sr)
    q2, s2 = tq.rot_quant_rows_i8(o.cuda().permute(1, 0, 2).reshape(m, h * 128).contiguous())
    assert torch.equal(q, q2) and torch.equal(s, s2)
    og = torch.randn(2, 100, 2048, generator=g).to(torch.bfloat16)  # two rank groups of 16 heads
    q, s = tq.quant_groups_i8(og.cuda(), rotate=True)
    qr, sr = oq.rot_quant_rows_i8(og.permute(1, 0, 2).reshape(100, 4096))
    assert torch.equal(q.cpu(), qr) and torch.equal(s.cpu(), sr)


def test_swiglu_rot_quant_close(ops):
    tq, kernels, lib = ops
    g = inputs.gen(14)
    m, f = 300, 2048
    x = torch.randn(m, 2 * f, generator=g).to(torch.bfloat16)
    q, s = tq.swiglu_rot_quant_rows_i8(x.cuda())
    qr, sr = oq.swiglu_rot_quant_rows_i8(x)
    assert torch.allclose(s.cpu(), sr, rtol=1e-5)
    d = (q.cpu().int() - qr.int()).abs()
    assert d.max() <= 1 and (d > 0).float().mean() < 2e-3


def test_int8_rot_linear_beats_rowwise_on_outliers(ops):
    """The point of the rotation: a few huge channels no longer set the scale of the whole row. x W^T through
    `int8_rot` must match the exact int8 arithmetic of the oracle and be closer to fp32 than `int8_rowwise`."""
    tq, kernels, lib = ops
    g = inputs.gen(15)
    m, k, n = 256, 1024, 512
    x = torch.randn(m, k, generator=g)
    x[:, ::97] *= 60.0
    x = x.to(torch.bfloat16)
    w = (torch.randn(n, k, generator=g) / k ** 0.5).to(torch.bfloat16)
    ref = x.double() @ w.double().t()
    err = {}
    for mode in ("int8_rowwise", "int8_rot"):
        qw = kernels.quantize_weight(w.cuda(), mode)
        y = kernels.linear(x.cuda(), qw, mode)
        lib.check_status()
        wq, ws = ol.quantize_weight(w, mode)
        assert torch.equal(qw.q.cpu(), wq) and torch.equal(qw.scale.cpu(), ws)
        yr = ol.linear(x, wq, ws, mode)
        assert torch.equal(y.cpu(), yr)
        err[mode] = ((y.cpu().double() - ref).norm() / ref.norm()).item()
    assert err["int8_rot"] < 0.5 * err["int8_rowwise"], err


def test_rotated_codes_match_the_reference_convrot_fixture(ops):
    """The CUDA H256 rotation + int8 row quantizer against what the reference's own `triton_fp8.convrot` and
    `kernels.quantize_weight(w, "int8_rot")` produced on CPU (tests/golden/rot_ref.pt): its own criterion, at most
    one step apart on fewer than 1e-3 of the codes, scales equal to fp32 rounding."""
    import os
    from rapid_h3_b200 import kernels, quantizers
    g = torch.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "rot_ref.pt"))
    for got, want_q, want_s in ((quantizers.rot_quant_rows_i8(g["x"].cuda()), g["x_q"], g["x_s"]),
                                (kernels.quantize_weight(g["w"].cuda(), "int8_rot"), g["w_q"], g["w_s"])):
        q, s = (got.q, got.scale) if hasattr(got, "q") else got
        d = (q.cpu().int() - want_q.int()).abs()
        assert (d > 0).float().mean().item() < 1e-3 and int(d.max()) <= 1
        assert ((s.cpu().reshape(-1) - want_s.reshape(-1)).abs() / want_s.reshape(-1)).max() < 1e-6
