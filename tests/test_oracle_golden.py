"""The CPU oracle against golden vectors produced by the reference's own PyTorch emulation
(tests/golden/make_golden.py imports custom_nodes/rapid_h3/kernels.py)."""
import pytest
import torch

from oracle import linear as ol
from oracle import quant as oq


def _codes(t):
    return t.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t


@pytest.mark.parametrize("case", ["a", "b"])
@pytest.mark.parametrize("mode", ["int8_rowwise", "fp8_rowwise"])
def test_quantizers_match_reference(golden_linear, case, mode):
    c = golden_linear[case]
    g = c[mode]
    xq, xs = ol.quantize_rows(c["x"], mode)
    wq, ws = ol.quantize_weight(c["w"], mode)
    assert torch.equal(_codes(xq), g["xq"]) and torch.equal(xs, g["xs"])
    assert torch.equal(_codes(wq), g["wq"]) and torch.equal(ws, g["ws"])


@pytest.mark.parametrize("case", ["a", "b"])
def test_int8_linear_matches_reference(golden_linear, case):
    c = golden_linear[case]
    g = c["int8_rowwise"]
    y = ol.linear(c["x"], g["wq"], g["ws"], "int8_rowwise")
    assert torch.equal(y, g["y"])  # same expression order as kernels.py:137


@pytest.mark.parametrize("case", ["a", "b"])
def test_fp8_linear_matches_reference(golden_linear, case):
    c = golden_linear[case]
    g = c["fp8_rowwise"]
    wq = g["wq"].view(torch.float8_e4m3fn)
    y = ol.linear(c["x"], wq, g["ws"], "fp8_rowwise").float()
    # the reference's _scaled_mm rounds the product to bf16 before the scales are applied
    # (kernels.py:133-137); the fused epilogue keeps fp32, so the two differ by one bf16 rounding
    rel = (y - g["y"].float()).norm() / g["y"].float().norm()
    assert rel < 4e-3


def test_fp8_tensor_mode_matches_reference(golden_tensor):
    # kernels.py:63-65 and :125-128: one scale per tensor. The codes and the scale are the reference's bit for bit;
    # the product goes through a different matrix routine there, so the bf16 outputs agree to rounding only.
    c = golden_tensor
    wq, ws = ol.quantize_weight(c["w"], "fp8_tensor")
    assert torch.equal(_codes(wq), c["wq"])
    assert torch.equal(ws, c["ws"].reshape(1, 1).expand(1, c["w"].shape[0]))
    y = ol.linear(c["x"], wq, ws, "fp8_tensor").float()
    assert (y - c["y"].float()).norm() / c["y"].float().norm() < 4e-3


def test_int_mm_fallback_is_exact():
    g = torch.Generator().manual_seed(1)
    a = torch.randint(-127, 128, (9, 48), generator=g, dtype=torch.int8)
    b = torch.randint(-127, 128, (10, 48), generator=g, dtype=torch.int8)
    assert torch.equal(ol.int_mm(a, b), (a.long() @ b.long().t()).to(torch.int32))
    a = torch.randint(-127, 128, (64, 64), generator=g, dtype=torch.int8)
    b = torch.randint(-127, 128, (32, 64), generator=g, dtype=torch.int8)
    assert torch.equal(ol.int_mm(a, b), (a.long() @ b.long().t()).to(torch.int32))


def test_swiglu_perm_and_epilogue():
    f = 16
    perm = ol.swiglu_perm(2 * f)
    assert perm[:8].tolist() == [0, 1, 2, 3, f, f + 1, f + 2, f + 3]
    g = torch.Generator().manual_seed(2)
    acc = torch.randint(-5000, 5000, (4, 2 * f), generator=g, dtype=torch.int32)
    xs = torch.rand(4, generator=g) * 1e-2
    ws = torch.rand(2 * f, generator=g) * 1e-2
    h = ol.swiglu_epilogue(acc[:, perm], xs, ws[perm]).float()
    y = ol.dequant(acc, xs, ws).float()
    ref = torch.nn.functional.silu(y[:, :f]) * y[:, f:]
    assert torch.allclose(h, ref, rtol=2e-2, atol=1e-6)


def test_fixed_order_sumsq_close_to_plain_sum():
    g = torch.Generator().manual_seed(3)
    for k in (256, 4096, 5376, 16384):
        x = torch.randn(5, k, generator=g)
        a = oq.fixed_order_sumsq(x)
        b = (x.double() ** 2).sum(1)
        assert torch.allclose(a.double(), b, rtol=1e-5)


def test_norm_mod_matches_fp32_expression():
    # the reference's fp32 expression for the fused prologue: bench/rot_test.py:42-51
    g = torch.Generator().manual_seed(4)
    m, k = 33, 512
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(k, generator=g)).to(torch.bfloat16)
    shift = 0.1 * torch.randn(3, k, generator=g)
    scale = 0.1 * torch.randn(3, k, generator=g)
    idx = torch.randint(0, 3, (m,), generator=g, dtype=torch.int32)
    y = oq.norm_mod(x, w, 1e-6, idx, shift, scale)
    xf = x.float()
    ref = xf * torch.rsqrt(xf.pow(2).mean(1, keepdim=True) + 1e-6) * w.float() * (1 + scale[idx.long()]) + shift[idx.long()]
    assert torch.allclose(y, ref, rtol=1e-5, atol=1e-6)
    q, s = oq.norm_mod_quant_rows_i8(x, w, 1e-6, idx, shift, scale)
    assert q.abs().max() == 127 and s.shape == (m, 1)


def test_rotation_butterfly_equals_hadamard_product():
    """The oracle's radix-4 butterflies against the reference's definition of the rotation, x @ blockdiag(H256)^T
    with H256 the Kronecker power of the regular 4x4 Hadamard matrix (triton_fp8.py:70-92), and its orthonormality
    (which is what lets rotated activations meet rotated weights)."""
    from oracle import linear as ol
    g = torch.Generator().manual_seed(3)
    x = torch.randn(7, 768, generator=g)
    y = ol.rotate256(x)
    assert (y.double() - ol.convrot_matmul(x)).abs().max() < 2e-6
    h = ol.regular_hadamard(256)
    assert torch.allclose(h @ h.T, torch.eye(256, dtype=torch.float64), atol=1e-12)
    assert torch.allclose(y.double().norm(dim=1), x.double().norm(dim=1), rtol=1e-6)
    # int8_rot linear == int8 arithmetic on rotated operands, and stays close to the exact product
    w = torch.randn(32, 768, generator=g).to(torch.bfloat16)
    xb = x.to(torch.bfloat16)
    wq, ws = ol.quantize_weight(w, "int8_rot")
    out = ol.linear(xb, wq, ws, "int8_rot").double()
    ref = xb.double() @ w.double().t()
    assert ((out - ref).norm() / ref.norm()).item() < 2e-2


# ---------------------------------------------------------------------------------------------
# fixtures made by the reference's own H256 ConvRot code and its attention emulation script
# ---------------------------------------------------------------------------------------------
import os  # noqa: E402

_GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _code_agreement(q, q0):
    """(fraction of codes that differ, largest difference): the reference's own yardstick, bench/rot_test.py:22-26."""
    d = (q.int() - q0.int()).abs()
    return (d > 0).float().mean().item(), int(d.max())


def test_rotation_matches_the_reference_convrot():
    """H256 itself, the rotated activations, and the rotated int8 codes of activations and weights against what
    triton_fp8.regular_hadamard / convrot and kernels.quantize_weight("int8_rot") of the reference return. The
    reference rotates with a matrix product (summation order unspecified), so codes are held to its own
    criterion: at most one step apart on fewer than 1e-3 of the elements, scales equal to fp32 rounding."""
    g = torch.load(os.path.join(_GOLDEN, "rot_ref.pt"))
    assert torch.equal(ol.regular_hadamard(256).float(), g["h256"])
    r = ol.rotate256(g["x"].float())
    assert (r - g["x_rot"]).abs().max() <= 4e-6 * g["x_rot"].abs().max()
    xq, xs = ol.quantize_rows(g["x"], "int8_rot")
    frac, worst = _code_agreement(xq, g["x_q"])
    assert frac < 1e-3 and worst <= 1
    assert ((xs - g["x_s"]).abs() / g["x_s"]).max() < 1e-6
    wq, ws = ol.quantize_weight(g["w"], "int8_rot")
    frac, worst = _code_agreement(wq, g["w_q"])
    assert frac < 1e-3 and worst <= 1
    assert ((ws - g["w_s"]).abs() / g["w_s"]).max() < 1e-6


def test_attention_operands_match_the_reference_emulation():
    """Block-64 int8 Q and K (K mean-smoothed) and per-channel e4m3 V: codes x scales of the oracle's pre-pass
    equal, bit for bit, the fake-quantized tensors of bench/attn_emulate.py `q8(x, 1, 64)` / `f8(x, 0)` when both
    are given the same channel means."""
    from oracle import attention as oa
    g = torch.load(os.path.join(_GOLDEN, "attn_ref.pt"))
    q, k, v = g["q"], g["k"], g["v"]
    l = q.shape[0]
    kmean, vmean, vscale = oa.kv_stats(k, v)
    assert torch.equal(kmean, g["kmean"]) and torch.equal(vmean, g["vmean"])
    q8, qs = oa.quant_block64(q, pad=256)
    k8, ks = oa.quant_block64(k, kmean)
    vt = oa.quant_v(v, vmean, vscale)
    blk = torch.arange(l) // 64
    for h, ref in enumerate(g["heads"]):
        assert torch.equal(q8[h, :l].float() * qs[h][blk][:, None], ref["q_fq"])
        assert torch.equal(k8[h, :l].float() * ks[h][blk][:, None], ref["k_fq"])
        vdec = vt[h, :, :l].view(torch.float8_e4m3fn).float().t() * vscale[h][None]
        assert torch.equal(vdec, ref["v_fq"])


def test_attention_output_is_bounded_by_the_reference_emulation():
    """The main loop against `attn(..., pmode="run_fp8")` of bench/attn_emulate.py on the same fake-quantized
    operands. The two are not the same arithmetic: the reference scales P to 448 against the final row maximum,
    here P is scaled to 2^8 against the row maximum rounded up to an integer (base 2), so each P lands on a
    different point of the e4m3 grid. What must hold: both sit at the same distance from the exact-P result
    (within 25 %), and they differ from each other by no more than the two rounding errors combined."""
    from oracle import attention as oa
    g = torch.load(os.path.join(_GOLDEN, "attn_ref.pt"))
    out = oa.attention(g["q"], g["k"], g["v"]).float()
    for h, ref in enumerate(g["heads"]):
        exact = ref["out_exact_p"]
        e_ref = ((ref["out_run_fp8"] - exact).norm() / exact.norm()).item()
        e_own = ((out[:, h] - exact).norm() / exact.norm()).item()
        between = ((out[:, h] - ref["out_run_fp8"]).norm() / exact.norm()).item()
        assert e_own <= 1.25 * e_ref + 4e-3      # 4e-3: the bf16 rounding of the output
        assert between <= e_own + e_ref
