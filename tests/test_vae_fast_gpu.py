"""fp16 ops of the VAE transformer decoder (through the C ABI) against the CPU oracle: the head-major ConvRot
quantizer with nan_to_num, the row-major quantizer, the fp16 GEMM epilogues (bias, residual addcmul) and the
w1 + SwiGLU epilogue. Shapes follow the reference's decoder (dims 2048 / 6144 / 8192, D = 64; M a few thousand)."""
import pytest
import torch

from oracle import inputs
from oracle import vae_ops as ov

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def vf():
    from rapid_h3_b200 import _lib, vae_fast
    assert torch.cuda.is_available()
    _lib.lib()
    return vae_fast, _lib


@pytest.mark.parametrize("shape", [(1, 32, 1797, 64), (2, 4, 300, 64), (1, 8, 5, 32), (1, 128, 33, 64)])
def test_vae_out_quant_bit_exact(vf, shape):
    vae_fast, lib = vf
    g = inputs.gen(sum(shape))
    o = (torch.randn(shape, generator=g) * (1 + 3 * torch.rand(shape[0], shape[1], 1, 1, generator=g))).half()
    o[0, 0, 0, :4] = torch.tensor([float("nan"), float("inf"), float("-inf"), 65504.0]).half()
    if shape[2] > 2:
        o[:, :, 2] = 0  # an all-zero row: scale floor
    q, s = vae_fast.vae_out_quant(o.cuda())
    lib.check_status()
    qr, sr = ov.vae_out_quant(o)
    assert torch.equal(s.cpu(), sr)
    assert torch.equal(q.cpu(), qr)


@pytest.mark.parametrize("shape", [(1000, 2048), (77, 8192), (5, 256)])
def test_vae_quant_rows_bit_exact(vf, shape):
    vae_fast, lib = vf
    g = inputs.gen(shape[0])
    x = torch.randn(shape, generator=g).half()
    x[:, 7] *= 30.0
    q, s = vae_fast._quantize(x.cuda())
    lib.check_status()
    qr, sr = ov.quant_rows_f16(x)
    assert torch.equal(s.cpu().reshape(-1), sr) and torch.equal(q.cpu(), qr)
    with pytest.raises(RuntimeError):
        vae_fast._quantize(x.cuda()[:, :128])  # width must be whole groups of 256
    with pytest.raises(RuntimeError):
        vae_fast._quantize(x)  # CPU tensor: no CPU path


def _gemm_case(m, n, k, seed):
    g = inputs.gen(seed)
    xq = torch.randint(-127, 128, (m, k), generator=g, dtype=torch.int8)
    wq = torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8)
    xs = (0.01 + 0.02 * torch.rand(m, generator=g)).float()
    ws = (0.5 + torch.rand(n, generator=g)).float() * 1e-3
    bias = (0.1 * torch.randn(n, generator=g)).half()
    return xq, wq, xs, ws, bias, g


@pytest.mark.parametrize("shape", [(1797, 2048, 2048), (300, 6144, 2048), (130, 2048, 8192), (64, 264, 256)])
@pytest.mark.parametrize("residual", [False, True])
def test_vae_gemm_bit_exact(vf, shape, residual):
    vae_fast, lib = vf
    m, n, k = shape
    xq, wq, xs, ws, bias, g = _gemm_case(m, n, k, m + n)
    rs = resid = None
    if residual:
        rs = (1 + 0.1 * torch.randn(n, generator=g)).half()
        resid = torch.randn(m, n, generator=g).half()
    out = vae_fast.vae_gemm(xq.cuda(), wq.cuda(), xs.cuda(), ws.cuda(), bias.cuda(),
                            None if rs is None else rs.cuda(), None if resid is None else resid.cuda())
    lib.check_status()
    ref = ov.vae_gemm(xq, wq, xs, ws, bias, rs, resid)
    assert torch.equal(out.cpu(), ref)


def test_vae_gemm_swiglu_close(vf):
    vae_fast, lib = vf
    m, n, k = 700, 4096, 2048
    xq, wq, xs, ws, bias, g = _gemm_case(m, n, k, 3)
    wq_p, ws_p, bias_p = (vae_fast._interleave_rows(t, n) for t in (wq, ws, bias))
    assert torch.equal(wq_p, ov.interleave_rows(wq, n))
    out = vae_fast.vae_gemm_swiglu(xq.cuda(), wq_p.contiguous().cuda(), xs.cuda(), ws_p.contiguous().cuda(),
                                   bias_p.contiguous().cuda())
    lib.check_status()
    ref = ov.vae_gemm_swiglu(xq, wq_p, xs, ws_p, bias_p)
    # the epilogue's e^-g is the hardware approximation: fp16 results may differ in the last place
    d = (out.cpu().float() - ref.float()).abs()
    assert (d <= 2e-3 * ref.float().abs() + 1e-6).all()
    assert (out.cpu() != ref).float().mean() < 0.02
    # equals the unfused path: plain GEMM on the original row order, SwiGLU afterwards
    y = ov.vae_gemm(xq, wq, xs, ws, bias).float()
    gate, up = y[:, : n // 2], y[:, n // 2:]
    unfused = ((gate / (1 + torch.exp(-gate))) * up).half()
    assert torch.equal(unfused, ref)


def test_vae_linear_end_to_end(vf):
    """x W^T + b through rotated quantizer and rotated int8 weight stays close to the fp32 product."""
    vae_fast, lib = vf
    from oracle import linear as ol
    g = inputs.gen(9)
    m, k, n = 512, 2048, 2048
    x = torch.randn(m, k, generator=g).half()
    w = (torch.randn(n, k, generator=g) / k ** 0.5).half()
    b = (0.1 * torch.randn(n, generator=g)).half()
    wr = ov.fht256(w.float())                       # weight stored as W . blockdiag(H256)^T
    ws = wr.abs().amax(dim=1) / 127.0
    wq = (wr / ws[:, None]).round().clamp(-127, 127).to(torch.int8)
    resid = torch.randn(m, n, generator=g).half()
    rs = torch.ones(n).half()
    y = vae_fast._linear(wq.cuda(), ws.cuda(), b.cuda(), x.cuda(), residual=resid.cuda(), residual_scale=rs.cuda())
    lib.check_status()
    ref = x.double() @ w.double().t() + b.double() + resid.double()
    assert ((y.cpu().double() - ref).norm() / ref.norm()).item() < 2e-2
    xq, xs = ov.quant_rows_f16(x)
    assert torch.equal(y.cpu(), ov.vae_gemm(xq, wq, xs, ws, b, rs, resid))
    del ol


@pytest.mark.parametrize("shape", [(1000, 2048), (77, 8192), (5, 256)])
@pytest.mark.parametrize("with_weight", [True, False])
def test_vae_quantizer_rms_norm_prologue(vf, shape, with_weight):
    """`act="rms_norm"`: the quantizer of the inputs of to_qkv and w1. Scales bit-exact, codes bit-exact (every
    operation of the prologue is an IEEE operation in a fixed order)."""
    vae_fast, lib = vf
    g = inputs.gen(shape[0] + 1)
    x = (torch.randn(shape, generator=g) * (0.5 + torch.rand(shape[0], 1, generator=g))).half()
    x[:, 5] *= 25.0
    if shape[0] > 3:
        x[3] = 0
    w = (1 + 0.2 * torch.randn(shape[1], generator=g)).half() if with_weight else None
    q, s = vae_fast._quantize(x.cuda(), "rms_norm", None if w is None else w.cuda(), 1e-6)
    lib.check_status()
    qr, sr = ov.quant_rows_f16(x, "rms_norm", w, 1e-6)
    assert torch.equal(s.cpu().reshape(-1), sr) and torch.equal(q.cpu(), qr)


@pytest.mark.parametrize("shape", [(700, 2048), (33, 4096)])
def test_vae_quantizer_swiglu_prologue(vf, shape):
    """`act="swiglu"`: x = [gate | up]. The device's expf may differ from the CPU's in the last place, so codes are
    held to the reference's own criterion for fused quantizers (at most one step apart on < 1e-3 of the elements,
    bench/rot_test.py:36-40) and scales to 1e-6."""
    vae_fast, lib = vf
    m, k = shape
    x = torch.randn(m, 2 * k, generator=inputs.gen(m)).half()
    q, s = vae_fast._quantize(x.cuda(), "swiglu")
    lib.check_status()
    qr, sr = ov.quant_rows_f16(x, "swiglu")
    assert q.shape == (m, k)
    assert torch.allclose(s.cpu().reshape(-1), sr, rtol=1e-6, atol=0)
    d = (q.cpu().int() - qr.int()).abs()
    assert d.max() <= 1 and (d != 0).float().mean() < 1e-3


@pytest.mark.parametrize("epilogue", [True, False])
def test_vae_ff_forward(vf, epilogue):
    """The decoder's feed-forward block (rms_norm -> w1 -> SwiGLU -> w2 -> * residual_scale + residual) on its two
    routes: SwiGLU in w1's epilogue, or as the prologue of w2's quantizer. Decoder shapes: dim 2048, hidden 8192."""
    vae_fast, lib = vf
    g = inputs.gen(21)
    m, k, f = 600, 2048, 8192

    def rotated_weight(n, kk):
        w = (torch.randn(n, kk, generator=g) / kk ** 0.5).half()
        wr = ov.fht256(w.float())
        ws = wr.abs().amax(dim=1) / 127.0
        return w, (wr / ws[:, None]).round().clamp(-127, 127).to(torch.int8), ws

    w1, w1q, w1s = rotated_weight(2 * f, k)
    w2, w2q, w2s = rotated_weight(k, f)
    b1, b2 = (0.05 * torch.randn(2 * f, generator=g)).half(), (0.05 * torch.randn(k, generator=g)).half()
    x = torch.randn(m, k, generator=g).half()
    nw = (1 + 0.1 * torch.randn(k, generator=g)).half()
    resid, rs = torch.randn(m, k, generator=g).half(), (1 + 0.1 * torch.randn(k, generator=g)).half()
    l1 = vae_fast.Int8Linear(w1q.cuda(), w1s.cuda(), b1.cuda())
    l2 = vae_fast.Int8Linear(w2q.cuda(), w2s.cuda(), b2.cuda())
    vae_fast.install_swiglu(epilogue)
    try:
        y = vae_fast._ff_forward(l1, l2, x.cuda().view(2, m // 2, k), nw.cuda(), 1e-6, resid.cuda().view(2, m // 2, k), rs.cuda())
    finally:
        vae_fast.install_swiglu(True)
    lib.check_status()
    assert y.shape == (2, m // 2, k) and y.dtype == torch.float16
    ref = ov.ff_forward(x, nw, 1e-6, w1q, w1s, b1, w2q, w2s, b2, resid, rs, swiglu_epilogue=epilogue)
    rel = ((y.cpu().reshape(m, k).float() - ref.float()).norm() / ref.float().norm()).item()
    assert rel < 1e-3          # the SwiGLU exponential is the only inexact step between the two sides
    # and the quantized block stays close to the fp32 block
    xn = x.float() * torch.rsqrt(x.float().pow(2).mean(1, keepdim=True) + 1e-6) * nw.float()
    hh = xn @ w1.float().t() + b1.float()
    hh = torch.nn.functional.silu(hh[:, :f]) * hh[:, f:]
    full = (hh @ w2.float().t() + b2.float()) * rs.float() + resid.float()
    assert ((y.cpu().reshape(m, k).float() - full).norm() / full.norm()).item() < 2e-2
