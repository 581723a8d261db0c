"""Parity of the token-scaled INT8 attention (per-token Q/K after the 128-point Hadamard rotation, int8 V, u8 P
against each key tile's own maximum, per-tile fold: the numerics of the reference's production attention,
custom_nodes/rapid_h3/csrc/README.md "What it computes") with the CPU oracle: operands bit-exact, bf16 output
within rel-L2 1e-3 of the emulation of the same quantized op, and the error against fp32 attention in the range
the reference reports for this numerics class (0.8-1.0 %, docs of bench/results/attn_custom_56h.json)."""
import pytest
import torch

from oracle import attention as oa
from oracle import attention_tok as ot
from oracle import inputs

pytestmark = pytest.mark.gpu
TOL = 1e-3


def rel_l2(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm().clamp_min(1e-20)).item()


@pytest.fixture(scope="module")
def ops():
    from rapid_h3_b200 import _lib, attn_int8
    assert torch.cuda.is_available()
    return attn_int8, _lib


def qkv_buffer(s, h, seed=0):
    g = inputs.gen(seed)
    x = torch.randn(s, 3, h, 128, generator=g)
    chs = torch.exp(0.8 * torch.randn(1, 3, h, 128, generator=g))
    off = torch.zeros(1, 3, h, 128)
    off[:, 1] = 2.0 * torch.randn(1, h, 128, generator=g)
    return (x * chs + off).reshape(s, 3 * h * 128).to(torch.bfloat16)


def views(buf, h):
    s = buf.shape[0]
    q, k, v = buf.split(h * 128, dim=-1)
    return q.view(s, h, 128), k.view(s, h, 128), v.view(s, h, 128)


def assert_operands(pre, ref):
    for name in ("kmean", "vmean", "vscale", "qs", "q8", "k8", "vt"):
        assert torch.equal(getattr(pre, name).cpu(), ref[name]), name
    # -inf == -inf under torch.equal; the multipliers of padding keys are zero on both sides
    assert torch.equal(pre.ksb.cpu(), ref["ksb"])


def test_hadamard_is_its_own_inverse_up_to_128():
    x = torch.randn(5, 3, 128, generator=inputs.gen(4)).to(torch.bfloat16)
    y = ot.hadamard128(x)
    assert torch.allclose(ot.hadamard128(y) / 128.0, x.float(), atol=1e-4)
    h = ot.hadamard128(torch.eye(128))
    assert torch.equal(h.abs(), torch.ones(128, 128)) and torch.equal(h @ h.t(), 128.0 * torch.eye(128))


@pytest.mark.parametrize("s", [1000, 4096, 64, 129])
def test_token_prepass_operands_bit_exact(ops, s):
    attn, lib = ops
    h = 4
    buf = qkv_buffer(s, h, seed=s + 1)
    q, k, v = views(buf, h)
    pre = attn.tok_prepass(*views(buf.cuda(), h))
    lib.check_status()
    assert_operands(pre, ot.prepass(q, k, v))


@pytest.mark.parametrize("shape", [(128, 128), (1000, 1000), (4096, 4096), (777, 512), (200, 64), (64, 1300)])
def test_token_attention_matches_oracle(ops, shape):
    attn, lib = ops
    lq, lk = shape
    h = 3
    q, _, _ = inputs.attention_case(lq, h, seed=lq)
    _, k, v = inputs.attention_case(lk, h, seed=lk + 7)
    pre = attn.tok_prepass(q.cuda(), k.cuda(), v.cuda())
    out = attn.attention_tok_pre(pre)
    lib.check_status()
    ref_pre = ot.prepass(q, k, v)
    assert_operands(pre, ref_pre)
    ref = ot.attention_pre(ref_pre)
    assert rel_l2(out.cpu(), ref) <= TOL
    # 8-bit P against the tile maximum and per-token scales: several times closer to fp32 attention than the
    # e4m3-P kernel (about 0.04 on the same inputs)
    full = oa.attention_fp32(q, k, v)
    assert rel_l2(out.cpu(), full) < 0.02
    assert torch.equal(attn.attention(q.cuda(), k.cuda(), v.cuda(), rotate=True), out)


def test_token_attention_rr_and_strided_output(ops):
    attn, lib = ops
    s, h = 1500, 4
    buf = qkv_buffer(s, h, seed=3)
    q, k, v = views(buf, h)
    tab = inputs.rope_table(inputs.random_positions(s, seed=2))
    qw, kw = inputs.norm_weights()
    bd = buf.cuda()
    qd, kd, vd = views(bd, h)
    o = torch.zeros(1, h, s, 128, dtype=torch.bfloat16, device="cuda")
    raw_q = qd.clone()
    attn.attention_rr(qd, kd, vd, tab.cuda(), qw.cuda(), kw.cuda(), 1e-5, out=o[0].transpose(0, 1), k_roped=kd, rotate=True)
    lib.check_status()
    qn, kn = oa.rmsnorm_rope(q, qw, 1e-5, tab), oa.rmsnorm_rope(k, kw, 1e-5, tab)
    assert torch.equal(qd, raw_q) and torch.equal(kd.cpu(), kn)       # q untouched, k normalised in place
    ref = ot.attention(qn, kn, v)
    assert rel_l2(o[0].transpose(0, 1).cpu(), ref) <= TOL
    # the reference's own check of this fusion (bench/rmsrope_fuse.py:87-115): RMSNorm + RoPE as a separate pass, then
    # the plain call, gives the same bits as the fused pre-pass, operand by operand and in the output
    b2 = buf.cuda()
    q2, k2, v2 = views(b2, h)
    qc = attn.rms_rope(q2, qw.cuda(), 1e-5, tab.cuda())
    kc = attn.rms_rope(k2, kw.cuda(), 1e-5, tab.cuda())
    plain = attn.tok_prepass(qc, kc, v2)
    fused = attn.tok_prepass(q2, k2, v2, tab.cuda(), qw.cuda(), kw.cuda(), 1e-5)
    for name in ("q8", "qs", "k8", "ksb", "vt", "vscale", "vmean", "kmean"):
        assert torch.equal(getattr(plain, name), getattr(fused, name)), name
    assert torch.equal(attn.attention_tok_pre(plain), o[0].transpose(0, 1))


def test_token_attention_constant_v_and_one_dominant_key(ops):
    attn, lib = ops
    lq, lk, h = 300, 900, 2
    q, _, _ = inputs.attention_case(lq, h, seed=5)
    _, k, _ = inputs.attention_case(lk, h, seed=6)
    c = torch.randn(1, h, 128, generator=inputs.gen(9)).to(torch.bfloat16)
    v = c.expand(lk, h, 128).contiguous()
    out = attn.attention(q.cuda(), k.cuda(), v.cuda(), rotate=True)
    assert rel_l2(out.cpu(), c.expand(lq, h, 128)) < 4e-3
    # one key far above the rest in the FIRST tile: the later tiles are quantized against their own maxima, so
    # their many small weights still count (a running-maximum P would round them all to zero)
    g = inputs.gen(12)
    q = torch.randn(256, 1, 128, generator=g).to(torch.bfloat16)
    k = (0.05 * torch.randn(2048, 1, 128, generator=g))
    k[3] = 0.6 * q[:, 0].float().mean(0, keepdim=True) + 0.3 * torch.randn(1, 128, generator=g)
    k = k.to(torch.bfloat16)
    v = torch.randn(2048, 1, 128, generator=g).to(torch.bfloat16)
    out = attn.attention(q.cuda(), k.cuda(), v.cuda(), rotate=True)
    lib.check_status()
    assert rel_l2(out.cpu(), ot.attention(q, k, v)) <= TOL
    assert rel_l2(out.cpu(), oa.attention_fp32(q, k, v)) < 0.02


def test_token_attention_full_size_sampled_rows(ops):
    """B=1, H=32, D=128, L=36,288: sampled rows of two heads against the oracle."""
    attn, lib = ops
    l, h = 36288, 32
    g = torch.Generator(device="cuda").manual_seed(0)
    q = torch.randn(l, h, 128, device="cuda", generator=g).to(torch.bfloat16)
    k = (torch.randn(l, h, 128, device="cuda", generator=g) +
         2.0 * torch.randn(1, h, 128, device="cuda", generator=g)).to(torch.bfloat16)
    v = torch.randn(l, h, 128, device="cuda", generator=g).to(torch.bfloat16)
    out = attn.attention(q, k, v, rotate=True)
    lib.check_status()
    heads = [0, 17]
    rows = torch.randint(0, l, (128,), generator=inputs.gen(1))
    rows[0], rows[1] = 0, l - 1
    ref = ot.attention(q[:, heads].cpu(), k[:, heads].cpu(), v[:, heads].cpu(), rows=rows)
    assert rel_l2(out[rows][:, heads].cpu(), ref) <= TOL
    assert torch.isfinite(out.float()).all()


def test_error_against_fp32_on_the_reference_benchmark_distribution(ops):
    """The reference reports 2.06 % (S = 22,332) for its production numerics against fp32 attention on its synthetic
    outlier inputs, and about 2.3x less on real activations (csrc/attn_cake/DESIGN.md, "Correctness"). The same
    distribution, same size, two heads: the token-scaled kernel must land there, and the fast kernel's e4m3 numerics
    are recorded beside it."""
    attn, lib = ops
    s, h = 22332, 2
    q, k, v = inputs.attention_outlier_case(s, h, seed=0, device="cuda")
    out_tok = attn.attention(q, k, v, rotate=True)
    out_fast = attn.attention(q, k, v)
    lib.check_status()
    ref = torch.empty(s, h, 128, device="cuda")
    for hh in range(h):
        for r0 in range(0, s, 4096):
            w = torch.softmax((q[r0:r0 + 4096, hh].float() @ k[:, hh].float().t()) * 128 ** -0.5, -1)
            ref[r0:r0 + 4096, hh] = w @ v[:, hh].float()
    e_tok, e_fast = rel_l2(out_tok, ref), rel_l2(out_fast, ref)
    print(f"error vs fp32 at S={s} on the outlier distribution: token-scaled {e_tok:.4f}, fast (e4m3 P, V) {e_fast:.4f}")
    assert 0.017 < e_tok < 0.024      # observed 0.0204; the reference's figure for its kernel is 0.0206
    assert e_tok < e_fast
