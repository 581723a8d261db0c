"""Parity of the attention pre-pass (bit-exact operands) and of the INT8-QK / FP8-PV flash attention
kernel (bf16 output within rel-L2 1e-3 of the emulation of the same quantized op) with the CPU oracle.
Input generators follow bench/rmsrope_fuse.py:22-54 and bench/attn_cake.py:20-35 of the reference."""
import pytest
import torch

from oracle import attention as oa
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
    """[S, 3*H*128] bf16 like a qkv GEMM output: per-channel scale spread and a per-channel K offset."""
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


@pytest.mark.parametrize("s", [1000, 4096, 37])
def test_rmsnorm_rope_bit_exact(ops, s):
    attn, lib = ops
    h = 6
    buf = qkv_buffer(s, h, seed=s)
    q, k, v = views(buf, h)
    tab = inputs.rope_table(inputs.random_positions(s, seed=1))
    qw, kw = inputs.norm_weights()
    bd = buf.cuda()
    qd, kd, vd = views(bd, h)
    raw = bd.clone()
    y = attn.rms_rope(qd, qw.cuda(), 1e-5, tab.cuda())
    assert torch.equal(bd, raw)  # input untouched
    assert torch.equal(y.cpu(), oa.rmsnorm_rope(q, qw, 1e-5, tab))
    y2 = attn.rms_rope(kd, kw.cuda(), 1e-5, None)
    assert torch.equal(y2.cpu(), oa.rmsnorm_rope(k, kw, 1e-5, None))
    attn.rms_rope(kd, kw.cuda(), 1e-5, tab.cuda(), out=kd)  # in place on a strided view
    assert torch.equal(kd.cpu(), oa.rmsnorm_rope(k, kw, 1e-5, tab))
    assert torch.equal(vd.cpu(), v)
    lib.check_status()


@pytest.mark.parametrize("s", [1000, 4096, 64, 129])
def test_prepass_operands_bit_exact(ops, s):
    attn, lib = ops
    h = 4
    buf = qkv_buffer(s, h, seed=s + 1)
    q, k, v = views(buf, h)
    pre = attn.int8_prepass(*views(buf.cuda(), h))
    lib.check_status()
    ref = oa.prepass(q, k, v)
    assert torch.equal(pre.kmean.cpu(), ref["kmean"])
    assert torch.equal(pre.vmean.cpu(), ref["vmean"])
    assert torch.equal(pre.vscale.cpu(), ref["vscale"])
    assert torch.equal(pre.qs.cpu(), ref["qs"]) and torch.equal(pre.q8.cpu(), ref["q8"])
    assert torch.equal(pre.ks.cpu(), ref["ks"]) and torch.equal(pre.k8.cpu(), ref["k8"])
    assert torch.equal(pre.vt.cpu().view(torch.uint8), ref["vt"])


@pytest.mark.parametrize("shape", [(128, 128), (1000, 1000), (4096, 4096), (777, 512), (200, 64), (64, 1300)])
def test_attention_matches_oracle(ops, shape):
    attn, lib = ops
    lq, lk = shape
    h = 3
    q, _, _ = inputs.attention_case(lq, h, seed=lq)
    _, k, v = inputs.attention_case(lk, h, seed=lk + 7)
    pre = attn.int8_prepass(q.cuda(), k.cuda(), v.cuda())
    out = attn.attention_pre(pre)
    lib.check_status()
    ref_pre = oa.prepass(q, k, v)
    assert torch.equal(pre.q8.cpu(), ref_pre["q8"]) and torch.equal(pre.k8.cpu(), ref_pre["k8"])
    ref = oa.attention_pre(ref_pre)
    assert rel_l2(out.cpu(), ref) <= TOL
    # and the quantization error against fp32 attention stays in the range of this numerics class
    full = oa.attention_fp32(q, k, v)
    assert rel_l2(out.cpu(), full) < 0.05   # the oracle itself sits near 0.04 on these inputs (e4m3 P dominates)


@pytest.mark.parametrize("tile", [(0, 0, 0), (2, 9, 1), (2, 7, 10)])
def test_int32_scores_of_a_tile_are_exact(ops, tile):
    """The int32 accumulator the softmax reads (Q8 . K8^T of one 128 x 128 tile, kept pre-biased by 1.5 * 2^23 in
    TMEM) against the integer matrix product of the same codes: bit for bit, including a tile that holds the
    ragged end of the queries and the keys (zero padding) and scores near the largest magnitude int8 rows reach."""
    attn, lib = ops
    head, q_tile, kv_tile = tile
    lq, lk, h = 1230, 1390, 3
    q, _, _ = inputs.attention_case(lq, h, seed=21)
    _, k, v = inputs.attention_case(lk, h, seed=22)
    q[5] = 40.0                      # rows whose codes are all +-127: |s| up to 127 * 127 * 128 = 2.06e6 < 2^22
    k[7] = -40.0
    pre = attn.int8_prepass(q.cuda(), k.cuda(), v.cuda())
    out = torch.empty(lq, h, 128, device="cuda", dtype=torch.bfloat16)
    dump = torch.full((128, 128), -1, dtype=torch.int32, device="cuda")
    lib.call("rh3_attn_int8_dump_scores", pre.q8.data_ptr(), pre.qs.data_ptr(), pre.k8.data_ptr(), pre.ks.data_ptr(),
             pre.vt.data_ptr(), pre.vscale.data_ptr(), pre.vmean.data_ptr(), lq, pre.q8.shape[1], lk, pre.k8.shape[1], h,
             float(128 ** -0.5), out.data_ptr(), out.stride(0), out.stride(1), head, q_tile, kv_tile, dump.data_ptr(),
             lib.stream())
    lib.check_status()
    q8 = pre.q8[head, q_tile * 128:(q_tile + 1) * 128].cpu().long()
    k8 = pre.k8[head, kv_tile * 128:(kv_tile + 1) * 128].cpu().long()
    want = (q8 @ k8.t()).to(torch.int32)
    assert torch.equal(dump.cpu(), want)
    if tile == (0, 0, 0):
        assert want.abs().max() > 1_000_000          # the large scores are in this tile
    assert torch.equal(out, attn.attention_pre(pre))  # the dump changes nothing else


def test_attention_rr_and_strided_output(ops):
    attn, lib = ops
    s, h = 1500, 4
    buf = qkv_buffer(s, h, seed=3)
    q, k, v = views(buf, h)
    tab = inputs.rope_table(inputs.random_positions(s, seed=2))
    qw, kw = inputs.norm_weights()
    bd = buf.cuda()
    qd, kd, vd = views(bd, h)
    o = torch.zeros(1, h, s, 128, dtype=torch.bfloat16, device="cuda")  # head-major, as the fused block wants it
    attn.attention_rr(qd, kd, vd, tab.cuda(), qw.cuda(), kw.cuda(), 1e-5, out=o[0].transpose(0, 1))
    lib.check_status()
    qn, kn = oa.rmsnorm_rope(q, qw, 1e-5, tab), oa.rmsnorm_rope(k, kw, 1e-5, tab)
    ref = oa.attention(qn, kn, v)
    assert rel_l2(o[0].transpose(0, 1).cpu(), ref) <= TOL
    o2 = attn.attention_bhsd(qn.cuda().transpose(0, 1).unsqueeze(0), kn.cuda().transpose(0, 1).unsqueeze(0),
                             vd.transpose(0, 1).unsqueeze(0))
    assert torch.equal(o2, o)


def test_constant_v_returns_the_constant(ops):
    # softmax weights sum to one: a V that is constant over tokens must come back unchanged
    attn, lib = ops
    lq, lk, h = 300, 900, 2
    q, k, _ = inputs.attention_case(lq, h, seed=5)
    _, k, _ = inputs.attention_case(lk, h, seed=6)
    c = torch.randn(1, h, 128, generator=inputs.gen(9)).to(torch.bfloat16)
    v = c.expand(lk, h, 128).contiguous()
    out = attn.attention(q.cuda(), k.cuda(), v.cuda())
    assert rel_l2(out.cpu(), c.expand(lq, h, 128)) < 4e-3  # bf16 rounding of the mean path


def test_config1_full_size_properties(ops):
    """B=1, H=32, D=128, L=36,288; K with a per-channel mean offset ~ N(0,2). Checks sampled rows of two
    heads against the oracle, and invariance under a permutation of whole 64-key blocks."""
    attn, lib = ops
    l, h = 36288, 32
    g = torch.Generator(device="cuda").manual_seed(0)
    q = torch.randn(l, h, 128, device="cuda", generator=g).to(torch.bfloat16)
    k = (torch.randn(l, h, 128, device="cuda", generator=g) +
         2.0 * torch.randn(1, h, 128, device="cuda", generator=g)).to(torch.bfloat16)
    v = torch.randn(l, h, 128, device="cuda", generator=g).to(torch.bfloat16)
    out = attn.attention(q, k, v)
    lib.check_status()
    heads = [0, 17]
    rows = torch.randint(0, l, (192,), generator=inputs.gen(1))
    rows[0], rows[1] = 0, l - 1
    ref = oa.attention(q[:, heads].cpu(), k[:, heads].cpu(), v[:, heads].cpu(), rows=rows)
    got = out[rows][:, heads].cpu()
    assert rel_l2(got, ref) <= TOL
    perm = (torch.randperm(l // 64, generator=inputs.gen(2))[:, None] * 64 + torch.arange(64)[None]).reshape(-1).cuda()
    out_p = attn.attention(q, k[perm], v[perm])
    assert rel_l2(out_p, out) < 3e-3  # bf16 output rounding amplifies last-bit changes of the statistics
    assert torch.isfinite(out.float()).all()


def test_prepass_operands_match_the_reference_emulation_fixture(ops):
    """The CUDA pre-pass against the fake-quantized tensors the reference's bench/attn_emulate.py produced on CPU
    (`q8(q, 1, 64)`, `q8(k - kmean, 1, 64)`, `f8(v - vmean, 0)`; tests/golden/attn_ref.pt): codes x scales equal them
    bit for bit, and the channel means the fixture was made with are the ones the kernels compute."""
    import os
    attn, lib = ops
    g = torch.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "attn_ref.pt"))
    q, k, v = g["q"], g["k"], g["v"]
    l = q.shape[0]
    pre = attn.int8_prepass(q.cuda(), k.cuda(), v.cuda())
    lib.check_status()
    assert torch.equal(pre.kmean.cpu(), g["kmean"]) and torch.equal(pre.vmean.cpu(), g["vmean"])
    blk = torch.arange(l) // 64
    for h, ref in enumerate(g["heads"]):
        assert torch.equal(pre.q8[h, :l].cpu().float() * pre.qs[h].cpu()[blk][:, None], ref["q_fq"])
        assert torch.equal(pre.k8[h, :l].cpu().float() * pre.ks[h].cpu()[blk][:, None], ref["k_fq"])
        vdec = pre.vt[h, :, :l].cpu().float().t() * pre.vscale[h].cpu()[None]
        assert torch.equal(vdec, ref["v_fq"])
