"""The fused DiT block and the transformer step on the GPU against the CPU oracle block, stage by stage,
plus the step-divergence check against the unquantized bf16 model (the reference's RapidH3Shadow idea,
custom_nodes/rapid_h3/__init__.py:459-487: noise floor = bf16 model on inputs jittered by one bf16 ulp)."""
import pytest
import torch

from oracle import block as ob

pytestmark = pytest.mark.gpu


def rel_l2(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm().clamp_min(1e-20)).item()


@pytest.fixture(scope="module")
def pkg():
    import rapid_h3_b200 as r
    assert torch.cuda.is_available()
    return r


def _case(r, cfg, grid=(5, 4, 5), n_audio=7, text_len=48, seed=0):
    latent, audio, t_emb, rope, ctx = r.step.make_inputs(cfg, grid, n_audio, 1, text_len, seed=seed)
    n_video = grid[0] * grid[1] * grid[2]
    s = n_video + n_audio
    segs = [(0, n_video, 0), (n_video, s, 1)]
    return latent, audio, t_emb, rope, ctx, segs, s


@pytest.mark.parametrize("mode", ["int8_rowwise", "int8_rot"])
@pytest.mark.parametrize("cross", [True, False])
def test_fused_block_matches_oracle_stage_by_stage(pkg, cross, mode):
    r = pkg
    cfg = r.model.H3Config.tiny(cross_attention=cross, text_dim=256)  # rotated widths: whole groups of 256
    blk = r.model.init_weights(r.model.DiTBlock(cfg), seed=1)
    latent, audio, t_emb, rope, ctx, segs, s = _case(r, cfg)
    x = torch.randn(s, cfg.d_model, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16)
    ref_trace = {}
    ref = ob.fused_block(blk, x, t_emb[0], segs, rope, ctx[0], trace=ref_trace, mode=mode)

    import copy
    blk_d = copy.deepcopy(blk).cuda()
    model = torch.nn.Module()
    model.blocks = torch.nn.ModuleList([blk_d])
    patched, = r.nodes.RapidH3LinearQuant().patch(model, mode)
    fb = patched.block_forward[0]
    assert isinstance(fb, r.nodes.FusedBlock) and fb.rotate == (mode == "int8_rot")
    trace = {}
    xd = x.cuda()
    out = fb.forward(xd, t_emb[0].cuda(), segs, rope.cuda(), ctx[0].cuda(), trace=trace)
    r._lib.check_status()
    assert out.data_ptr() == xd.data_ptr()  # residual updated in place, as the reference does
    # everything up to the attention operands is bit-exact
    assert torch.equal(trace["attn_in_q"].cpu(), ref_trace["attn_in_q"])
    assert torch.equal(trace["attn_in_s"].cpu(), ref_trace["attn_in_s"])
    assert torch.equal(trace["qkv"].cpu(), ref_trace["qkv"])
    assert torch.equal(trace["qkv_rr"].cpu(), ref_trace["qkv_rr"])
    # bf16 outputs: rel-L2 <= 1e-3 against the emulation of the same quantized ops
    assert rel_l2(trace["attn_out"].cpu(), ref_trace["attn_out"]) <= 1e-3
    assert rel_l2(trace["x_attn"].cpu(), ref_trace["x_attn"]) <= 1e-3
    if cross:
        assert rel_l2(trace["x_cross"].cpu(), ref_trace["x_cross"]) <= 1e-3
    assert rel_l2(trace["mlp_h"].cpu(), ref_trace["mlp_h"]) <= 2e-3  # int8 codes downstream of attention may flip
    assert rel_l2(out.cpu(), ref) <= 1e-3


@pytest.mark.parametrize("mode", ["int8_rowwise", "int8_rot"])
def test_step_matches_manual_chain_and_bf16_noise_floor(pkg, mode):
    r = pkg
    cfg = r.model.H3Config.tiny(n_blocks=3, text_dim=256)
    model = r.model.init_weights(r.model.H3Transformer(cfg), seed=2).cuda()
    grid, n_audio = (6, 5, 4), 9
    latent, audio, t_emb, rope, ctx = r.step.make_inputs(cfg, grid, n_audio, 2, 40, seed=3)
    dev = [t.cuda() for t in (latent, audio, t_emb, rope, ctx)]
    rt = r.step.H3Runtime(model, mode)
    vid, aud = rt.step(*dev)
    r._lib.check_status()
    assert vid.shape == latent.shape and aud.shape == audio.shape and vid.dtype == torch.bfloat16

    # the quantized step against the unquantized bf16 model, in units of the bf16 one-ulp noise floor
    with torch.no_grad():
        ref = [model(dev[0][i], dev[1][i], dev[2][i], dev[3], dev[4][i]) for i in range(2)]
        g = torch.Generator(device="cuda").manual_seed(1234)
        jit = [t * (1 + 2.0 ** -8 * torch.randn(t.shape, generator=g, device="cuda").to(t.dtype)) for t in dev[:2]]
        noisy = [model(jit[0][i], jit[1][i], dev[2][i], dev[3], dev[4][i]) for i in range(2)]
    ref_v = torch.stack([v for v, _ in ref])
    err = rel_l2(vid, ref_v)
    floor = rel_l2(torch.stack([v for v, _ in noisy]), ref_v)
    print(f"step divergence ({mode}): quantized {err:.4e}, bf16 one-ulp floor {floor:.4e}, ratio {err / floor:.2f}")
    # row-wise int8 on this tiny 3-block model with Gaussian weights sits at ~2.5x the floor with or without
    # the rotation (there are no outlier channels for it to spread); the 2x criterion is quoted for the
    # full-size trained model, so the bound here only guards regressions
    assert err <= 4.0 * floor


@pytest.mark.parametrize("mode", ["int8_rowwise", "int8_rot"])
@pytest.mark.parametrize("attn", ["fast", "token"])
def test_fused_block_at_the_benchmark_width_matches_oracle(pkg, mode, attn):
    """One block of the benchmark configuration (d_model 4096, 32 heads x 128, MLP hidden 16384, cross-attention
    to 512 text tokens of width 4096) on 4096 video + 148 audio tokens: two modality segments, a ragged last
    64-token block, K = 16384 rows in the fc2 quantizer. Stage by stage against the CPU oracle."""
    import copy
    r = pkg
    cfg = r.model.H3Config(n_blocks=1)
    assert (cfg.d_model, cfg.heads, cfg.head_dim, cfg.mlp_hidden, cfg.text_dim) == (4096, 32, 128, 16384, 4096)
    blk = r.model.init_weights(r.model.DiTBlock(cfg), seed=11)
    latent, audio, t_emb, rope, ctx, segs, s = _case(r, cfg, grid=(16, 16, 16), n_audio=148, text_len=512, seed=4)
    assert s == 4244 and s % 64 != 0
    x = torch.randn(s, cfg.d_model, generator=torch.Generator().manual_seed(6)).to(torch.bfloat16)
    model = torch.nn.Module()
    model.blocks = torch.nn.ModuleList([copy.deepcopy(blk).cuda()])
    # the modulation tables are an input of the quantized path: both sides get the ones the device computes (a
    # 4096-long bf16 dot product sums in a different order on the CPU)
    adaln = tuple(t.cpu() for t in model.blocks[0].adaln_proj(t_emb[0].cuda()))
    patched, = r.nodes.RapidH3LinearQuant().patch(model, mode)
    trace = {}
    r.nodes.ATTN_ROTATE = attn == "token"     # both attention numerics go through the same block and the same checks
    try:
        out = patched.block_forward[0].forward(x.cuda(), t_emb[0].cuda(), segs, rope.cuda(), ctx[0].cuda(), trace=trace)
        r._lib.check_status()
    finally:
        r.nodes.ATTN_ROTATE = False
    got = {k: v.cpu() for k, v in trace.items()}
    # every stage of the oracle starts from the residual stream the device produced, so each stage is compared on
    # identical inputs: what is integer (codes, scales, and the bf16 GEMM outputs that follow from them) must be
    # bit-identical, what passes through the attention kernel's exponentials is held to 1e-3
    want = {}
    ref = ob.fused_block(blk, x, t_emb[0], segs, rope, ctx[0], trace=want, mode=mode, adaln=adaln,
                         replay={k: got[k] for k in ("x_attn", "x_cross", "mlp_h")}, attn=attn)
    for name in ("attn_in_q", "attn_in_s", "qkv", "qkv_rr", "cross_in_q", "cross_in_s", "cross_q", "cross_k", "cross_v",
                 "mlp_in_q", "mlp_in_s", "fc2_in_q", "fc2_in_s"):
        assert torch.equal(got[name], want[name]), name
    for name in ("attn_out", "x_attn", "cross_out", "x_cross", "mlp_h", "x_out"):
        assert rel_l2(got[name], want[name]) <= 1e-3, name
    assert rel_l2(out.cpu(), ref) <= 1e-3


@pytest.mark.parametrize("mode", ["int8_rowwise", "int8_rot"])
def test_step_divergence_at_the_benchmark_width(pkg, mode):
    """The step-level acceptance measure at the benchmark width: four random-init blocks (d_model 4096, 32 heads, MLP
    16384, cross-attention) on a 6 x 24 x 42 token grid + 148 audio tokens. The quantized step against the
    unquantized bf16 model, in units of the divergence the bf16 model itself shows when its inputs move by one bf16
    ulp (the reference's RapidH3Shadow measure, __init__.py:459-487).

    The stated bar is 2x that floor. This random-init model does NOT meet it: row-wise W8A8 sits near 5x with or
    without the H256 rotation (Gaussian weights and activations have no outlier channels for the rotation to
    spread; every int8 row quantizer then costs about 1 % per linear, 28 linears deep). The test records the
    ratios, separates the share of the linears from the share of the attention kernel, and holds the measured level
    as a regression bound; it does not claim the 2x bar."""
    r = pkg
    cfg = r.model.H3Config(n_blocks=4)
    model = r.model.init_weights_on_device(
        r.model.H3Transformer(cfg).cuda(), torch.Generator(device="cuda").manual_seed(12))
    grid, n_audio = (6, 24, 42), 148
    latent, audio, t_emb, rope, ctx = r.step.make_inputs(cfg, grid, n_audio, 1, 512, seed=13)
    dev = [t.cuda() for t in (latent, audio, t_emb, rope, ctx)]
    args = (dev[0][0], dev[1][0], dev[2][0], dev[3], dev[4][0])
    with torch.no_grad():
        ref_v, ref_a = model(*args)
        g = torch.Generator(device="cuda").manual_seed(1234)
        jit = [t * (1 + 2.0 ** -8 * torch.randn(t.shape, generator=g, device="cuda").to(t.dtype)) for t in dev[:2]]
        noisy_v, _ = model(jit[0][0], jit[1][0], *args[2:])
        # quantized linears with the stock bf16 attention: the linears' share of the divergence
        lin_only, = r.nodes.RapidH3LinearQuant().patch(model, mode, fuse_block=False)
        lin_v, _ = lin_only(*args)
    rt = r.step.H3Runtime(model, mode)
    vid, aud = rt.step(*dev)
    r._lib.check_status()
    # the same step with the token-scaled attention (the reference's production numerics)
    r.nodes.ATTN_ROTATE = True
    try:
        vid_tok, _ = rt.step(*dev)
        r._lib.check_status()
    finally:
        r.nodes.ATTN_ROTATE = False
    floor = rel_l2(noisy_v, ref_v)
    err, err_lin, err_tok = rel_l2(vid[0], ref_v), rel_l2(lin_v, ref_v), rel_l2(vid_tok[0], ref_v)
    err_attn = max(err * err - err_lin * err_lin, 0.0) ** 0.5
    err_attn_tok = max(err_tok * err_tok - err_lin * err_lin, 0.0) ** 0.5
    print(f"step divergence at d=4096 ({mode}): floor {floor:.3e}; quantized step {err:.3e} = {err / floor:.2f}x; "
          f"linears alone {err_lin:.3e} = {err_lin / floor:.2f}x; attention kernel (in quadrature) {err_attn:.3e} = "
          f"{err_attn / floor:.2f}x; with the token-scaled attention: step {err_tok:.3e} = {err_tok / floor:.2f}x, "
          f"attention {err_attn_tok:.3e} = {err_attn_tok / floor:.2f}x")
    assert torch.isfinite(vid.float()).all() and torch.isfinite(vid_tok.float()).all()
    assert err <= 6.5 * floor            # regression bound at the measured level (5.3x / 4.7x), not the 2x bar
    assert err_lin <= err * 1.05         # the fused path adds the attention kernel's error, it does not hide any
    assert err_tok <= err                # 8-bit P against the tile maximum is the more accurate attention


def test_fused_block_refuses_unsupported_calls(pkg):
    r = pkg
    cfg = r.model.H3Config.tiny()
    model = torch.nn.Module()
    model.blocks = torch.nn.ModuleList([r.model.init_weights(r.model.DiTBlock(cfg), seed=1).cuda()])
    patched, = r.nodes.RapidH3LinearQuant().patch(model, "int8_rowwise")
    x = torch.zeros(8, cfg.d_model, device="cuda")
    with pytest.raises(NotImplementedError):
        patched.block_forward[0].forward(x, None, [], None)
    with pytest.raises(NotImplementedError):
        r.nodes.RapidH3LinearQuant().patch(model, "nvfp4_fake")
    with pytest.raises(ValueError):
        r.nodes.RapidH3LinearQuant().patch(model, "nope")
    same, = r.nodes.RapidH3LinearQuant().patch(model, "bf16")
    assert same.block_forward is None


def test_quant_linear_adapter(pkg):
    r = pkg
    lin = torch.nn.Linear(256, 384, bias=True, dtype=torch.bfloat16).cuda()
    q = r.nodes._QuantLinear(lin, "blocks.0.attn.qkv_proj", "int8_rowwise")
    x = torch.randn(3, 50, 256, device="cuda", dtype=torch.bfloat16)
    y = q(x)
    assert y.shape == (3, 50, 384) and q.calls == 1
    ref = torch.nn.functional.linear(x, lin.weight, lin.bias)
    assert rel_l2(y, ref) < 0.05
    with pytest.raises(NotImplementedError):
        q(x.float())


def test_quant_linear_adopts_prerotated_int8_weight(pkg):
    """A weight that already carries int8 codes of W . blockdiag(H256)^T and per-row scales (the layout of
    ComfyUI's int8_convrot checkpoints) is used as is by `int8_rot` (reference __init__.py:107-117)."""
    import types
    r = pkg
    lin = torch.nn.Linear(512, 256, bias=False, dtype=torch.bfloat16).cuda()
    own = r.kernels.quantize_weight(lin.weight.detach(), "int8_rot")

    class Stored(torch.Tensor):
        pass

    w = torch.empty(0, device="cuda").as_subclass(Stored)
    w._qdata = own.q.clone()
    w._params = types.SimpleNamespace(convrot=True, convrot_groupsize=256, transposed=False, scale=own.scale.reshape(-1, 1))
    mod = types.SimpleNamespace(weight=w, bias=None)
    q = r.nodes._QuantLinear(mod, "blocks.0.mlp.fc2", "int8_rot")
    x = torch.randn(40, 512, device="cuda", dtype=torch.bfloat16)
    y = q(x)
    assert torch.equal(q.qweight.q, own.q) and torch.equal(q.qweight.scale, own.scale)
    assert torch.equal(y, r.kernels.linear(x, own, "int8_rot"))
    assert rel_l2(y, torch.nn.functional.linear(x, lin.weight)) < 0.05


def test_unfused_patch_paths_and_error_statistics(pkg):
    """Blocks that are not fused run their stock forward with the quantized linears installed on the modules
    for the duration of the call: `measure_every` records per-linear errors, `targets="fc1,fc2"` fuses only the
    MLP (SwiGLU inside fc2's quantizer), `keep_bf16_blocks` leaves whole blocks alone."""
    r = pkg
    cfg = r.model.H3Config.tiny(n_blocks=2, text_dim=256)
    model = r.model.init_weights(r.model.H3Transformer(cfg), seed=4).cuda()
    latent, audio, t_emb, rope, ctx = (t.cuda() for t in r.step.make_inputs(cfg, (4, 4, 4), 5, 1, 24, seed=6))
    args = (latent[0], audio[0], t_emb[0], rope, ctx[0])
    with torch.no_grad():
        ref_v, _ = model(*args)

        patched, = r.nodes.RapidH3LinearQuant().patch(model, "int8_rot", measure_every=1)
        assert not any(isinstance(f, r.nodes.FusedBlock) for f in patched.block_forward)
        v, _ = patched(*args)
        assert rel_l2(v, ref_v) < 0.05
        assert len(patched.stats) == len(patched.linears) and all(0 < e[0] < 0.05 for e in patched.stats.values())
        assert "forward" not in model.blocks[0].attn.qkv_proj.__dict__  # the replacement forwards are removed again

        patched, = r.nodes.RapidH3LinearQuant().patch(model, "int8_rowwise", targets="fc1,fc2")
        assert len(patched.linears) == 4 and len(patched.wrappers) == 6  # 4 linears + 2 fused MLPs
        v2, _ = patched(*args)
        assert rel_l2(v2, ref_v) < 0.05
        assert all(q.calls == 1 for n, q in patched.linears.items() if n.endswith("fc1"))
        assert all(q.calls == 0 for n, q in patched.linears.items() if n.endswith("fc2"))  # fc2 ran inside the fused MLP

        patched, = r.nodes.RapidH3LinearQuant().patch(model, "int8_rowwise", keep_bf16_blocks="0")
        assert not isinstance(patched.block_forward[0], r.nodes.FusedBlock)
        assert isinstance(patched.block_forward[1], r.nodes.FusedBlock)
        v3, _ = patched(*args)
        assert rel_l2(v3, ref_v) < 0.05


def test_attention_override_takes_its_calls_and_hands_on_the_rest(pkg):
    """The override of RapidH3Int8Attention: [1, H, S, 128] bf16 calls with S >= 1024 and equal shapes run the INT8
    kernel; short, masked or differently shaped calls go to the override installed before, else to the framework's
    function; `exact_rows` recomputes the named segments' query rows with bf16 SDPA."""
    import types
    r = pkg
    g = torch.Generator(device="cuda").manual_seed(3)
    q, k, v = (torch.randn(1, 2, 1100, 128, device="cuda", generator=g).to(torch.bfloat16) for _ in range(3))
    calls = []

    def stock(q_, k_, v_, **kw):
        calls.append("stock")
        return torch.nn.functional.scaled_dot_product_attention(q_, k_, v_, scale=kw.get("scale"))

    _, ov = r.nodes.RapidH3Int8Attention().patch(None, config=80)
    out = ov(stock, q, k, v, heads=2, skip_reshape=True, skip_output_reshape=True)
    assert not calls and out.shape == q.shape
    want = r.attn_int8.attention_bhsd(q, k, v)
    assert torch.equal(out, want)
    assert ov(stock, q, k, v, heads=2, skip_reshape=True).shape == (1, 1100, 256)
    # not ours: a short sequence, a mask, k shorter than q
    ov(stock, q[:, :, :512], k[:, :, :512], v[:, :, :512], heads=2, skip_reshape=True, skip_output_reshape=True)
    ov(stock, q, k, v, heads=2, mask=torch.zeros(1100, 1100, device="cuda", dtype=torch.bfloat16), skip_reshape=True)
    ov(stock, q, k[:, :, :1024], v[:, :, :1024], heads=2, skip_reshape=True, skip_output_reshape=True)
    assert calls == ["stock"] * 3
    # an override that was there before gets the calls that are not ours
    _, ov2 = r.nodes.RapidH3Int8Attention().patch(None, config=80, previous=lambda f, *a, **kw: "previous")
    assert ov2(stock, q[:, :, :100], k[:, :, :100], v[:, :, :100], skip_reshape=True) == "previous"
    # exact rows: the audio segment's rows equal bf16 SDPA, the others the INT8 kernel
    layout = types.SimpleNamespace(seq_len=1100, segments=[(0, 1000, "video"), (1000, 1100, "audio")])
    _, ov3 = r.nodes.RapidH3Int8Attention().patch(None, config=80, exact_rows="audio")
    out3 = ov3(stock, q, k, v, skip_reshape=True, skip_output_reshape=True, transformer_options={"minimax_h3_layout": layout})
    sdpa = torch.nn.functional.scaled_dot_product_attention(q[:, :, 1000:], k, v)
    assert torch.equal(out3[:, :, 1000:], sdpa) and torch.equal(out3[:, :, :1000], want[:, :, :1000])
    assert ov.rapidh3_rmsrope is None and ov3.rapidh3_rmsrope is None


def test_fused_rope_prepass_self_check(pkg, tmp_path, monkeypatch):
    """config >= 200 switches on the per-call check of the fused RMSNorm + RoPE pre-pass against the unfused one:
    bit-identical output and operands, one JSON line per fused self-attention call."""
    import json
    r = pkg
    log = tmp_path / "rrcheck.jsonl"
    monkeypatch.setenv("RAPIDH3_RRCHECK", str(log))
    try:
        _, ov = r.nodes.RapidH3Int8Attention().patch(None, config=290)
        assert ov.rapidh3_rmsrope == 90 and ov.rapidh3_rrcheck
        cfg = r.model.H3Config.tiny(n_blocks=2, text_dim=256)
        model = r.model.init_weights(r.model.H3Transformer(cfg), seed=2).cuda()
        dev = [t.cuda() for t in r.step.make_inputs(cfg, (6, 5, 4), 9, 1, 40, seed=3)]
        r.step.H3Runtime(model).step(*dev)
        torch.cuda.synchronize()
    finally:
        r.nodes.RR_CHECK = None
    recs = [json.loads(line) for line in log.read_text().splitlines()]
    assert len(recs) == 2 and all(x["out_equal"] and x["operands_equal"] and x["max_abs_diff"] == 0.0 for x in recs)
