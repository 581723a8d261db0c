"""The conv3d implicit-GEMM kernel, GroupNorm + SiLU, upsampling and the whole decoder against the CPU
oracle (oracle/vae.py; the reference has no convolutional decoder, so the oracle defines the contract).
bf16 outputs: rel-L2 <= 1e-3 per op (fp32 accumulation order differs between the tensor core and the CPU)."""
import pytest
import torch

from oracle import vae as ov

pytestmark = pytest.mark.gpu


def rel_l2(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm().clamp_min(1e-20)).item()


@pytest.fixture(scope="module")
def vae():
    from rapid_h3_b200 import _lib, vae
    assert torch.cuda.is_available()
    return vae, _lib


@pytest.mark.parametrize("shape", [(1, 3, 6, 21, 64, 64), (2, 4, 9, 10, 128, 256), (1, 2, 24, 42, 64, 512),
                                   (1, 5, 7, 5, 192, 192), (1, 1, 1, 1, 64, 16),
                                   (1, 2, 6, 7, 64, 288), (1, 2, 5, 9, 64, 480),   # split tiles that are not 32 wide
                                   (1, 3, 8, 16, 128, 128), (1, 2, 8, 16, 256, 64)])  # 2 and 4 K chunks per ring stage
def test_conv3d_causal_matches_oracle(vae, shape):
    v, lib = vae
    n, t, h, w, cin, cout = shape
    g = torch.Generator().manual_seed(sum(shape))
    x = torch.randn(n, t, h, w, cin, generator=g).to(torch.bfloat16)
    wt = (0.05 * torch.randn(cout, 27, cin, generator=g)).to(torch.bfloat16)
    b = (0.1 * torch.randn(cout, generator=g)).to(torch.bfloat16)
    res = torch.randn(n, t, h, w, cout, generator=g).to(torch.bfloat16)
    stats = cout % 32 == 0 and 32 % (cout // 32) == 0
    y, part = v.conv3d_causal(x.cuda(), wt.cuda(), b.cuda(), res.cuda(), want_stats=stats)
    lib.check_status()
    ref = ov.conv3d_causal(x, wt, b, res)
    assert rel_l2(y.cpu(), ref) <= 1e-3
    y2, _ = v.conv3d_causal(x.cuda(), wt.cuda())
    assert rel_l2(y2.cpu(), ov.conv3d_causal(x, wt)) <= 1e-3
    if stats:
        sums = v.gn_sums(part, n).cpu()
        yd = y.cpu().double().reshape(n, -1, 32, cout // 32)
        assert torch.allclose(sums[..., 0], yd.sum(dim=(1, 3)), rtol=1e-5, atol=1e-2)
        assert torch.allclose(sums[..., 1], (yd * yd).sum(dim=(1, 3)), rtol=1e-5)


@pytest.mark.parametrize("shape", [(1, 3, 6, 21, 64, 64), (2, 4, 9, 10, 128, 256), (1, 5, 7, 5, 192, 192),
                                   (1, 2, 24, 42, 64, 512), (1, 2, 6, 7, 64, 288), (1, 3, 8, 16, 128, 128),
                                   (1, 2, 8, 16, 256, 64), (1, 2, 4, 8, 64, 32), (1, 2, 4, 9, 128, 96)])
def test_cta_pair_kernel_equals_the_single_cta_kernel(vae, shape):
    """The convolution on CTA pairs (two site tiles per pair, half of the weight rows per CTA; the default) against
    the single-CTA kernel on the same inputs: outputs and GroupNorm partial sums bit for bit, including an odd number
    of site tiles (the odd CTA of the last pair has no tile) and column tiles split over several accumulators."""
    v, lib = vae
    n, t, h, w, cin, cout = shape
    g = torch.Generator().manual_seed(sum(shape) + 1)
    x = torch.randn(n, t, h, w, cin, generator=g).to(torch.bfloat16).cuda()
    wt = (0.05 * torch.randn(cout, 27, cin, generator=g)).to(torch.bfloat16).cuda()
    b = (0.1 * torch.randn(cout, generator=g)).to(torch.bfloat16).cuda()
    res = torch.randn(n, t, h, w, cout, generator=g).to(torch.bfloat16).cuda()
    stats = cout % 32 == 0 and 32 % (cout // 32) == 0
    prev = lib.lib().rh3_gemm_use_pairs(1)   # returns the previous setting
    try:
        y_pair, part_pair = v.conv3d_causal(x, wt, b, res, want_stats=stats)
        lib.lib().rh3_gemm_use_pairs(0)
        y_one, part_one = v.conv3d_causal(x, wt, b, res, want_stats=stats)
    finally:
        lib.lib().rh3_gemm_use_pairs(prev)
    lib.check_status()
    assert torch.equal(y_pair, y_one)
    if stats:
        assert torch.equal(part_pair, part_one)


def test_causality(vae):
    """Changing frame t must leave every output frame before t untouched."""
    v, lib = vae
    g = torch.Generator().manual_seed(3)
    x = torch.randn(1, 6, 8, 8, 64, generator=g).to(torch.bfloat16).cuda()
    wt = (0.05 * torch.randn(64, 27, 64, generator=g)).to(torch.bfloat16).cuda()
    y, _ = v.conv3d_causal(x, wt)
    x2 = x.clone()
    x2[:, 4] += 1
    y2, _ = v.conv3d_causal(x2, wt)
    assert torch.equal(y[:, :4], y2[:, :4]) and not torch.equal(y[:, 4], y2[:, 4])


def test_halo_frames_replace_the_causal_padding(vae):
    """A time shard's convolution: with halo_frames=2 the first two frames of the input buffer are the frames
    before the shard, so output, residual and GroupNorm partials equal those frames of the unsharded convolution
    bit for bit (same kernel, same tiles, same accumulation order)."""
    v, lib = vae
    g = torch.Generator().manual_seed(7)
    n, t, h, w, cin, cout = 2, 7, 6, 10, 64, 64
    x = torch.randn(n, t, h, w, cin, generator=g).to(torch.bfloat16).cuda()
    wt = (0.05 * torch.randn(cout, 27, cin, generator=g)).to(torch.bfloat16).cuda()
    b = (0.1 * torch.randn(cout, generator=g)).to(torch.bfloat16).cuda()
    res = torch.randn(n, t, h, w, cout, generator=g).to(torch.bfloat16).cuda()
    full, _ = v.conv3d_causal(x, wt, b, res)
    t0 = 3  # the shard owns frames 3..6; frames 1, 2 are its halo
    shard, part = v.conv3d_causal(x[:, t0 - 2:].contiguous(), wt, b, res[:, t0:].contiguous(), want_stats=True,
                                  halo_frames=2)
    lib.check_status()
    assert shard.shape == (n, t - t0, h, w, cout) and torch.equal(shard, full[:, t0:])
    sums = v.gn_sums(part, n)
    ref = v.gn_sums_from_tensor(full[:, t0:].contiguous())
    assert torch.allclose(sums, ref, rtol=1e-6)
    # a zero halo is the causal padding itself
    first, _ = v.conv3d_causal(torch.cat([torch.zeros_like(x[:, :2]), x[:, :t0]], 1), wt, b, res[:, :t0].contiguous(),
                               halo_frames=2)
    assert torch.equal(first, full[:, :t0])


def test_gn_silu_and_upsample(vae):
    v, lib = vae
    g = torch.Generator().manual_seed(4)
    x = (torch.randn(2, 3, 5, 7, 128, generator=g) * 2 + 0.5).to(torch.bfloat16)
    gamma = (1 + 0.1 * torch.randn(128, generator=g)).to(torch.bfloat16)
    beta = (0.1 * torch.randn(128, generator=g)).to(torch.bfloat16)
    xd = x.cuda()
    y = v.gn_silu(xd, v.gn_sums_from_tensor(xd), x.numel() // (2 * 32), gamma.cuda(), beta.cuda())
    assert rel_l2(y.cpu(), ov.gn_silu(x, gamma, beta)) <= 1e-3
    assert torch.equal(v.upsample(xd).cpu(), ov.upsample(x))


def test_decoder_matches_oracle(vae):
    v, lib = vae
    dec = v.VAEDecoder(seed=1, widths=(128, 64, 64), blocks_per_stage=1)
    g = torch.Generator().manual_seed(5)
    latent = torch.randn(1, 16, 3, 3, 4, generator=g).to(torch.bfloat16)
    rgb = dec.decode(latent.cuda())
    lib.check_status()
    assert rgb.shape == (1, 3, 9, 96, 128)
    ref = ov.decode(dec.cpu, latent, widths=(128, 64, 64), blocks=1)
    # every layer rounds to bf16 (2^-9 relative); rounding flips compound over the 9 layers, so the whole
    # decoder is compared at a few bf16 ulps while each op alone is held to 1e-3 above
    assert rel_l2(rgb.cpu(), ref) <= 2e-2


def test_decoder_at_the_benchmark_widths_layer_by_layer(vae):
    """The decoder of the benchmark configuration (widths 512 -> 256 -> 128, two residual blocks per stage) on a
    16 x 5 x 6 x 8 latent. Every layer (convolution with bias and residual, GroupNorm + SiLU, causal upsampling)
    is replayed on the oracle's own input of that layer and held to rel-L2 <= 1e-3; the whole 21-layer chain,
    where one-ulp bf16 flips compound from layer to layer, is reported and held to 2e-2."""
    v, lib = vae
    dec = v.VAEDecoder(seed=2)
    assert dec.widths == (512, 256, 128) and dec.blocks == 2
    latent = torch.randn(1, 16, 5, 6, 8, generator=torch.Generator().manual_seed(8)).to(torch.bfloat16)
    trace = []
    ref = ov.decode(dec.cpu, latent, trace=trace)
    worst = {}
    for op, name, ins, want in trace:
        if op == "conv":
            x, res = ins
            got, _ = v.conv3d_causal(x.contiguous().cuda(), dec.p[name + ".w"], dec.p[name + ".b"],
                                     None if res is None else res.contiguous().cuda())
        elif op == "gn":
            xd = ins[0].contiguous().cuda()
            got = v.gn_silu(xd, v.gn_sums_from_tensor(xd), xd.numel() // (xd.shape[0] * 32), dec.p[name + ".g"],
                            dec.p[name + ".be"])
        else:
            got = v.upsample(ins[0].contiguous().cuda())
            assert torch.equal(got.cpu(), want)
        e = rel_l2(got.cpu(), want)
        worst[op] = max(worst.get(op, 0.0), e)
        assert e <= 1e-3, (op, name, e)
    lib.check_status()
    rgb = dec.decode(latent.cuda())
    lib.check_status()
    assert rgb.shape == (1, 3, 17, 192, 256)
    whole = rel_l2(rgb.cpu(), ref)
    print(f"decoder at widths (512, 256, 128): worst layer rel-L2 {worst}, whole chain {whole:.2e}")
    assert whole <= 2e-2


def test_depth_to_space_is_the_head_permutation(vae):
    v, lib = vae
    g = torch.Generator().manual_seed(9)
    n, t, h, w = 2, 3, 5, 7
    y = torch.randn(n, t, h, w, 192, generator=g).to(torch.bfloat16).cuda()
    rgb = v.depth_to_space8(y)
    lib.check_status()
    ref = y.view(n, t, h, w, 3, 8, 8).permute(0, 4, 1, 2, 5, 3, 6).reshape(n, 3, t, h * 8, w * 8)
    assert torch.equal(rgb, ref)


def test_tiled_decode_batches_tiles_across_rows(vae):
    """Spatial tiles, several per decoder call: every decoder call sees at least two tiles, the canvas has the
    untiled shape, and a region no seam touches equals that tile decoded in the same group (the per-tile arithmetic
    does not depend on the other tiles of the call: every op is per sample)."""
    v, lib = vae
    from rapid_h3_b200 import vae_fast
    dec = v.VAEDecoder(seed=4, widths=(128, 64, 64), blocks_per_stage=1)
    latent = torch.randn(1, 16, 2, 5, 7, generator=torch.Generator().manual_seed(6)).to(torch.bfloat16).cuda()
    calls = []
    plain_decode = dec.decode

    def counting(z, sp=None):
        calls.append(z.shape[0])
        return plain_decode(z, sp)

    dec.decode = counting
    rgb = dec.tiled_decode(latent, tile=96, overlap=32, batch=3)
    lib.check_status()
    assert rgb.shape == (1, 3, 5, 160, 224) and torch.isfinite(rgb.float()).all()
    ny, nx = len(vae_fast.split_tiles(160, 96, 32)[0]), len(vae_fast.split_tiles(224, 96, 32)[0])
    assert calls == vae_fast._tile_groups(ny * nx, 3) and min(calls) >= 2
    # tile (0, 0): its first 64 x 64 pixels lie before the first seams
    first = torch.cat([latent[..., 0:3, 0:3], latent[..., 0:3, 2:5], latent[..., 0:3, 4:7]])[: calls[0]]
    alone = plain_decode(first.contiguous())[0:1]
    assert torch.equal(rgb[..., :64, :64], alone[..., :64, :64])
