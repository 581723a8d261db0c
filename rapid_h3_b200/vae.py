"""Causal 3-D convolution VAE decoder (latent -> RGB video) on the conv3d implicit-GEMM kernel.

The benchmark configuration asks for a causal 3x3x3-conv decoder with channel widths 512 -> 256 -> 128 and
GroupNorm + SiLU; the reference repository contains no such decoder (its fast VAE path patches a transformer
decoder, custom_nodes/rapid_h3/vae_fast.py:430-437), so the layer list is defined here:

    conv_in 16 -> 512                                               @ T x H x W
    stage A: 2 x ResBlock(512); upsample (t 2x causal, s 2x); conv 512 -> 256    @ (2T-1) x 2H x 2W
    stage B: 2 x ResBlock(256); upsample;                     conv 256 -> 128    @ (4T-3) x 4H x 4W
    stage C: 2 x ResBlock(128)
    head:    GroupNorm + SiLU; conv 128 -> 3*8*8; depth-to-space 8 -> RGB [3, 4T-3, 32H, 32W]
    ResBlock(c): x + conv(GN_SiLU(conv(GN_SiLU(x))))    (GroupNorm: 32 groups, eps 1e-6)

A 16 x 36 x 24 x 42 latent becomes 3 x 141 x 768 x 1344. Activations are channels-last bf16; the statistics
of every GroupNorm come from the epilogue of the convolution that produced its input. With `sp` (a
TimeShards object) every rank decodes a slab of frames: two halo frames travel to the next rank before each
convolution and the GroupNorm sums are all-reduced.
"""
import torch
import torch.distributed as dist

from . import _lib

GROUPS = 32
EPS = 1e-6


def conv3d_causal(x, w, bias=None, residual=None, want_stats=False, halo=None):
    """x [N,T,H,W,Cin] bf16 channels-last, w [Cout,27,Cin] bf16 -> (out [N,T,H,W,Cout], partial GN sums or None).
    `halo` ([N,2,H,W,Cin], the two frames preceding x on the previous time shard) replaces the causal zero
    padding: the convolution then runs on the concatenation and the first two output frames are dropped."""
    _lib.require_cuda(x, w)
    if halo is not None:
        x = torch.cat([halo, x], 1)
        if residual is not None:
            residual = torch.cat([torch.zeros_like(residual[:, :2]), residual], 1)
    n, t, h, wd, cin = x.shape
    cout = w.shape[0]
    assert x.is_contiguous() and w.is_contiguous() and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    assert w.shape[1] == 27 and w.shape[2] == cin
    out = torch.empty((n, t, h, wd, cout), device=x.device, dtype=torch.bfloat16)
    part = None
    if want_stats and halo is None:
        rows = _lib.lib().rh3_conv3d_gn_part_rows(n, t, h, wd)
        part = torch.empty((rows, GROUPS, 2), device=x.device, dtype=torch.float32)
    _lib.call("rh3_conv3d_causal", x.data_ptr(), w.data_ptr(), _lib.ptr(bias), _lib.ptr(residual), out.data_ptr(),
              _lib.ptr(part), n, t, h, wd, cin, cout, _lib.stream())
    if halo is not None:
        out = out[:, 2:].contiguous()
        if want_stats:  # statistics of the kept frames only: recomputed from the output (halo frames excluded)
            return out, None
    return out, part


def gn_sums(part, n):
    """fp64 [N, 32, 2] (sum, sum of squares) from the convolution's partials."""
    sums = torch.empty((n, GROUPS, 2), device=part.device, dtype=torch.float64)
    _lib.call("rh3_gn_reduce", part.data_ptr(), part.shape[0] // n, n, sums.data_ptr(), _lib.stream())
    return sums


def gn_sums_from_tensor(x):
    """The same sums taken from a stored tensor (used where a halo made the convolution's partials unusable)."""
    n, c = x.shape[0], x.shape[-1]
    xf = x.reshape(n, -1, GROUPS, c // GROUPS).double()
    return torch.stack([xf.sum(dim=(1, 3)), (xf * xf).sum(dim=(1, 3))], -1)


def gn_silu(x, sums, count, gamma, beta):
    """GroupNorm(32 groups) + SiLU of x [N,T,H,W,C] given its (sum, sum of squares) per (sample, group)."""
    n, c = x.shape[0], x.shape[-1]
    mean = sums[..., 0] / count
    var = (sums[..., 1] / count - mean * mean).clamp_min(0.0)
    mr = torch.stack([mean, torch.rsqrt(var + EPS)], -1).float().contiguous()
    y = torch.empty_like(x)
    _lib.call("rh3_gn_silu_apply", x.data_ptr(), mr.data_ptr(), gamma.data_ptr(), beta.data_ptr(), n,
              x.numel() // (n * c), c, y.data_ptr(), _lib.stream())
    return y


def upsample(x):
    n, t, h, w, c = x.shape
    y = torch.empty((n, 2 * t - 1, 2 * h, 2 * w, c), device=x.device, dtype=x.dtype)
    _lib.call("rh3_upsample_causal2x", x.data_ptr(), y.data_ptr(), n, t, h, w, c, _lib.stream())
    return y


class TimeShards:
    """Frames of the decoder's activations split over ranks (contiguous slabs of LATENT frames). The slab of
    rank r > 0 starts after a causal upsampling at frame 2*t0 - 1, so slabs stay contiguous at every stage."""

    def __init__(self, latent_frames, group=None):
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        base, extra = divmod(latent_frames, self.world)
        self.bounds, a = [], 0
        for r in range(self.world):
            b = a + base + (1 if r < extra else 0)
            self.bounds.append((a, b))
            a = b
        self.t0, self.t1 = self.bounds[self.rank]

    def halo(self, x):
        """The last two frames of the previous rank's slab ([N,2,H,W,C]; zeros on rank 0 = causal padding)."""
        recv = torch.zeros_like(x[:, :2])
        ops = []
        if self.rank + 1 < self.world:
            ops.append(dist.P2POp(dist.isend, x[:, -2:].contiguous(), self.rank + 1, self.group))
        if self.rank > 0:
            ops.append(dist.P2POp(dist.irecv, recv, self.rank - 1, self.group))
        if ops:
            for req in dist.batch_isend_irecv(ops):
                req.wait()
        return recv

    def all_reduce(self, t):
        dist.all_reduce(t, group=self.group)
        return t

    def upsample(self, x):
        """Causal 2x upsampling of a slab: every rank but the first also repeats its first frame."""
        y = upsample(x)
        if self.rank == 0:
            return y
        return torch.cat([y[:, :1], y], 1)


class VAEDecoder:
    """Random-init decoder weights (conv weights ~ N(0, 0.02), biases ~ N(0, 0.01), GroupNorm gamma 1 + 0.1 N,
    beta 0.1 N) and the forward pass. Weights are generated on the CPU from `seed` so the oracle sees the same."""

    WIDTHS = (512, 256, 128)

    def __init__(self, latent_ch=16, seed=0, device="cuda", widths=None, blocks_per_stage=2):
        self.widths = tuple(widths or self.WIDTHS)
        self.latent_ch, self.blocks = latent_ch, blocks_per_stage
        g = torch.Generator().manual_seed(seed)
        self.p = {}

        def conv(name, cin, cout):
            self.p[name + ".w"] = (0.02 * torch.randn(cout, 27, cin, generator=g)).to(torch.bfloat16)
            self.p[name + ".b"] = (0.01 * torch.randn(cout, generator=g)).to(torch.bfloat16)

        def norm(name, c):
            self.p[name + ".g"] = (1 + 0.1 * torch.randn(c, generator=g)).to(torch.bfloat16)
            self.p[name + ".be"] = (0.1 * torch.randn(c, generator=g)).to(torch.bfloat16)

        conv("conv_in", 64, self.widths[0])  # latent channels are zero-padded to one 64-channel chunk
        self.p["conv_in.w"][:, :, latent_ch:] = 0
        for si, c in enumerate(self.widths):
            for bi in range(blocks_per_stage):
                for k in (1, 2):
                    norm(f"s{si}.b{bi}.n{k}", c)
                    conv(f"s{si}.b{bi}.c{k}", c, c)
            if si + 1 < len(self.widths):
                conv(f"s{si}.up", c, self.widths[si + 1])
        norm("head.n", self.widths[-1])
        conv("head.c", self.widths[-1], 3 * 64)
        self.cpu = {k: v.clone() for k, v in self.p.items()}
        self.p = {k: v.to(device).contiguous() for k, v in self.p.items()}

    def flops(self, t, h, w):
        """Multiply-add operations x 2 of one decode of a t x h x w latent."""
        total, sites = 0, t * h * w
        total += 2 * sites * 64 * self.widths[0] * 27
        for si, c in enumerate(self.widths):
            total += 2 * sites * c * c * 27 * 2 * self.blocks
            if si + 1 < len(self.widths):
                t, h, w = 2 * t - 1, 2 * h, 2 * w
                sites = t * h * w
                total += 2 * sites * c * self.widths[si + 1] * 27
        return total + 2 * sites * self.widths[-1] * 192 * 27

    def decode(self, latent, sp=None):
        """latent [N, C, T, H, W] bf16 -> RGB [N, 3, 4T-3, 32H, 32W] bf16 (with `sp`: this rank's frames)."""
        p = self.p
        n, c, t, h, w = latent.shape
        x = torch.zeros((n, t, h, w, 64), device=latent.device, dtype=torch.bfloat16)
        x[..., :c] = latent.permute(0, 2, 3, 4, 1)

        def conv(name, x, residual=None, stats=True):
            halo = sp.halo(x) if sp is not None else None
            y, part = conv3d_causal(x, p[name + ".w"], p[name + ".b"], residual, want_stats=stats, halo=halo)
            if not stats:
                return y, None
            sums = gn_sums(part, n) if part is not None else gn_sums_from_tensor(y)
            count = y.numel() // (n * GROUPS)
            if sp is not None:
                sums = sp.all_reduce(sums)
                cnt = torch.tensor([float(count)], device=y.device, dtype=torch.float64)
                count = sp.all_reduce(cnt).item()
            return y, (sums, count)

        x, st = conv("conv_in", x)
        for si in range(len(self.widths)):
            for bi in range(self.blocks):
                hdn = gn_silu(x, *st, p[f"s{si}.b{bi}.n1.g"], p[f"s{si}.b{bi}.n1.be"])
                hdn, st2 = conv(f"s{si}.b{bi}.c1", hdn)
                hdn = gn_silu(hdn, *st2, p[f"s{si}.b{bi}.n2.g"], p[f"s{si}.b{bi}.n2.be"])
                x, st = conv(f"s{si}.b{bi}.c2", hdn, residual=x)
            if si + 1 < len(self.widths):
                x = upsample(x) if sp is None else sp.upsample(x)
                x, st = conv(f"s{si}.up", x)
        x = gn_silu(x, *st, p["head.n.g"], p["head.n.be"])
        y, _ = conv("head.c", x, stats=False)                      # [N, T', H', W', 3*8*8]
        n, t2, h2, w2, _ = y.shape
        y = y.view(n, t2, h2, w2, 3, 8, 8).permute(0, 4, 1, 2, 5, 3, 6)  # depth-to-space: pure data movement
        return y.reshape(n, 3, t2, h2 * 8, w2 * 8)
