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


def conv3d_causal(x, w, bias=None, residual=None, want_stats=False, halo_frames=0):
    """x [N,T,H,W,Cin] bf16 channels-last, w [Cout,27,Cin] bf16 -> (out [N,T,H,W,Cout], partial GN sums or None).
    `halo_frames=2`: x is [N,T+2,H,W,Cin] and its first two frames are the frames that precede output frame 0 (the
    previous time shard's last two) instead of the causal zero padding; the output still has T frames."""
    _lib.require_cuda(x, w)
    n, t_in, h, wd, cin = x.shape
    t = t_in - halo_frames
    cout = w.shape[0]
    assert x.is_contiguous() and w.is_contiguous() and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    assert w.shape[1] == 27 and w.shape[2] == cin and halo_frames in (0, 2) and t > 0
    assert residual is None or (residual.is_contiguous() and residual.shape == (n, t, h, wd, cout))
    out = torch.empty((n, t, h, wd, cout), device=x.device, dtype=torch.bfloat16)
    part = None
    if want_stats:
        rows = _lib.lib().rh3_conv3d_gn_part_rows(n, t, h, wd)
        part = torch.empty((rows, GROUPS, 2), device=x.device, dtype=torch.float32)
    _lib.call("rh3_conv3d_causal", x.data_ptr(), w.data_ptr(), _lib.ptr(bias), _lib.ptr(residual), out.data_ptr(),
              _lib.ptr(part), n, t, h, wd, cin, cout, halo_frames, _lib.stream())
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


def gn_silu(x, sums, count, gamma, beta, out=None):
    """GroupNorm(32 groups) + SiLU of x [N,T,H,W,C] given its (sum, sum of squares) per (sample, group);
    `out` may be a contiguous buffer of x's shape (e.g. the data frames of a halo-padded buffer)."""
    n, c = x.shape[0], x.shape[-1]
    mean = sums[..., 0] / count
    var = (sums[..., 1] / count - mean * mean).clamp_min(0.0)
    mr = torch.stack([mean, torch.rsqrt(var + EPS)], -1).float().contiguous()
    y = torch.empty_like(x) if out is None else out
    assert y.shape == x.shape and y.is_contiguous() and y.dtype == x.dtype
    _lib.call("rh3_gn_silu_apply", x.data_ptr(), mr.data_ptr(), gamma.data_ptr(), beta.data_ptr(), n,
              x.numel() // (n * c), c, y.data_ptr(), _lib.stream())
    return y


def upsample(x, out=None):
    n, t, h, w, c = x.shape
    y = torch.empty((n, 2 * t - 1, 2 * h, 2 * w, c), device=x.device, dtype=x.dtype) if out is None else out
    assert y.shape == (n, 2 * t - 1, 2 * h, 2 * w, c) and y.is_contiguous()
    _lib.call("rh3_upsample_causal2x", x.data_ptr(), y.data_ptr(), n, t, h, w, c, _lib.stream())
    return y


def depth_to_space8(y):
    """y [N, T, H, W, 192] (channel = (ch*8 + dy)*8 + dx) -> [N, 3, T, 8H, 8W]."""
    n, t, h, w, c = y.shape
    assert c == 192 and y.is_contiguous() and y.dtype == torch.bfloat16
    rgb = torch.empty((n, 3, t, 8 * h, 8 * w), device=y.device, dtype=torch.bfloat16)
    _lib.call("rh3_depth_to_space8", y.data_ptr(), rgb.data_ptr(), n, t, h, w, _lib.stream())
    return rgb


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

    def frames_per_rank(self, upsamples):
        """Frames every rank holds after `upsamples` causal 2x upsamplings (rank 0: 2t-1 each time, others 2t)."""
        out = []
        for r, (a, b) in enumerate(self.bounds):
            f = b - a
            for _ in range(upsamples):
                f = 2 * f - 1 if r == 0 else 2 * f
            out.append(f)
        return out

    def padded(self, n, t, h, w, c, device):
        """A buffer [N, t+2, H, W, C] and the view of its last t frames: producers write the view, `exchange`
        fills the two leading frames, and the convolution reads the whole buffer with halo_frames=2."""
        buf = torch.empty((n, t + 2, h, w, c), device=device, dtype=torch.bfloat16)
        return buf, buf[:, 2:]

    def exchange(self, buf):
        """Fill frames 0, 1 of a padded buffer with the previous rank's last two frames (zeros on rank 0: causal
        padding) and send this rank's last two to the next one."""
        n = buf.shape[0]
        ops, recv = [], None
        if self.rank + 1 < self.world:
            ops.append(dist.P2POp(dist.isend, buf[:, -2:].contiguous(), self.rank + 1, self.group))
        if self.rank > 0:
            recv = buf[:, :2] if n == 1 else torch.empty_like(buf[:, :2].contiguous())
            ops.append(dist.P2POp(dist.irecv, recv, self.rank - 1, self.group))
        else:
            buf[:, :2].zero_()
        if ops:
            for req in dist.batch_isend_irecv(ops):
                req.wait()
        if recv is not None and n != 1:
            buf[:, :2] = recv
        return buf

    def all_reduce(self, t):
        dist.all_reduce(t, group=self.group)
        return t


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

    RATIO = 32  # output pixels per latent cell along height and width

    def tiled_decode(self, latent, tile=512, overlap=128, batch=4):
        """Decode in spatial tiles of `tile` output pixels sharing `overlap` pixels, `batch` tiles per decoder call
        across tile rows, seams cross-faded (vae_fast.tiled_decode_batched; the reference's whole-chunk tile
        batching, custom_nodes/rapid_h3/vae_fast.py:336-400). For latents whose activations do not fit at once; the
        GroupNorm statistics are then per tile, so the picture is not the untiled one."""
        from . import vae_fast
        return vae_fast.tiled_decode_batched(lambda z: self.decode(z.contiguous()), latent, self.RATIO, tile, overlap, batch)

    def decode(self, latent, sp=None):
        """latent [N, C, T, H, W] bf16 -> RGB [N, 3, 4T-3, 32H, 32W] bf16 (with `sp`: this rank's frames).
        With `sp` every activation that feeds a convolution is produced straight into a halo-padded buffer, the
        two halo frames arrive from the previous rank, and nothing is copied or recomputed for the halo."""
        p = self.p
        n, c, t, h, w = latent.shape
        dev = latent.device
        ups = 0  # causal upsamplings so far (for the global element count of the GroupNorm statistics)

        def new_act(t_, h_, w_, c_):
            """(buffer handed to the next convolution, view the producer writes)."""
            if sp is None:
                y = torch.empty((n, t_, h_, w_, c_), device=dev, dtype=torch.bfloat16)
                return y, y
            return sp.padded(n, t_, h_, w_, c_, dev)

        def conv(name, buf, residual=None, stats=True):
            if sp is not None:
                sp.exchange(buf)
            y, part = conv3d_causal(buf, p[name + ".w"], p[name + ".b"], residual, want_stats=stats,
                                    halo_frames=0 if sp is None else 2)
            if not stats:
                return y, None
            sums = gn_sums(part, n)
            count = y.numel() // (n * GROUPS)
            if sp is not None:
                sums = sp.all_reduce(sums)
                count = sum(sp.frames_per_rank(ups)) * (count // y.shape[1])
            return y, (sums, count)

        def norm_act(x, st, name):
            """GroupNorm + SiLU of x written where the next convolution reads it."""
            buf, view = new_act(*x.shape[1:])
            if view.is_contiguous():
                gn_silu(x, *st, p[name + ".g"], p[name + ".be"], out=view)
            else:  # several samples in a padded buffer: the data frames of a sample are not adjacent to the next one's
                view.copy_(gn_silu(x, *st, p[name + ".g"], p[name + ".be"]))
            return buf

        buf, view = new_act(t, h, w, 64)
        view.zero_()
        view[..., :c] = latent.permute(0, 2, 3, 4, 1)
        x, st = conv("conv_in", buf)
        for si in range(len(self.widths)):
            for bi in range(self.blocks):
                hdn, st2 = conv(f"s{si}.b{bi}.c1", norm_act(x, st, f"s{si}.b{bi}.n1"))
                x, st = conv(f"s{si}.b{bi}.c2", norm_act(hdn, st2, f"s{si}.b{bi}.n2"), residual=x)
            if si + 1 < len(self.widths):
                _, tx, hx, wx, cx = x.shape
                dup = 0 if sp is None or sp.rank == 0 else 1  # later shards also repeat their first frame
                buf, view = new_act(2 * tx - 1 + dup, 2 * hx, 2 * wx, cx)
                if view.is_contiguous():
                    upsample(x, out=view[:, dup:])
                else:
                    view[:, dup:] = upsample(x)
                if dup:
                    view[:, 0] = view[:, 1]
                ups += 1
                x, st = conv(f"s{si}.up", buf)
        buf = norm_act(x, st, "head.n")
        y, _ = conv("head.c", buf, stats=False)                    # [N, T', H', W', 3*8*8]
        return depth_to_space8(y)
