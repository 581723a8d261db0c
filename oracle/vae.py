"""Oracle: the causal conv3d VAE decoder on CPU (TEST INFRASTRUCTURE ONLY).

Parity unpinned: the reference repository has no convolutional VAE decoder (its fast path patches a
transformer decoder, custom_nodes/rapid_h3/vae_fast.py:430-437), so this file defines the arithmetic the
CUDA path is compared with: fp32 `conv3d` of bf16 operands with two zero frames before t = 0, bias and
residual added in fp32, one rounding to bf16 per layer; GroupNorm (32 groups, eps 1e-6) with fp64 statistics
of the stored bf16 tensor, then SiLU; nearest 2x upsampling in space and causal 2x in time.
`params` is the `cpu` dict of rapid_h3_b200.vae.VAEDecoder (weights [Cout, 27, Cin], tap = (dt*3+dh)*3+dw).
"""
import torch
import torch.nn.functional as F

GROUPS, EPS = 32, 1e-6


def conv3d_causal(x, w, bias=None, residual=None):
    """x [N,T,H,W,Cin] bf16 -> [N,T,H,W,Cout] bf16."""
    cout, _, cin = w.shape
    xf = F.pad(x.float().permute(0, 4, 1, 2, 3), (1, 1, 1, 1, 2, 0))
    wf = w.float().view(cout, 3, 3, 3, cin).permute(0, 4, 1, 2, 3)
    y = F.conv3d(xf, wf).permute(0, 2, 3, 4, 1)
    if bias is not None:
        y = y + bias.float()
    if residual is not None:
        y = y + residual.float()
    return y.to(torch.bfloat16)


def gn_silu(x, gamma, beta):
    n, c = x.shape[0], x.shape[-1]
    xd = x.double().reshape(n, -1, GROUPS, c // GROUPS)
    mean = xd.mean(dim=(1, 3), keepdim=True)
    var = (xd * xd).mean(dim=(1, 3), keepdim=True) - mean * mean
    rstd = torch.rsqrt(var.clamp_min(0) + EPS)
    t = ((x.float().reshape(xd.shape) - mean.float()) * rstd.float()).reshape(x.shape) * gamma.float() + beta.float()
    return (t / (1 + torch.exp(-t))).to(torch.bfloat16)


def upsample(x):
    y = x.repeat_interleave(2, 1)[:, 1:].repeat_interleave(2, 2).repeat_interleave(2, 3)
    return y.contiguous()


def decode(params, latent, widths=(512, 256, 128), blocks=2, trace=None):
    """latent [N,C,T,H,W] bf16 -> RGB [N,3,4T-3,32H,32W] bf16 (for three stages). `trace` (a list) receives one
    record (op, layer name, inputs, output) per layer, so that a caller can replay every layer on the oracle's own
    input."""
    p = params

    def rec(op, name, ins, y):
        if trace is not None:
            trace.append((op, name, ins, y))
        return y

    def conv(name, x, residual=None):
        return rec("conv", name, (x, residual), conv3d_causal(x, p[name + ".w"], p[name + ".b"], residual))

    def norm(name, x):
        return rec("gn", name, (x,), gn_silu(x, p[name + ".g"], p[name + ".be"]))

    n, c, t, h, w = latent.shape
    x = torch.zeros(n, t, h, w, 64, dtype=torch.bfloat16)
    x[..., :c] = latent.permute(0, 2, 3, 4, 1)
    x = conv("conv_in", x)
    for si in range(len(widths)):
        for bi in range(blocks):
            hdn = conv(f"s{si}.b{bi}.c1", norm(f"s{si}.b{bi}.n1", x))
            x = conv(f"s{si}.b{bi}.c2", norm(f"s{si}.b{bi}.n2", hdn), residual=x)
        if si + 1 < len(widths):
            x = conv(f"s{si}.up", rec("up", f"s{si}", (x,), upsample(x)))
    y = conv("head.c", norm("head.n", x))
    n, t2, h2, w2, _ = y.shape
    return y.view(n, t2, h2, w2, 3, 8, 8).permute(0, 4, 1, 2, 5, 3, 6).reshape(n, 3, t2, h2 * 8, w2 * 8)
