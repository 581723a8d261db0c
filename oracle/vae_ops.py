"""Oracle: fp16 ops of the VAE transformer decoder (TEST INFRASTRUCTURE ONLY).

Restates custom_nodes/rapid_h3/csrc/vae_ops.cu: `vae_out_quant` (:63-142: nan_to_num on load, the ConvRot
rotation in radix-4 stages of stride 1, 4, 16, 64, int8 with value / scale / quotient rounded through fp16),
the fp16 GEMM epilogues (:150-227: fp16((acc*xs)*ws + bias), then fp16(that * rscale + resid)) and the w1 + SwiGLU
epilogue (:228-345). The reference checks these against comfy-kitchen binaries (bench/vae_fast_test.py) that are
not available here and builds with approximate division: parity unpinned; this file defines the arithmetic with
IEEE operations.
"""
import torch

from .linear import int_mm


def nan_to_num_f16(x):
    """torch.nan_to_num for fp16 as fp32 values: NaN -> 0, +-inf -> +-65504 (vae_ops.cu:85-91)."""
    return torch.nan_to_num(x.float(), nan=0.0, posinf=65504.0, neginf=-65504.0)


def fht256(y):
    """fp32 [M, K] -> every group of 256 columns times H256, stage strides 1, 4, 16, 64 (vae_ops.cu:51-60,120-137);
    per stage y0 = .5(((x0+x1)+x2)-x3), y1 = .5(((x0+x1)-x2)+x3), y2 = .5(((x0-x1)+x2)+x3), y3 = .5(((-x0+x1)+x2)+x3)."""
    m, k = y.shape
    assert k % 256 == 0
    v = y.float().reshape(m, k // 256, 4, 4, 4, 4)  # digits d3, d2, d1, d0 of the column index in its group
    for axis in (5, 4, 3, 2):
        x0, x1, x2, x3 = v.unbind(axis)
        v = torch.stack([(((x0 + x1) + x2) - x3) * 0.5, (((x0 + x1) - x2) + x3) * 0.5,
                         (((x0 - x1) + x2) + x3) * 0.5, (((x1 - x0) + x2) + x3) * 0.5], dim=axis)
    return v.reshape(m, k)


def _sumsq_rows(x):
    """Row sums of squares in the kernel's order: the 8 values of a thread in order, an xor butterfly (16, 8, 4, 2, 1)
    over the 32 threads of a warp (= 256 columns), then the warps in order."""
    m, k = x.shape
    sq = (x * x).view(m, k // 256, 32, 8)
    acc = torch.zeros(m, k // 256, 32, dtype=torch.float32)
    for j in range(8):
        acc = acc + sq[..., j]
    lanes = torch.arange(32)
    for o in (16, 8, 4, 2, 1):
        acc = acc + acc[:, :, lanes ^ o]
    tot = acc[:, 0, 0]
    for w in range(1, k // 256):
        tot = tot + acc[:, w, 0]
    return tot


def act_prologue(x, act, weight=None, eps=0.0):
    """fp32 rows the quantizer rotates: "none" = nan_to_num(x); "rms_norm" = (x * r) * weight with
    r = 1 / sqrt(mean(x^2) + eps); "swiglu" = gate / (1 + e^-gate) * up of x = [gate | up] (the `act` argument of the
    quantizer called in custom_nodes/rapid_h3/vae_fast.py:71-85; its per-row arithmetic lives in a third-party binary
    that is not part of the reference repository, so this definition is this project's own: parity unpinned)."""
    from .quant import ieee_sqrt
    v = nan_to_num_f16(x)
    if act in (None, "none"):
        return v
    if act == "rms_norm":
        k = v.shape[1]
        r = 1.0 / ieee_sqrt(_sumsq_rows(v) / float(k) + torch.tensor(eps, dtype=torch.float32))
        y = v * r[:, None]
        return y * weight.float()[None, :] if weight is not None else y
    if act == "swiglu":
        k = v.shape[1] // 2
        g, u = v[:, :k], v[:, k:]
        return (g * (1.0 / (1.0 + torch.exp(-g)))) * u
    raise ValueError(act)


def quant_rows_f16(x, act="none", weight=None, eps=0.0):
    """x fp16 [M, K] -> (q int8 [M, K], scale fp32 [M]): prologue, rotation, the fp16-rounded division
    (vae_ops.cu:139-147)."""
    y = fht256(act_prologue(x, act, weight, eps))
    amax = y.abs().amax(dim=1)
    scale = (amax.clamp(max=65504.0) * torch.tensor(1.0 / 127.0, dtype=torch.float32)).clamp_min(1.0e-30)
    sh = scale.half().float()
    qf = (y.half().float() / sh[:, None]).half().float()
    # an all-zero row divides 0 by fp16(1e-30) = 0: NaN, which the device's fmaxf(-128, NaN) turns into -128
    # (the reference's clamp order, vae_ops.cu:143-145); dequantised with the 1e-30 scale that is still zero
    lo = torch.full_like(qf, -128.0)
    return torch.fmin(torch.fmax(qf.round(), lo), torch.full_like(qf, 127.0)).to(torch.int8), scale


def vae_out_quant(o):
    """o fp16 [B, H, S, D] head-major -> (q int8 [B*S, H*D], scale [B*S]); row (b, s) column head*D+d (vae_ops.cu:94-111)."""
    b, h, s, d = o.shape
    return quant_rows_f16(o.permute(0, 2, 1, 3).reshape(b * s, h * d))


def vae_gemm(xq, wq, xs, ws, bias, rscale=None, resid=None):
    """fp16 [M, N]: y1 = fp16((acc * xs) * ws + bias); with a residual fp16(float(y1) * rscale + resid)."""
    acc = int_mm(xq, wq).float()
    y = ((acc * xs.reshape(-1, 1)) * ws.reshape(1, -1) + bias.float()[None, :]).half()
    if resid is None:
        return y
    return (y.float() * rscale.float()[None, :] + resid.float()).half()


def ff_forward(x, norm_w, eps, w1q, w1s, b1, w2q, w2s, b2, residual, residual_scale, swiglu_epilogue=True):
    """The decoder's feed-forward block on fp16 x [M, K] (custom_nodes/rapid_h3/vae_fast.py:298-318):
    h = SwiGLU(w1(rms_norm(x))), out = w2(h) * residual_scale + residual. With `swiglu_epilogue` the SwiGLU is w1's
    GEMM epilogue (h rounded to fp16 once, :265-296), otherwise w1 writes fp16 [M, 2F] and the SwiGLU is the prologue
    of w2's quantizer. w1q / w1s / b1 are in the module's row order [gate | up]."""
    n = w1q.shape[0]
    xq, xs = quant_rows_f16(x, "rms_norm", norm_w, eps)
    if swiglu_epilogue:
        h = vae_gemm_swiglu(xq, interleave_rows(w1q, n), xs, interleave_rows(w1s, n), interleave_rows(b1, n))
        hq, hs = quant_rows_f16(h)
    else:
        h = vae_gemm(xq, w1q, xs, w1s, b1)
        hq, hs = quant_rows_f16(h, "swiglu")
    return vae_gemm(hq, w2q, hs, w2s, b2, residual_scale, residual)


def interleave_rows(t, n):
    """Row order of w1 for the SwiGLU epilogue: groups of 8 = [gate 4j..4j+3 | up 4j..4j+3] (vae_fast.py:259-263)."""
    h = n // 2
    idx = torch.arange(n).reshape(-1, 8)
    grp = torch.arange(n // 8)[:, None] * 4
    perm = torch.where(torch.arange(8)[None, :] < 4, grp + torch.arange(8)[None, :], h + grp + torch.arange(8)[None, :] - 4)
    assert perm.shape == idx.shape
    return t[perm.reshape(-1)]


def vae_gemm_swiglu(xq, wq_perm, xs, ws_perm, bias_perm):
    """fp16 [M, N/2] from interleaved rows: g, u = fp16((acc*xs)*ws + bias); fp16(g / (1 + e^-g) * u)."""
    acc = int_mm(xq, wq_perm).float()
    y = ((acc * xs.reshape(-1, 1)) * ws_perm.reshape(1, -1) + bias_perm.float()[None, :]).half().float()
    m, n = y.shape
    y = y.reshape(m, n // 8, 2, 4)
    g, u = y[:, :, 0], y[:, :, 1]
    return ((g / (1.0 + torch.exp(-g))) * u).reshape(m, n // 2).half()
