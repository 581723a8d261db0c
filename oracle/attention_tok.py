"""Oracle: the token-scaled INT8 attention (per-token Q/K after a 128-point Hadamard rotation, int8 V, 8-bit P
against each key tile's own maximum, per-tile fold). TEST INFRASTRUCTURE ONLY.

What it follows in the reference (the numerics of its production attention, configs 80 / 90 / 94 / 190 / 194):
custom_nodes/rapid_h3/csrc/README.md "What it computes" (pre-pass: K/V statistics, per-token Q/K with `hadamard128`
and mean-smoothed K, per-channel mean-smoothed int8 V; main kernel: P as u8 relative to each tile's own row maximum
`2^(t*c - tm*c + log2 255)`, `ts = 2^(tm - m)`, row sums from the quantized P, epilogue `O / l * v_scale + v_mean`),
custom_nodes/rapid_h3/csrc/attn_cake/DESIGN.md section 2 (`l = fma(ts, rs, l*a)`, the per-tile fold of the int32
P.V accumulator into the fp32 output).

Parity unpinned: the reference's kernels are CUDA only (no CPU emulation of this variant exists in its tree, and its
kernels use hardware .approx operations), so no golden vector can be produced here. This file fixes IEEE arithmetic
in a stated order; the device path must reproduce the operands bit for bit and the output within 1e-3 rel-L2
(the device's exp2 is the hardware approximation).

Definitions:
  rotation   unnormalised fast Walsh-Hadamard transform over the 128 channels, butterflies (a, b) -> (a+b, a-b) over
             channel distance 1, 2, 4, ..., 64 in that order, each add a correctly rounded fp32 add
  Q, K       code = rint(y / s), s = max(amax(y), 1e-8) / 127 per token; K is rotated after its channel mean (the
             fixed-order statistics of oracle.attention.kv_stats) is subtracted
  key tile   128 keys: multiplier ks_j / 128 (the rotation scales Q.K^T by 128), bias 0, or -inf for padding keys
  V          code = rint((v - vmean) / vscale), vscale = max(max(vmax - vmean, vmean - vmin), 1e-8) / 127
  main loop  per 128-key tile: t = s * mult + bias; tm = max t; tmc = tm * c (c = qs * softmax_scale * log2 e);
             m' = max(m, tmc); a = 2^(m - m'); ts = 2^(tmc - m'); P = rint(2^(fma(t, c, log2 255 - tmc)));
             l = fma(ts, sum P, l * a); O = fma(ts, P . V8, O * a); out = bf16(fma(O / l, vscale, vmean))
"""
import math

import torch

from . import attention as oa

D = 128
LOG2_255 = torch.tensor(7.99435343685886, dtype=torch.float32)


def hadamard128(x):
    """Unnormalised Walsh-Hadamard transform of the last dimension (128), fp32, butterfly distances 1, 2, ..., 64."""
    y = x.float().clone()
    shape = y.shape
    d = 1
    while d < D:
        y = y.reshape(shape[:-1] + (D // (2 * d), 2, d))
        a, b = y[..., 0, :], y[..., 1, :]
        y = torch.stack([a + b, a - b], dim=-2).reshape(shape)
        d *= 2
    return y


def quant_tok(x, mean=None, pad=128):
    """x bf16 [L,H,128] -> (int8 [H,Lpad,128], fp32 scales [H,Lpad]); padding rows: zero codes, scale 1e-8/127."""
    l, h, _ = x.shape
    lpad = (l + pad - 1) // pad * pad
    xf = x.float()
    if mean is not None:
        xf = xf - mean[None]
    y = hadamard128(xf)
    s = y.abs().amax(-1).clamp_min(1e-8) / 127.0                    # [L, H]
    q = (y / s[..., None]).round().clamp(-127, 127).to(torch.int8)
    q8 = torch.zeros(h, lpad, D, dtype=torch.int8)
    q8[:, :l] = q.permute(1, 0, 2)
    sc = torch.full((h, lpad), 1e-8, dtype=torch.float32) / 127.0
    sc[:, :l] = s.t()
    return q8, sc


def prepass(q, k, v):
    kmean, vmean, vs448 = oa.kv_stats(k, v)
    vf = v.float()
    am = torch.maximum(vf.amax(0) - vmean, vmean - vf.amin(0))
    vscale = am.clamp_min(1e-8) / 127.0
    q8, qs = quant_tok(q, pad=256)
    k8, ks = quant_tok(k, kmean)
    lk = k.shape[0]
    h, lkp = ks.shape
    ksb = torch.zeros(h, lkp // 128, 2, 128, dtype=torch.float32)
    mult = ks * 0.0078125
    mult[:, lk:] = 0.0
    bias = torch.zeros(h, lkp)
    bias[:, lk:] = -math.inf
    ksb[:, :, 0] = mult.view(h, lkp // 128, 128)
    ksb[:, :, 1] = bias.view(h, lkp // 128, 128)
    v8 = ((vf - vmean[None]) / vscale[None]).round().clamp(-127, 127).to(torch.int8)
    vt = torch.zeros(h, D, lkp, dtype=torch.int8)
    vt[:, :, :lk] = v8.permute(1, 2, 0)
    return dict(q8=q8, qs=qs, k8=k8, ksb=ksb, vt=vt, vscale=vscale, vmean=vmean, kmean=kmean, lq=q.shape[0], lk=lk)


def attention_pre(pre, scale=None, heads=None, rows=None):
    """bf16 [len(rows), len(heads), 128] from the operands of prepass()."""
    lq, lk = pre["lq"], pre["lk"]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    sl2 = torch.tensor(float(scale) * 1.4426950408889634, dtype=torch.float32)
    heads = list(range(pre["q8"].shape[0])) if heads is None else list(heads)
    rows = torch.arange(lq) if rows is None else torch.as_tensor(rows)
    out = torch.empty(len(rows), len(heads), D, dtype=torch.bfloat16)
    ntile = (lk + 127) // 128
    for hi, h in enumerate(heads):
        for r0 in range(0, len(rows), 512):
            rr = rows[r0:r0 + 512]
            n = len(rr)
            c = (pre["qs"][h][rr] * sl2)[:, None]                              # fp32 [n, 1]
            qf = pre["q8"][h, rr].double()
            m = torch.full((n, 1), -math.inf, dtype=torch.float32)
            l = torch.zeros(n, 1, dtype=torch.float32)
            o = torch.zeros(n, D, dtype=torch.float32)
            for j in range(ntile):
                kt = pre["k8"][h, j * 128:(j + 1) * 128].double()
                s = (qf @ kt.t()).float()                                      # exact integers
                mult, bias = pre["ksb"][h, j, 0][None], pre["ksb"][h, j, 1][None]
                t = oa._fma32(s, mult.expand_as(s), bias.expand_as(s))
                tm = t.amax(1, keepdim=True)
                tmc = tm * c
                m_new = torch.maximum(m, tmc)
                a, ts = torch.exp2(m - m_new), torch.exp2(tmc - m_new)
                off = LOG2_255 - tmc
                p = torch.exp2(oa._fma32(t, c.expand_as(t), off.expand_as(t))).round().clamp(0, 255)
                rs = p.sum(1, keepdim=True)                                    # exact (<= 128 * 255)
                l = oa._fma32(ts, rs, l * a)
                acc = (p.double() @ pre["vt"][h, :, j * 128:(j + 1) * 128].double().t()).float()  # exact integers
                o = oa._fma32(ts.expand_as(o), acc, o * a)
                m = m_new
            y = oa._fma32(o * (1.0 / l), pre["vscale"][h][None].expand_as(o), pre["vmean"][h][None].expand_as(o))
            out[r0:r0 + 512, hi] = y.to(torch.bfloat16)
    return out


def attention(q, k, v, scale=None, heads=None, rows=None):
    return attention_pre(prepass(q, k, v), scale, heads, rows)
