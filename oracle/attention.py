"""Oracle: attention pre-pass and INT8-QK / FP8-PV flash attention (TEST INFRASTRUCTURE ONLY).

What it follows in the reference:
  * RMSNorm + split-half partial 3-D RoPE: custom_nodes/rapid_h3/csrc/attn_int8.cu:217-260
    (bf16 re-rounding after the norm and after the rotation, pairs (i, i+48), table (cos,-sin,sin,cos));
  * K/V statistics: attn_int8.cu:82-109 (256-token chunks, then chunks in order);
  * operand quantizers: bench/attn_emulate.py:10-23 (`q8(x, 1, 64)`, `f8(x, 0)`) and :88, :101;
  * main loop: attn_int8.cu:1640-1759 (attn_fwd5: l summed before the e4m3 rounding, P.V in fp32,
    epilogue O/l*vscale+vmean) and bench/attn_emulate.py:33-65 (`run_fp8`).
Parity unpinned: the reference holds no vectors for this block-64 / e4m3-V variant (its production
kernel is per-token int8 with u8 P), and its rms/rope uses hardware .approx operations. This oracle
defines IEEE arithmetic with a fixed summation order, the exponent as the reference's magic-number
dequantisation t = fma(1.5*2^23 + s, c, (8 - M) - 1.5*2^23*c) (attn_int8.cu:22-27, :2365-2370), and
P = e4m3(2^t) with M the row maximum rounded up to an integer (so the result does not depend on the
key-tile order). On a fixed subset of the key columns (POLY_MASK) 2^t is a cubic polynomial, restated
here operation for operation.
"""
import math

import torch

from .quant import ieee_sqrt

D = 128
FP8 = torch.float8_e4m3fn
MAGIC = 12582912.0  # 1.5 * 2^23: the bias that turns int32 accumulator bits into floats

# Which exponentials are a cubic polynomial instead of exp2 (the kernel moves them from the special-function unit
# to the FMA pipe, the idea of the reference's softmax rebalancing, csrc/attn_cake/attn_cake.cuh:75-95): the 32
# columns of a chunk are taken four at a time, bit i of the mask selects columns 4i+2 and 4i+3 of group i.
POLY_MASK = 0x55
POLY_CLAMP = -60.0
POLY_C = [float.fromhex(h) for h in ("0x1.fff694p-1", "0x1.62f31ap-1", "0x1.f0ddf6p-3", "0x1.c3f6fp-5")]


def _fma32(a, b, c):
    """fp32 fused multiply-add of fp32 tensors: the product is exact in float64, one rounding of the sum to 53
    bits and one to 24 (a double rounding changes the result only on ties of measure zero)."""
    return (a.double() * b.double() + c.double()).float()


def exp2_poly(t):
    """2^t as the kernel's polynomial path computes it, operation for operation, for an fp32 tensor t."""
    tc = t.clamp_min(POLY_CLAMP)
    r = tc + torch.tensor(MAGIC, dtype=torch.float32)          # fp32 add: rint(t) in the low mantissa bits
    n = r - torch.tensor(MAGIC, dtype=torch.float32)           # exact
    f = tc - n                                                  # exact, in [-1/2, 1/2]
    c0, c1, c2, c3 = (torch.tensor(c, dtype=torch.float32) for c in POLY_C)
    q = _fma32(c3.expand_as(f), f, c2.expand_as(f))
    q = _fma32(q, f, c1.expand_as(f))
    q = _fma32(q, f, c0.expand_as(f))
    return torch.ldexp(q, n.to(torch.int32))                    # adds n to the exponent field


def poly_columns(lk):
    """bool [lk]: key columns whose exponential is the polynomial."""
    c = torch.arange(lk) % 32
    return (((POLY_MASK >> (c // 4)) & 1) == 1) & ((c % 4) >= 2)


def _bf(x):
    return x.to(torch.bfloat16).float()


def rmsnorm_rope(x, weight, eps, tab=None):
    """x bf16 [S,H,128] -> bf16 [S,H,128]. Sum of squares in the kernel's order: a lane holds 8 consecutive
    channels and adds their squares in order, then an xor butterfly (8, 4, 2, 1) over the 16 lanes of the row."""
    s, h, _ = x.shape
    xf = x.float()
    sq = (xf * xf).view(s, h, 16, 8)
    acc = torch.zeros(s, h, 16)
    for j in range(8):
        acc = acc + sq[..., j]
    lanes = torch.arange(16)
    for o in (8, 4, 2, 1):
        acc = acc + acc[..., lanes ^ o]
    ss = acc[..., 0]
    r = 1.0 / ieee_sqrt(ss / 128.0 + torch.tensor(eps, dtype=torch.float32))
    n = _bf((r[..., None] * xf) * weight.float())
    if tab is None:
        return n.to(torch.bfloat16)
    t = tab.float().view(s, 1, 48, 2, 2)
    a, b = n[..., :48], n[..., 48:96]
    o1 = _bf(a * t[..., 0, 0] + b * t[..., 0, 1])
    o2 = _bf(a * t[..., 1, 0] + b * t[..., 1, 1])
    return torch.cat([o1, o2, n[..., 96:]], -1).to(torch.bfloat16)


def chunked_column_sum(x, chunk=256, group=16):
    """Sum over dim 0 of fp32 x [L, ...] in the kernel's order: a 256-row chunk is 16 groups of 16 rows; rows of a
    group in order, then the groups in order, then the chunks in order."""
    l = x.shape[0]
    nchunk = (l + chunk - 1) // chunk
    pad = torch.zeros((nchunk * chunk,) + x.shape[1:], dtype=torch.float32)
    pad[:l] = x
    pad = pad.view((nchunk, chunk // group, group) + x.shape[1:])
    grp = torch.zeros((nchunk, chunk // group) + x.shape[1:], dtype=torch.float32)
    for i in range(group):
        grp = grp + pad[:, :, i]
    part = torch.zeros((nchunk,) + x.shape[1:], dtype=torch.float32)
    for g in range(chunk // group):
        part = part + grp[:, g]
    tot = torch.zeros(x.shape[1:], dtype=torch.float32)
    for c in range(nchunk):
        tot = tot + part[c]
    return tot


def kv_stats(k, v):
    """(kmean, vmean, vscale), each fp32 [H,128]."""
    l = k.shape[0]
    kf, vf = k.float(), v.float()
    kmean = chunked_column_sum(kf) / float(l)
    vmean = chunked_column_sum(vf) / float(l)
    am = torch.maximum(vf.amax(0) - vmean, vmean - vf.amin(0))
    return kmean, vmean, am.clamp_min(1e-8) / 448.0


def quant_block64(x, mean=None, pad=128):
    """x bf16 [L,H,128] -> (int8 [H,Lpad,128], fp32 [H,Lpad/64]); Lpad = L rounded up to `pad`."""
    l, h, _ = x.shape
    lpad = (l + pad - 1) // pad * pad
    xf = x.float()
    if mean is not None:
        xf = xf - mean[None]
    buf = torch.zeros(lpad, h, D)
    buf[:l] = xf
    blk = buf.view(lpad // 64, 64, h, D)
    s = blk.abs().amax(dim=(1, 3)).clamp_min(1e-8) / 127.0  # [nblk, H]
    q = (blk / s[:, None, :, None]).round().clamp(-127, 127).to(torch.int8)
    return q.view(lpad, h, D).permute(1, 0, 2).contiguous(), s.t().contiguous()


def quant_v(v, vmean, vscale):
    """e4m3 codes of (v - vmean)/vscale as uint8 [H,128,Lpad] (zero padded)."""
    l, h, _ = v.shape
    lpad = (l + 127) // 128 * 128
    y = ((v.float() - vmean[None]) / vscale[None]).clamp(-448, 448).to(FP8)
    out = torch.zeros(h, D, lpad, dtype=torch.uint8)
    out[:, :, :l] = y.view(torch.uint8).permute(1, 2, 0)
    return out


def prepass(q, k, v):
    kmean, vmean, vscale = kv_stats(k, v)
    q8, qs = quant_block64(q, pad=256)  # the main kernel works on pairs of 128-query tiles
    k8, ks = quant_block64(k, kmean)
    return dict(q8=q8, qs=qs, k8=k8, ks=ks, vt=quant_v(v, vmean, vscale), vscale=vscale, vmean=vmean, kmean=kmean,
                lq=q.shape[0], lk=k.shape[0])


def attention_pre(pre, scale=None, heads=None, rows=None):
    """bf16 [Lq(or len(rows)), len(heads), 128] from pre-pass operands; `heads` / `rows` select a subset."""
    lq, lk = pre["lq"], pre["lk"]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    sl2 = torch.tensor(float(scale) * 1.4426950408889634, dtype=torch.float32)
    heads = list(range(pre["q8"].shape[0])) if heads is None else list(heads)
    rows = torch.arange(lq) if rows is None else torch.as_tensor(rows)
    out = torch.empty(len(rows), len(heads), D, dtype=torch.bfloat16)
    for hi, h in enumerate(heads):
        kf = pre["k8"][h, :lk].float()
        vf = pre["vt"][h, :, :lk].view(FP8).float().t().contiguous()  # [Lk, 128]
        kc = pre["ks"][h][torch.arange(lk) // 64]                      # per-key scale
        pcols = poly_columns(lk)
        for r0 in range(0, len(rows), 512):
            rr = rows[r0:r0 + 512]
            s = pre["q8"][h, rr].float() @ kf.t()                      # exact: |s| < 2^24
            c = (pre["qs"][h][rr // 64] * sl2)[:, None] * kc[None, :]  # fp32: (qs * sl2) * ks
            b = MAGIC * c                                              # fp32, one rounding
            sf = (s + MAGIC).double()                                  # exact float 1.5*2^23 + s
            # t = fma(sf, c, off): the product is exact in float64 and so is the sum (48 + 24 bits)
            m = torch.ceil((sf * c.double() - b.double()).float().amax(1, keepdim=True))
            off = (8.0 - m) - b
            t = (sf * c.double() + off.double()).float()
            p = torch.where(pcols[None, :], exp2_poly(t), torch.exp2(t))
            l = p.sum(1, keepdim=True)
            o = p.to(FP8).float() @ vf
            y = (o / l) * pre["vscale"][h][None] + pre["vmean"][h][None]
            out[r0:r0 + 512, hi] = y.to(torch.bfloat16)
    return out


def attention(q, k, v, scale=None, heads=None, rows=None):
    return attention_pre(prepass(q, k, v), scale, heads, rows)


def attention_fp32(q, k, v, scale=None, heads=None, rows=None):
    """Unquantized fp32 softmax attention (the yardstick of bench/attn_cake.py:38-40)."""
    lq, h, _ = q.shape
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    heads = list(range(h)) if heads is None else list(heads)
    rows = torch.arange(lq) if rows is None else torch.as_tensor(rows)
    out = torch.empty(len(rows), len(heads), D)
    for hi, hh in enumerate(heads):
        kf, vf = k[:, hh].float(), v[:, hh].float()
        for r0 in range(0, len(rows), 1024):
            rr = rows[r0:r0 + 1024]
            out[r0:r0 + 1024, hi] = torch.softmax((q[rr, hh].float() @ kf.t()) * scale, -1) @ vf
    return out
