"""Oracle: fused-prologue row quantizers (TEST INFRASTRUCTURE ONLY).

Follows custom_nodes/rapid_h3/triton_fp8.py:128-148 (`_load_act` prologues) and :165-172 (RMS
statistics), with and without the H256 rotation (:70-112). The reference pins these only by a
mismatch fraction against an fp32 expression (bench/rot_test.py:42-51), so the summation order of the
sum of squares and of the rotation butterflies is defined here and mirrored by the CUDA kernel:
parity unpinned beyond that reference expression.
"""
import numpy as np
import torch

from .linear import ROT_GROUP, convrot_matmul, quantize_rows, regular_hadamard, rotate256  # noqa: F401


def ieee_sqrt(t):
    """Correctly rounded fp32 square root (torch's vectorised CPU sqrt is not; numpy's is)."""
    return torch.from_numpy(np.sqrt(t.contiguous().numpy()))


def launch_shape(k):
    """(threads per row, 8-element chunks per thread) the kernel uses for a row of K elements."""
    nchunk = k // 8
    for limit, t, cpt in ((128, 128, 1), (256, 128, 2), (512, 128, 4), (1024, 128, 8), (2048, 256, 8),
                          (4096, 512, 8), (8192, 1024, 8)):
        if nchunk <= limit:
            return t, cpt
    raise ValueError(k)


def fixed_order_sumsq(x):
    """Sum of squares of each row of x (fp32 [M,K]) in the kernel's order: a thread adds the squares
    of its chunks t, t+T, ... element by element, lanes combine in an xor butterfly (16, 8, 4, 2, 1),
    warps are added in index order."""
    m, k = x.shape
    t, cpt = launch_shape(k)
    sq = torch.zeros(m, cpt * t * 8, dtype=torch.float32)
    sq[:, :k] = x * x
    sq = sq.view(m, cpt, t, 8)
    acc = torch.zeros(m, t, dtype=torch.float32)
    for i in range(cpt):
        for j in range(8):
            acc = acc + sq[:, i, :, j]
    v = acc.view(m, t // 32, 32)
    lanes = torch.arange(32)
    for o in (16, 8, 4, 2, 1):
        v = v + v[:, :, lanes ^ o]
    v = v[:, :, 0]
    tot = v[:, 0]
    for w in range(1, t // 32):
        tot = tot + v[:, w]
    return tot


def norm_mod(x, weight, eps, idx, shift, scale):
    """fp32 rms_norm(x) * w * (1 + scale[idx]) + shift[idx], each operation rounded separately."""
    xf = x.float()
    k = xf.shape[1]
    ss = fixed_order_sumsq(xf)
    rstd = 1.0 / ieee_sqrt(ss / k + torch.tensor(eps, dtype=torch.float32))
    y = xf * rstd[:, None]
    if weight is not None:
        y = y * weight.float()[None, :]
    r = idx.long()
    return y * (1.0 + scale[r]) + shift[r]


def _quant_fp32_rows(y):
    amax = y.abs().amax(dim=-1, keepdim=True)
    s = (amax / 127.0).clamp_min(1e-12)
    return (y / s).round().clamp(-127, 127).to(torch.int8), s


def norm_mod_quant_rows_i8(x, weight, eps, idx, shift, scale):
    return _quant_fp32_rows(norm_mod(x, weight, eps, idx, shift, scale))


def swiglu_quant_rows_i8(x):
    """x [M, 2F] -> int8 of silu(x[:, :F]) * x[:, F:] (triton_fp8.py:137-139)."""
    f = x.shape[1] // 2
    g, u = x[:, :f].float(), x[:, f:].float()
    return _quant_fp32_rows(g * (1.0 / (1.0 + torch.exp(-g))) * u)


def quant_heads_i8(o):
    """o [H, M, 128] head-major -> rows [M, H*128] (triton_fp8.py:134-135), then the plain quantizer."""
    h, m, d = o.shape
    return quantize_rows(o.permute(1, 0, 2).reshape(m, h * d), "int8_rowwise")


def rot_quant_rows_i8(x):
    """int8 of rotate(x) with per-row scales (triton_fp8.py:424-426)."""
    return _quant_fp32_rows(rotate256(x.float()))


def rot_quant_heads_i8(o):
    """o [H, M, 128] head-major -> rows [M, H*128], rotated and quantized (triton_fp8.py:429-434)."""
    h, m, d = o.shape
    return _quant_fp32_rows(rotate256(o.permute(1, 0, 2).reshape(m, h * d).float()))


def swiglu_rot_quant_rows_i8(x):
    """int8 of rotate(silu(gate) * up) (triton_fp8.py:437-439)."""
    f = x.shape[1] // 2
    g, u = x[:, :f].float(), x[:, f:].float()
    return _quant_fp32_rows(rotate256(g * (1.0 / (1.0 + torch.exp(-g))) * u))


def norm_mod_rot_quant_rows_i8(x, weight, eps, idx, shift, scale):
    """int8 of rotate(rms_norm(x) * w * (1 + scale[idx]) + shift[idx]) (triton_fp8.py:442-446)."""
    return _quant_fp32_rows(rotate256(norm_mod(x, weight, eps, idx, shift, scale)))


def rot_residual_quant_rows_i8(x, q1, s1, rows):
    """Second pass of the text encoder's int8_rot linear on rows `rows` (te_quant.py:100-103):
    r = rotate(x[rows]) - q1[rows] * s1[rows] in fp32 (x fp32), then the int8 row quantizer."""
    r = rotate256(x[rows].float()) - q1[rows].float() * s1[rows].reshape(-1, 1)
    return _quant_fp32_rows(r)
