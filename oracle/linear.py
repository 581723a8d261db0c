"""Oracle: per-row quantizers and the row-wise-scaled W8A8 linear (TEST INFRASTRUCTURE ONLY).

Follows the reference's PyTorch emulation: custom_nodes/rapid_h3/kernels.py:52-72
(quantize_weight), :75-82 (quantize_rows), :129-137 (linear), the H256 ConvRot rotation of
custom_nodes/rapid_h3/triton_fp8.py:70-92 (as radix-4 butterflies with a fixed rounding order; the
reference's own expression is a matrix product whose summation order is not defined, so rotated codes are
pinned only by a mismatch fraction: parity unpinned for `int8_rot` beyond that), and the fused epilogues of
custom_nodes/rapid_h3/csrc/fp8_rowwise.cu:294-304 (dequant + bias), :333-336 (gated residual),
:74-93 (SwiGLU store) with the row order of custom_nodes/rapid_h3/cutlass_fp8.py:55-62.
"""
import torch

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0
ROT_GROUP = 256


def regular_hadamard(n):
    """Kronecker powers of the regular 4x4 Hadamard matrix, orthonormal (triton_fp8.py:70-82), fp64."""
    h4 = torch.tensor([[1, 1, 1, -1], [1, 1, -1, 1], [1, -1, 1, 1], [-1, 1, 1, 1]], dtype=torch.float64)
    h = h4
    while h.shape[0] < n:
        h = torch.kron(h, h4)
    return h / n ** 0.5


def convrot_matmul(x):
    """x @ blockdiag(H256)^T as one fp64 matrix product (the expression of triton_fp8.py:88-92);
    the yardstick the butterfly below is compared with."""
    m, k = x.shape
    return (x.double().reshape(-1, ROT_GROUP) @ regular_hadamard(ROT_GROUP).T).reshape(m, k)


def rotate256(y):
    """fp32 y [M, K] -> y @ blockdiag(H256)^T as four radix-4 stages over the base-4 digits of the
    channel index inside its group of 256, lowest digit first, then one multiplication by 1/16. With
    a = e0+e1, b = e2+e3, c = e0-e1, d = e2-e3 a stage maps the four values that differ in that digit to
    (a+d, a-d, b+c, b-c): H4 with every rounding fixed, the order the CUDA kernel uses."""
    m, k = y.shape
    assert k % ROT_GROUP == 0
    v = y.float().reshape(m, k // ROT_GROUP, 4, 4, 4, 4)
    for axis in (5, 4, 3, 2):
        e0, e1, e2, e3 = v.unbind(axis)
        a, b, c, d = e0 + e1, e2 + e3, e0 - e1, e2 - e3
        v = torch.stack([a + d, a - d, b + c, b - c], dim=axis)
    return (v * 0.0625).reshape(m, k)


def quantize_rows(x, mode):
    """(q, s[M,1]): kernels.py:75-82. int8: s = max(amax/127, 1e-12), q = clamp(round(x/s), +-127)."""
    if mode == "int8_rot":  # kernels.py:115-117: rotate, then the int8 row quantizer
        x, mode = rotate256(x.float()), "int8_rowwise"
    if mode == "fp8_tensor":  # kernels.py:126-127: one scale for the tensor, repeated per row for the row-scaled product
        s = (x.abs().amax().float() / FP8_MAX).clamp_min(1e-12)
        return (x.float() / s).clamp(-FP8_MAX, FP8_MAX).to(FP8), s.reshape(1, 1).expand(x.shape[0], 1).contiguous()
    amax = x.abs().amax(dim=-1, keepdim=True).float()
    if mode == "int8_rowwise":
        s = (amax / 127.0).clamp_min(1e-12)
        return (x.float() / s).round().clamp(-127, 127).to(torch.int8), s
    if mode == "fp8_rowwise":
        s = (amax / FP8_MAX).clamp_min(1e-12)
        return (x.float() / s).clamp(-FP8_MAX, FP8_MAX).to(FP8), s
    raise ValueError(mode)


def quantize_weight(w, mode):
    """(q [N,K], scale [1,N]): kernels.py:52-72, row-wise modes."""
    w = w.float()
    if mode == "int8_rot":  # kernels.py:58-60: W . blockdiag(H256)^T, then int8 per output row
        w, mode = rotate256(w), "int8_rowwise"
    if mode == "fp8_tensor":  # kernels.py:63-65 (the scalar scale repeated per output row)
        s = (w.abs().amax() / FP8_MAX).clamp_min(1e-12)
        return (w / s).clamp(-FP8_MAX, FP8_MAX).to(FP8), s.reshape(1, 1).expand(1, w.shape[0]).contiguous()
    if mode == "fp8_rowwise":
        s = (w.abs().amax(dim=1, keepdim=True) / FP8_MAX).clamp_min(1e-12)
        return (w / s).clamp(-FP8_MAX, FP8_MAX).to(FP8), s.t().contiguous()
    if mode == "int8_rowwise":
        s = (w.abs().amax(dim=1, keepdim=True) / 127.0).clamp_min(1e-12)
        return (w / s).round().clamp(-127, 127).to(torch.int8), s.t().contiguous()
    raise ValueError(mode)


def int_mm(xq, wq):
    """Exact int32 accumulators of xq [M,K] int8 times wq [N,K] int8 (transposed)."""
    m, k = xq.shape
    if m > 16 and k % 8 == 0 and wq.shape[0] % 8 == 0:
        try:
            return torch._int_mm(xq.contiguous(), wq.t())
        except RuntimeError:
            pass
    # float64 products of 8-bit integers are exact far beyond K = 2^20
    return (xq.double() @ wq.double().t()).to(torch.int32)


def fp8_mm(xq, wq):
    """fp32 accumulators of e4m3 operands (products exact in fp32; summation order is free)."""
    return xq.float() @ wq.float().t()


def dequant(acc, xs, ws, bias=None):
    """bf16(((acc * xs[m]) * ws[n]) + bias[n]): fp8_rowwise.cu:294-304; kernels.py:137 without bias."""
    y = acc.float() * xs.reshape(-1, 1) * ws.reshape(1, -1)
    if bias is not None:
        y = y + bias.float().reshape(1, -1)
    return y.to(torch.bfloat16)


def linear(x, wq, ws, mode, bias=None):
    """x bf16 [M,K] through quantize_rows + the W8A8 product + dequant (kernels.py:129-137)."""
    xq, xs = quantize_rows(x, mode)
    acc = int_mm(xq, wq) if mode in ("int8_rowwise", "int8_rot") else fp8_mm(xq, wq)
    return dequant(acc, xs, ws, bias)


def gated_residual(acc, xs, ws, gate, resid):
    """bf16(fma(bf16((acc*xs)*ws), gate[n], resid)): fp8_rowwise.cu:333-336 (= x.addcmul_(y, gate)).
    The fused multiply-add is evaluated in float64, where the bf16 x bf16 product is exact."""
    y = dequant(acc, xs, ws)
    return (y.double() * gate.double().reshape(1, -1) + resid.double()).float().to(torch.bfloat16)


def swiglu_perm(n2):
    """cutlass_fp8.py:55-62: rows [gate | up] -> groups of 8 = [gate 4j..4j+3 | up 4j..4j+3]."""
    f = n2 // 2
    j = torch.arange(0, f, 4)
    blk = torch.arange(4)
    return torch.stack([j[:, None] + blk, f + j[:, None] + blk], dim=1).reshape(-1)


def swiglu_epilogue(acc, xs, ws_perm):
    """h[M, N/2] = bf16(silu(bf16 g) * bf16 u) from interleaved columns: fp8_rowwise.cu:74-93."""
    y = dequant(acc, xs, ws_perm).float()
    m, n = y.shape
    y = y.view(m, n // 8, 2, 4)
    g, u = y[:, :, 0], y[:, :, 1]
    return (g / (1.0 + torch.exp(-g)) * u).reshape(m, n // 2).to(torch.bfloat16)
