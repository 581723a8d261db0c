"""Row-wise-scaled W8A8 GEMMs; same names and argument meaning as the reference's
custom_nodes/rapid_h3/cutlass_fp8.py (`int8_gemm`, `fp8_gemm`, `int8_gemm_gated_residual`,
`swiglu_perm`, `int8_gemm_swiglu`). `config` (the reference's CUTLASS tile id) and `fast_accum`
are accepted and ignored: there is one tcgen05 kernel per epilogue.
"""
import torch

from . import _lib


def _check(xq, xs, wq, ws, dtype):
    _lib.require_cuda(xq, xs, wq, ws)
    if xq.dtype != dtype or wq.dtype != dtype:
        raise RuntimeError(f"expected {dtype} codes, got {xq.dtype} / {wq.dtype}")
    if xq.ndim != 2 or wq.ndim != 2 or xq.shape[1] != wq.shape[1]:
        raise RuntimeError(f"shape mismatch: xq {tuple(xq.shape)} wq {tuple(wq.shape)}")
    if xq.stride(1) != 1 or not wq.is_contiguous():
        raise RuntimeError("xq needs unit column stride and wq must be contiguous")
    m, k = xq.shape
    n = wq.shape[0]
    xs, ws = xs.reshape(-1), ws.reshape(-1)
    if xs.numel() != m or ws.numel() != n or xs.dtype != torch.float32 or ws.dtype != torch.float32:
        raise RuntimeError("xs / ws must be fp32 with M / N elements")
    return m, n, k, xs.contiguous(), ws.contiguous()


def _gemm(xq, xs, wq, ws, bias, kind, dtype, acc_dump=None, out=None):
    m, n, k, xs, ws = _check(xq, xs, wq, ws, dtype)
    if bias is not None:
        _lib.require_cuda(bias)
        if bias.dtype != torch.bfloat16 or bias.numel() != n:
            raise RuntimeError("bias must be bf16 with N elements")
        bias = bias.contiguous()
    if out is None:
        out = torch.empty((m, n), device=xq.device, dtype=torch.bfloat16)
    _lib.call("rh3_gemm_w8a8", xq.data_ptr(), xq.stride(0), wq.data_ptr(), xs.data_ptr(), ws.data_ptr(),
              _lib.ptr(bias), m, n, k, kind, out.data_ptr(), out.stride(0), _lib.ptr(acc_dump), _lib.stream())
    return out


def int8_gemm(xq, xs, wq, ws, bias=None, config=2, acc_dump=None, out=None):
    """W8A8 int8 GEMM with row-wise scales: bf16 [M, N] = ((acc * xs[m]) * ws[n]) + bias[n], acc the exact int32
    dot product of row m of xq [M, K] with row n of wq [N, K]. xs / ws are fp32 with M / N elements in any shape.
    Extras of this library: `acc_dump` (int32 [M, N]) receives the raw accumulators for parity checks, `out`
    (bf16, unit column stride) is written instead of a new tensor. `config` is accepted and ignored."""
    return _gemm(xq, xs, wq, ws, bias, _lib.KIND_I8, torch.int8, acc_dump, out)


def fp8_gemm(xq, xs, wq, ws, bias=None, config=2, fast_accum=True, acc_dump=None, out=None):
    """The same GEMM on e4m3 codes with fp32 accumulation (`acc_dump` is then fp32 bits). `config` and
    `fast_accum` are accepted and ignored: the tensor core accumulates in fp32 either way."""
    return _gemm(xq, xs, wq, ws, bias, _lib.KIND_F8, torch.float8_e4m3fn, acc_dump, out)


def int8_gemm_gated_residual(xq, xs, wq, ws, gate, resid, config=6):
    """In place: resid[m, n] = bf16(fma(bf16((acc * xs[m]) * ws[n]), gate[n], resid[m, n])), which is what
    `resid.addcmul_(y, gate)` gives for the bf16 GEMM result y. `resid` may be a row slice of a larger tensor (any
    row stride, unit column stride); M = 0 does nothing. Returns `resid`."""
    m, n, k, xs, ws = _check(xq, xs, wq, ws, torch.int8)
    _lib.require_cuda(gate, resid)
    if gate.dtype != torch.bfloat16 or gate.numel() != n or not gate.is_contiguous():
        raise RuntimeError("gate must be contiguous bf16 with N elements")
    if resid.dtype != torch.bfloat16 or resid.shape != (m, n) or resid.stride(1) != 1:
        raise RuntimeError("resid must be bf16 [M,N] with unit column stride")
    _lib.call("rh3_gemm_w8a8_gated_residual", xq.data_ptr(), xq.stride(0), wq.data_ptr(), xs.data_ptr(),
              ws.data_ptr(), gate.data_ptr(), resid.data_ptr(), resid.stride(0) if m else n, m, n, k, _lib.KIND_I8,
              _lib.stream())
    return resid


def swiglu_perm(n2, device):
    """Index tensor [n2] that re-orders the rows of an fc1 weight stored as F gate rows followed by F up rows
    (n2 = 2F, F a multiple of 4) into runs of eight: four gate rows, then the four up rows they multiply. The
    SwiGLU epilogue finds gate and up of an output column in the same 8-column group of its accumulator tile that
    way. Entry 8j + i is 4j + i for i < 4 and F + 4j + (i - 4) otherwise (layout contract of the reference's
    fused fc1 GEMM, cutlass_fp8.py:55-62)."""
    f = n2 // 2
    if n2 != 2 * f or f % 4:
        raise RuntimeError("swiglu_perm: the hidden width must be a multiple of 4")
    rows = torch.arange(n2, device=device).view(2, f // 4, 4)   # [gate | up] x groups of four
    return rows.transpose(0, 1).reshape(-1)


def int8_gemm_swiglu(xq, xs, wq_perm, ws_perm, config=6, out=None):
    """fc1 and SwiGLU in one kernel: with g, u = bf16((acc * xs) * ws) of a gate row and its up row,
    out [M, N/2] = bf16(g / (1 + exp(-g)) * u). `wq_perm` / `ws_perm` are the weight codes and scales re-ordered with
    swiglu_perm (N = 2F rows, a multiple of 16)."""
    m, n, k, xs, ws = _check(xq, xs, wq_perm, ws_perm, torch.int8)
    if n % 16:
        raise RuntimeError("int8_gemm_swiglu: N must be a multiple of 16")
    if out is None:
        out = torch.empty((m, n // 2), device=xq.device, dtype=torch.bfloat16)
    _lib.call("rh3_gemm_w8a8_swiglu", xq.data_ptr(), xq.stride(0), wq_perm.data_ptr(), xs.data_ptr(), ws.data_ptr(),
              m, n, k, _lib.KIND_I8, out.data_ptr(), out.stride(0), _lib.stream())
    return out
