"""Per-token activation quantizers; same names and argument meaning as the reference's
custom_nodes/rapid_h3/triton_fp8.py (`quant_rows`, `quant_rows_i8`, `rot_quant_rows_i8`,
`rot_quant_heads_i8`, `swiglu_rot_quant_rows_i8`, `norm_mod_rot_quant_rows_i8`), each a single
CUDA kernel launch through the C ABI.

The `rot_*` functions apply the H256 ConvRot rotation (groups of 256 channels) by default, as in the
reference; `rotate=False` gives the un-rotated `int8_rowwise` recipe through the same kernels.
"""
import torch

from . import _lib

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0
ROT_GROUP = 256


def _check_rows(x):
    _lib.require_cuda(x)
    assert x.ndim == 2 and x.stride(1) == 1, "expected a 2-D tensor with unit column stride"
    if x.dtype != torch.bfloat16:
        raise RuntimeError(f"expected bf16 activations, got {x.dtype}")


def quant_rows_i8(x):
    """Per-row symmetric INT8: s = amax / 127, q = rint(x / s). Returns (q int8 [M,K], s fp32 [M,1])."""
    _check_rows(x)
    m, k = x.shape
    q = torch.empty((m, k), device=x.device, dtype=torch.int8)
    s = torch.empty((m, 1), device=x.device, dtype=torch.float32)
    _lib.call("rh3_quant_rows_i8", x.data_ptr(), x.stride(0), m, k, q.data_ptr(), q.stride(0), s.data_ptr(),
              _lib.stream())
    return q, s


def quant_rows(x):
    """Per-row FP8 e4m3: s = amax / 448. Returns (q fp8 [M,K], s fp32 [M,1])."""
    _check_rows(x)
    m, k = x.shape
    q = torch.empty((m, k), device=x.device, dtype=FP8)
    s = torch.empty((m, 1), device=x.device, dtype=torch.float32)
    _lib.call("rh3_quant_rows_fp8", x.data_ptr(), x.stride(0), m, k, q.data_ptr(), q.stride(0), s.data_ptr(),
              _lib.stream())
    return q, s


def quant_tensor(x):
    """FP8 e4m3 with one scale for the whole tensor: s = max|x| / 448. Returns (q fp8 [M,K], s fp32 [M,1]) with the
    same s in every row, so the pair feeds the row-scaled GEMM as it is."""
    _check_rows(x)
    m, k = x.shape
    q = torch.empty((m, k), device=x.device, dtype=FP8)
    s = torch.empty((m, 1), device=x.device, dtype=torch.float32)
    amax = torch.empty(1, device=x.device, dtype=torch.float32)
    _lib.call("rh3_quant_tensor_fp8", x.data_ptr(), x.stride(0), m, k, q.data_ptr(), q.stride(0), s.data_ptr(),
              amax.data_ptr(), _lib.stream())
    return q, s


def _rot_width(k):
    if k % ROT_GROUP:
        raise RuntimeError(f"the rotated width {k} must be a multiple of {ROT_GROUP}")


def rot_quant_rows_i8(x, rotate=True):
    """int8(x @ blockdiag(H256)^T) with per-row scales (`rotate=False`: plain quant_rows_i8)."""
    if not rotate:
        return quant_rows_i8(x)
    _check_rows(x)
    m, k = x.shape
    _rot_width(k)
    q = torch.empty((m, k), device=x.device, dtype=torch.int8)
    s = torch.empty((m, 1), device=x.device, dtype=torch.float32)
    _lib.call("rh3_rot_quant_rows_i8", x.data_ptr(), x.stride(0), m, k, q.data_ptr(), q.stride(0), s.data_ptr(),
              _lib.stream())
    return q, s


def rot_quant_heads_i8(o, rotate=True):
    """o [H, M, 128] bf16 head-major (attention output) -> (q int8 [M, H*128], s [M,1]), read in place."""
    if rotate:
        return quant_groups_i8(o, rotate=True)
    _lib.require_cuda(o)
    assert o.ndim == 3 and o.shape[2] == 128 and o.stride(2) == 1 and o.stride(1) == 128
    if o.dtype != torch.bfloat16:
        raise RuntimeError(f"expected bf16 activations, got {o.dtype}")
    h, m, _ = o.shape
    q = torch.empty((m, h * 128), device=o.device, dtype=torch.int8)
    s = torch.empty((m, 1), device=o.device, dtype=torch.float32)
    _lib.call("rh3_quant_heads_i8", o.data_ptr(), o.stride(0), h, m, q.data_ptr(), q.stride(0), s.data_ptr(),
              _lib.stream())
    return q, s


def quant_groups_i8(o, rotate=False):
    """o [G, M, gw] bf16 group-major -> (q int8 [M, G*gw], s [M,1]); the general form of rot_quant_heads_i8."""
    _lib.require_cuda(o)
    assert o.ndim == 3 and o.stride(2) == 1 and o.stride(1) == o.shape[2] and o.dtype == torch.bfloat16
    g, m, gw = o.shape
    if rotate:
        _rot_width(g * gw)
    q = torch.empty((m, g * gw), device=o.device, dtype=torch.int8)
    s = torch.empty((m, 1), device=o.device, dtype=torch.float32)
    _lib.call("rh3_rot_quant_groups_i8" if rotate else "rh3_quant_groups_i8", o.data_ptr(), o.stride(0), g, gw, m, q.data_ptr(), q.stride(0), s.data_ptr(),
              _lib.stream())
    return q, s


def swiglu_rot_quant_rows_i8(x, rotate=True):
    """x [M, 2F] = [gate | up] -> int8 of silu(gate) * up (rotated unless rotate=False), [M, F]."""
    _check_rows(x)
    m, k2 = x.shape
    f = k2 // 2
    if rotate:
        _rot_width(f)
    q = torch.empty((m, f), device=x.device, dtype=torch.int8)
    s = torch.empty((m, 1), device=x.device, dtype=torch.float32)
    _lib.call("rh3_swiglu_rot_quant_rows_i8" if rotate else "rh3_swiglu_quant_rows_i8", x.data_ptr(), x.stride(0), m, f, q.data_ptr(), q.stride(0), s.data_ptr(),
              _lib.stream())
    return q, s


def norm_mod_rot_quant_rows_i8(x, weight, eps, idx, shift, scale, rotate=True):
    """int8 of rms_norm(x) * weight * (1 + scale[idx]) + shift[idx], per-row scales.

    weight: bf16 [K] or None; idx: int32 [M]; shift / scale: fp32 [R, K] views with a common row
    stride (the six AdaLN tables of a block are views into one [R, 6K] tensor)."""
    _check_rows(x)
    m, k = x.shape
    if rotate:
        _rot_width(k)
    _lib.require_cuda(idx, shift, scale, weight)
    assert idx.dtype == torch.int32 and idx.numel() == m and idx.is_contiguous()
    assert shift.dtype == torch.float32 and scale.dtype == torch.float32
    assert shift.ndim == 2 and scale.ndim == 2 and shift.shape[1] == k and scale.shape[1] == k
    assert shift.stride(1) == 1 and scale.stride(1) == 1 and shift.stride(0) == scale.stride(0)
    if weight is not None:
        assert weight.dtype == torch.bfloat16 and weight.numel() == k and weight.is_contiguous()
    q = torch.empty((m, k), device=x.device, dtype=torch.int8)
    s = torch.empty((m, 1), device=x.device, dtype=torch.float32)
    _lib.call("rh3_norm_mod_rot_quant_rows_i8" if rotate else "rh3_norm_mod_quant_rows_i8", x.data_ptr(), x.stride(0), _lib.ptr(weight), float(eps), idx.data_ptr(),
              shift.data_ptr(), scale.data_ptr(), shift.stride(0), m, k, q.data_ptr(), q.stride(0), s.data_ptr(),
              _lib.stream())
    return q, s
