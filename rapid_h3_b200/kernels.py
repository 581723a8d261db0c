"""Quantized linear front end; same surface as the reference's custom_nodes/rapid_h3/kernels.py
(`QWeight`, `quantize_weight`, `quantize_rows`, `linear`, `gemm_config`), with every mode routed to
the CUDA kernels of this package. Unknown modes raise ValueError as in the reference; modes the
reference only emulates (nvfp4 fakes) and its per-tensor fp8 mode raise NotImplementedError.
"""
from dataclasses import dataclass

import torch

from . import gemm as _cf
from . import quantizers as _tq

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0


@dataclass
class QWeight:
    """A quantized weight: codes [N, K] and one fp32 scale per output row, shaped [1, N] (kernels.py:29-32 of the
    reference). `layout` says in which order the N rows are held: "rows" = the module's own order, "swiglu8" = the
    gate/up interleave of gemm.swiglu_perm that the fused fc1 + SwiGLU GEMM reads."""
    q: torch.Tensor
    scale: torch.Tensor
    layout: str = "rows"


_ROWWISE_I8 = ("int8_rowwise", "int8_fast")
_ROT_I8 = ("int8_rot",)
_ROWWISE_F8 = ("fp8_rowwise", "fp8_rowwise_torch")
_TENSOR_F8 = ("fp8_tensor",)
_UNSUPPORTED = ("nvfp4_fake", "nvfp4_rot_fake")


def quantize_weight(w, mode):
    """Per-output-row weight quantization (one-off, at load): W [N,K] -> QWeight(q [N,K], scale [1,N]).
    Runs through the same row quantizer kernels as the activations (same arithmetic as the reference's
    kernels.py:52-72 for the row-wise modes). `int8_rot` stores int8(W . blockdiag(H256)^T): the rotation is
    orthonormal, so rotated activations times rotated weights give x W^T (kernels.py:58-60)."""
    if mode in _UNSUPPORTED:
        raise NotImplementedError(f"mode {mode!r} is not implemented in rapid_h3_b200")
    if mode not in _ROWWISE_I8 + _ROWWISE_F8 + _ROT_I8 + _TENSOR_F8:
        raise ValueError(mode)
    w = w.detach()
    if w.dtype != torch.bfloat16:
        # the row quantizers read bf16; a weight that is not exactly representable would change codes
        if not torch.equal(w.to(torch.bfloat16).to(w.dtype), w):
            raise RuntimeError("quantize_weight: weight is not bf16-representable")
        w = w.to(torch.bfloat16)
    if mode in _TENSOR_F8:
        # one scale for the whole weight (kernels.py:63-65); kept as [1, N] equal entries for the row-scaled GEMM
        q, s = _tq.quant_tensor(w.contiguous())
        return QWeight(q, s.t().contiguous())
    fn = _tq.rot_quant_rows_i8 if mode in _ROT_I8 else (_tq.quant_rows_i8 if mode in _ROWWISE_I8 else _tq.quant_rows)
    q, s = fn(w.contiguous())
    return QWeight(q, s.t().contiguous())


def quantize_rows(x, mode):
    """Per-token (row) dynamic quantization -> (q, scale[M, 1] fp32)."""
    if mode in _ROWWISE_I8:
        return _tq.quant_rows_i8(x)
    if mode in _ROT_I8:
        return _tq.rot_quant_rows_i8(x)
    if mode in _ROWWISE_F8:
        return _tq.quant_rows(x)
    if mode in _TENSOR_F8:
        return _tq.quant_tensor(x)
    raise ValueError(mode)


def gemm_config(k, n):
    """Kept for interface compatibility: the reference returns its CUTLASS tile id; there is one kernel here."""
    return 6


def linear(x, qw, mode):
    """y = x @ W^T for x [M, K] bf16 and a QWeight of W [N, K]; returns bf16."""
    if mode in _UNSUPPORTED:
        raise NotImplementedError(f"mode {mode!r} is not implemented in rapid_h3_b200")
    xq, sa = quantize_rows(x.contiguous(), mode)
    if mode in _ROWWISE_F8 + _TENSOR_F8:
        return _cf.fp8_gemm(xq, sa, qw.q, qw.scale)
    return _cf.int8_gemm(xq, sa, qw.q, qw.scale)
