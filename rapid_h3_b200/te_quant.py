"""int8_rot linears of the text encoder: the W8A8 rotated linear plus a second int8 pass on the quantization
residual of outlier rows.

Mirrors `_TELinear` of the reference's custom_nodes/rapid_h3/te_quant.py:45-115 for its `int8_rot` and
`int8_rot_plain` modes (fp32 in, fp32 out, like the module it replaces). The weight is passed as a
`kernels.QWeight` holding int8 codes of W . blockdiag(H256)^T and per-row scales (what the reference adopts from an
int8_convrot checkpoint, `:33-42`). ComfyUI's CLIP cloning, weight casting contexts and the bf16 attention wrapper
are outside this path. CPU tensors raise: there is no fallback.
"""
import torch

from . import _lib, gemm, kernels, quantizers

# how often the second pass ran: [rows that took it, rows seen]; `residual_share()` reads it
_ROWS = [0, 0]


def residual_share():
    """Fraction of the rows seen so far that were given the residual pass (0.0 before any call)."""
    return _ROWS[0] / _ROWS[1] if _ROWS[1] else 0.0


def rot_residual_quant_rows_i8(x, q1, s1, rows):
    """int8 row quantizer of rotate(x[rows]) - q1[rows] * s1[rows] -> (q2 int8 [n, K], s2 fp32 [n, 1]); x fp32."""
    _lib.require_cuda(x, q1, s1, rows)
    if x.dtype != torch.float32 or x.ndim != 2 or x.stride(1) != 1:
        raise RuntimeError("x must be fp32 [M, K] with unit column stride")
    n, k = rows.numel(), x.shape[1]
    rows = rows.to(torch.int32).contiguous()
    q2 = torch.empty((n, k), device=x.device, dtype=torch.int8)
    s2 = torch.empty((n, 1), device=x.device, dtype=torch.float32)
    _lib.call("rh3_rot_residual_quant_rows_i8", x.data_ptr(), x.stride(0), q1.data_ptr(), q1.stride(0), s1.data_ptr(),
              rows.data_ptr(), n, k, q2.data_ptr(), s2.data_ptr(), _lib.stream())
    return q2, s2


class _TELinear:
    """Replacement forward for one linear of the language model (fp32 in, fp32 out)."""

    def __init__(self, qweight, bias=None, mode="int8_rot", outlier_ratio=8.0):
        if mode not in ("int8_rot", "int8_rot_plain"):
            raise NotImplementedError(f"text-encoder mode {mode!r} is not implemented")
        self.qweight, self.bias, self.mode, self.outlier_ratio = qweight, bias, mode, outlier_ratio

    def _outlier_rows(self, x32, s1):
        """Indices of the rows whose rotated peak is more than `outlier_ratio` times their rms. H256 is orthonormal,
        so the rotated row has the rms of the input row, and its abs-max is 127 * s1 by construction of the scale:
        nothing has to be rotated again to find them (selection rule of the reference, te_quant.py:97-99)."""
        rms = x32.square().mean(dim=-1).sqrt().clamp_min(1e-12)
        peak_over_rms = (127.0 * s1.reshape(-1)) / rms
        return torch.nonzero(peak_over_rms > self.outlier_ratio).reshape(-1)

    def _matmul(self, x2):
        """x2 [M, K] in the caller's dtype -> W8A8 product in bf16 or, when rows took the second pass, fp32."""
        qw = self.qweight
        x16 = x2.to(torch.bfloat16).contiguous()
        if self.mode == "int8_rot_plain":
            return kernels.linear(x16, qw, "int8_rot")
        q1, s1 = quantizers.rot_quant_rows_i8(x16)
        y = gemm.int8_gemm(q1, s1, qw.q, qw.scale)
        x32 = x2.float().contiguous()
        rows = self._outlier_rows(x32, s1)
        _ROWS[1] += x2.shape[0]
        if rows.numel() == 0:
            return y
        # second int8 pass on what the first quantization lost on those rows: rotate(x) - q1 * s1, quantized with
        # its own row scale and multiplied with the same weight; the two products add up in fp32
        q2, s2 = rot_residual_quant_rows_i8(x32, q1, s1, rows)
        y = y.float()
        y[rows] += gemm.int8_gemm(q2, s2, qw.q, qw.scale).float()
        _ROWS[0] += rows.numel()
        return y

    def __call__(self, x):
        if x.device.type != "cuda":
            raise NotImplementedError("_TELinear: CUDA tensors only (no fallback path)")
        lead, k = x.shape[:-1], x.shape[-1]
        y = self._matmul(x.reshape(-1, k)).to(x.dtype)
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        return y.reshape(*lead, y.shape[-1])
