"""fp16 int8-ConvRot linears of the VAE transformer decoder, over the CUDA kernels of this package.

Mirrors the operator layer of the reference's custom_nodes/rapid_h3/vae_fast.py and the extension it builds
(csrc/vae_ops.cu): `vae_out_quant`, `vae_gemm`, `vae_gemm_swiglu`, `_interleave_rows`, `gemm_config`, `_quantize`
(plain activations) and `_linear` (`vae_fast.py:55-63,71-85,118-169,259-263`). ComfyUI's `QuantizedTensor` and
comfy-kitchen are not required: a weight is passed as (int8 codes [N, K] of W . blockdiag(H256)^T, per-row scale
[N]), which is what the reference extracts from them (`vae_fast.py:131-142`). The D=64 rope + Q/K quantizer with
its K-anchor detector (`vae_qk_rope_quant`) and the tile batching are not built. No fallback path: CPU tensors or
other dtypes raise.
"""
import torch

from . import _lib


def gemm_config(m, n, k):
    """Kept for interface compatibility (the reference returns its CUTLASS tile id or None): one kernel here."""
    return 6


def _check_f16(*ts):
    _lib.require_cuda(*ts)
    for t in ts:
        if t.dtype != torch.float16:
            raise RuntimeError(f"expected fp16, got {t.dtype}")


def vae_out_quant(o):
    """o fp16 [B, H, S, D] contiguous head-major attention output -> [q int8 [B*S, H*D], scale fp32 [B*S]]
    (nan_to_num + ConvRot + int8), read in place."""
    _check_f16(o)
    if o.ndim != 4 or not o.is_contiguous():
        raise RuntimeError("o must be contiguous fp16 [B,H,S,D]")
    b, h, s, d = o.shape
    q = torch.empty((b * s, h * d), device=o.device, dtype=torch.int8)
    sc = torch.empty((b * s,), device=o.device, dtype=torch.float32)
    _lib.call("rh3_vae_out_quant", o.data_ptr(), b, h, s, d, q.data_ptr(), sc.data_ptr(), _lib.stream())
    return [q, sc]


def _quantize(x2d, act="none", act_weight=None, eps=0.0):
    """ConvRot int8 quantizer of a linear's fp16 input -> (xq [M, K], xs [M, 1]); plain activations only."""
    if act not in ("none", None, 0):
        raise NotImplementedError("fused activation prologues of the decoder's quantizer are not built")
    _check_f16(x2d)
    if x2d.ndim != 2 or x2d.stride(1) != 1:
        raise RuntimeError("x must be fp16 [M, K] with unit column stride")
    m, k = x2d.shape
    q = torch.empty((m, k), device=x2d.device, dtype=torch.int8)
    sc = torch.empty((m, 1), device=x2d.device, dtype=torch.float32)
    _lib.call("rh3_vae_quant_rows", x2d.data_ptr(), x2d.stride(0), m, k, q.data_ptr(), sc.data_ptr(), _lib.stream())
    return q, sc


def vae_gemm(xq, wq, xs, ws, bias, rscale=None, resid=None, config=6):
    """fp16 [M, N] = fp16((acc*xs)*ws + bias), and with a residual fp16(that * rscale + resid) (in separate roundings)."""
    _lib.require_cuda(xq, wq, xs, ws, bias)
    m, k = xq.shape
    n = wq.shape[0]
    if not (xq.is_contiguous() and wq.is_contiguous() and xq.dtype == torch.int8 and wq.dtype == torch.int8):
        raise RuntimeError("int8 contiguous inputs")
    if bias.dtype != torch.float16 or xs.dtype != torch.float32 or ws.dtype != torch.float32:
        raise RuntimeError("bias fp16, scales fp32")
    if (rscale is None) != (resid is None):
        raise RuntimeError("rscale and resid come together")
    if resid is not None:
        _check_f16(rscale, resid)
        if not resid.is_contiguous() or resid.shape != (m, n):
            raise RuntimeError("resid must be contiguous fp16 [M, N]")
    out = torch.empty((m, n), device=xq.device, dtype=torch.float16)
    _lib.call("rh3_vae_gemm", xq.data_ptr(), xq.stride(0), wq.data_ptr(), xs.data_ptr(), ws.data_ptr(), bias.data_ptr(),
              _lib.ptr(rscale), _lib.ptr(resid), n, m, n, k, out.data_ptr(), out.stride(0), _lib.stream())
    return out


def _interleave_rows(t, n):
    """Re-order the first axis of `t` (n rows: n/2 gate rows, then n/2 up rows) into runs of four gate rows
    followed by their four up rows, the order vae_gemm_swiglu reads weights, scales and biases in (same layout
    as gemm.swiglu_perm; the reference builds it in vae_fast.py:259-263)."""
    if n % 8:
        raise RuntimeError("_interleave_rows: n must be a multiple of 8")
    rest = tuple(t.shape[1:])
    return t.reshape(2, n // 8, 4, *rest).transpose(0, 1).reshape(n, *rest)


def vae_gemm_swiglu(xq, wq, xs, ws, bias, config=6):
    """w1 GEMM with SwiGLU in the epilogue; wq / ws / bias rows already interleaved; returns fp16 [M, N/2]."""
    _lib.require_cuda(xq, wq, xs, ws, bias)
    m, k = xq.shape
    n = wq.shape[0]
    if n % 16:
        raise RuntimeError("N must be a multiple of 16")
    out = torch.empty((m, n // 2), device=xq.device, dtype=torch.float16)
    _lib.call("rh3_vae_gemm_swiglu", xq.data_ptr(), xq.stride(0), wq.data_ptr(), xs.data_ptr(), ws.data_ptr(),
              bias.data_ptr(), m, n, k, out.data_ptr(), out.stride(0), _lib.stream())
    return out


def _linear(qdata, scale, bias, x, residual=None, residual_scale=None, xq_xs=None):
    """y = x W^T + b for fp16 x [..., K] and a ConvRot int8 weight (codes, per-row scales); with `residual`,
    y * residual_scale + residual in the GEMM epilogue (the pre-norm block's addcmul)."""
    lead = x.shape[:-1]
    n = qdata.shape[0]
    xq, xs = xq_xs if xq_xs is not None else _quantize(x.reshape(-1, x.shape[-1]).contiguous())
    ws = scale.reshape(-1).float()
    ws = ws if ws.numel() == n else ws.expand(n).contiguous()
    bias16 = bias.to(torch.float16) if bias is not None else torch.zeros(n, dtype=torch.float16, device=x.device)
    rs = resid = None
    if residual is not None:
        rs = residual_scale.to(torch.float16).reshape(-1).contiguous()
        resid = residual.reshape(-1, n).contiguous()
    out = vae_gemm(xq, qdata.contiguous(), xs.reshape(-1), ws, bias16, rs, resid)
    return out.reshape(*lead, n)
