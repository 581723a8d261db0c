"""INT8 flash attention front end; same entry points as the reference's
custom_nodes/rapid_h3/attn_int8.py (`attention`, `attention_bhsd`, `attention_rr`, `int8_prepass`).

q, k, v are bf16 [S, H, 128] views (last dim contiguous, e.g. slices of the qkv GEMM output).
Two numerics, chosen by `rotate`:
  rotate=False (default, the fast kernel): Q and K int8 with one scale per 64-token block per head (K
      mean-smoothed), V e4m3 per (head, channel), fp32 base-2 online softmax, e4m3 P against the running maximum
      (the reference's FP8-P.V family, its configs 50-56);
  rotate=True (the reference's production numerics, configs 80 / 90 / 94 / 190 / 194): Q and K int8 with one scale
      per token after a 128-point Hadamard rotation, V int8 per channel, P as u8 against each key tile's own maximum
      with a per-tile fold into the fp32 output.
`config` and `smooth_v` of the reference are accepted for signature compatibility; K and V smoothing are always on.
"""
import ctypes
import math
from dataclasses import dataclass

import torch

from . import _lib
from .timing import phase as _phase

D = 128


def _pad128(n):
    return (n + 127) // 128 * 128


def _pad256(n):
    """Query rows are padded to the 256-row pair of tiles one CTA of the main kernel works on."""
    return (n + 255) // 256 * 256


def _check_qkv(t, name):
    _lib.require_cuda(t)
    if t.dtype != torch.bfloat16 or t.ndim != 3 or t.shape[2] != D or t.stride(2) != 1:
        raise RuntimeError(f"{name}: expected bf16 [S, H, 128] with a contiguous last dim, got {tuple(t.shape)} {t.dtype}")


@dataclass
class Prepass:
    """Quantized operands of one attention call (the reference's int8_prepass list, as fields)."""
    q8: torch.Tensor      # int8 [H, Lq_pad, 128], Lq_pad a multiple of 256
    qs: torch.Tensor      # fp32 [H, Lq_pad/64]
    k8: torch.Tensor      # int8 [H, Lk_pad, 128]
    ks: torch.Tensor      # fp32 [H, Lk_pad/64]
    vt: torch.Tensor      # e4m3 [H, 128, Lk_pad]
    vscale: torch.Tensor  # fp32 [H, 128]
    vmean: torch.Tensor   # fp32 [H, 128]
    kmean: torch.Tensor   # fp32 [H, 128]
    lq: int
    lk: int


def rms_rope(x, weight, eps, tab=None, out=None):
    """Per-head RMSNorm (+ split-half partial 3-D RoPE when `tab` [.., S, .., 48, 2, 2] bf16 is given) of
    x [S, H, 128]; returns a new tensor unless `out` is given (`out=x` works in place)."""
    _check_qkv(x, "x")
    s, h, _ = x.shape
    if out is None:
        out = torch.empty((s, h, D), device=x.device, dtype=torch.bfloat16)
    _check_qkv(out, "out")
    if weight.dtype != torch.bfloat16 or weight.numel() != D:
        raise RuntimeError("norm weight must be bf16 [128]")
    weight = weight.contiguous()
    if tab is not None:
        if tab.dtype != torch.bfloat16 or tab.numel() != s * 48 * 4:
            raise RuntimeError("rope table must be bf16 [S, 48, 2, 2]")
        tab = tab.contiguous()
    _lib.call("rh3_rmsnorm_rope3d", x.data_ptr(), x.stride(0), x.stride(1), out.data_ptr(), out.stride(0),
              out.stride(1), s, h, weight.data_ptr(), float(eps), _lib.ptr(tab), _lib.stream())
    return out


def int8_prepass(q, k, v, tab=None, qw=None, kw=None, eps=1e-5, q_roped=None, k_roped=None, _tag="call"):
    """Quantize the operands of one attention call (three launches): K/V statistics, block-64 int8 Q and K, e4m3 V^T.
    With norm weights `qw` / `kw` (bf16 [128]) q and k are raw and get the per-head RMSNorm first, and with `tab`
    (bf16 [S, 48, 2, 2]) the 3-D RoPE as well; the normalised k is written to `k_roped` (a [Lk, H, 128] view, `k`
    itself for in place; a new tensor if None) and the normalised q only if `q_roped` is given."""
    with _phase(f"attn_{_tag}_prepass", (q.shape[0] + 2 * k.shape[0]) * q.shape[1] * D * 3):
        return _int8_prepass(q, k, v, tab, qw, kw, eps, q_roped, k_roped)


def _int8_prepass(q, k, v, tab, qw, kw, eps, q_roped, k_roped):
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        _check_qkv(t, n)
    lq, h, _ = q.shape
    lk = k.shape[0]
    if k.shape != v.shape or k.shape[1] != h:
        raise RuntimeError("k and v must have the same shape and q's head count")
    if (qw is None) != (kw is None):
        raise RuntimeError("q and k norm weights come together")
    dev = q.device
    if qw is not None:
        for w in (qw, kw):
            if w.dtype != torch.bfloat16 or w.numel() != D:
                raise RuntimeError("norm weight must be bf16 [128]")
        qw, kw = qw.contiguous(), kw.contiguous()
        if k_roped is None:
            k_roped = torch.empty((lk, h, D), device=dev, dtype=torch.bfloat16)
        _check_qkv(k_roped, "k_roped")
        if q_roped is not None:
            _check_qkv(q_roped, "q_roped")
    if tab is not None:
        if qw is None or lq != lk or tab.dtype != torch.bfloat16 or tab.numel() != lq * 48 * 4:
            raise RuntimeError("a rope table (bf16 [S, 48, 2, 2]) needs the norm weights and Lq == Lk")
        tab = tab.contiguous()
    lqp, lkp = _pad256(lq), _pad128(lk)
    f32 = dict(device=dev, dtype=torch.float32)
    kmean, vmean, vscale = (torch.empty((h, D), **f32) for _ in range(3))
    nbytes = _lib.lib().rh3_attn_kv_stats_scratch_bytes(lk, h)
    scratch = torch.empty(nbytes, device=dev, dtype=torch.uint8)
    q8 = torch.empty((h, lqp, D), device=dev, dtype=torch.int8)
    k8 = torch.empty((h, lkp, D), device=dev, dtype=torch.int8)
    qs = torch.empty((h, lqp // 64), **f32)
    ks = torch.empty((h, lkp // 64), **f32)
    vt = torch.empty((h, D, lkp), device=dev, dtype=torch.float8_e4m3fn)

    def view(t):
        return (None, 0, 0) if t is None else (t.data_ptr(), t.stride(0), t.stride(1))

    _lib.call("rh3_attn_prepass", q.data_ptr(), q.stride(0), q.stride(1), lq, lqp, k.data_ptr(), k.stride(0), k.stride(1),
              v.data_ptr(), v.stride(0), v.stride(1), lk, lkp, h, _lib.ptr(qw), _lib.ptr(kw), float(eps), _lib.ptr(tab),
              *view(q_roped), *view(k_roped if qw is not None else None), scratch.data_ptr(), nbytes, q8.data_ptr(),
              qs.data_ptr(), k8.data_ptr(), ks.data_ptr(), vt.data_ptr(), vscale.data_ptr(), vmean.data_ptr(),
              kmean.data_ptr(), _lib.stream())
    return Prepass(q8, qs, k8, ks, vt, vscale, vmean, kmean, lq, lk)


def attention_pre(pre, scale=None, out=None, scatter=None, _tag="call"):
    """Main kernel on pre-quantized operands -> out [Lq, H, 128] bf16 (strided `out` allowed).
    `scatter` = (device pointers, row starts [n+1], row stride, head stride) sends query rows
    [start[r], start[r+1]) to buffer r instead (rh3_attn_int8_scatter); nothing is returned then."""
    h = pre.q8.shape[0]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    if scatter is None:
        if out is None:
            out = torch.empty((pre.lq, h, D), device=pre.q8.device, dtype=torch.bfloat16)
        _check_qkv(out, "out")
        if out.shape[0] != pre.lq or out.shape[1] != h:
            raise RuntimeError("out must be [Lq, H, 128]")
    with _phase(f"attn_{_tag}_main", 4 * pre.lq * pre.lk * D * h):
        if scatter is None:
            _lib.call("rh3_attn_int8", pre.q8.data_ptr(), pre.qs.data_ptr(), pre.k8.data_ptr(), pre.ks.data_ptr(),
                      pre.vt.data_ptr(), pre.vscale.data_ptr(), pre.vmean.data_ptr(), pre.lq, pre.q8.shape[1], pre.lk,
                      pre.k8.shape[1], h, float(scale), out.data_ptr(), out.stride(0), out.stride(1), _lib.stream())
        else:
            ptrs, starts, o_ss, o_sh = scatter
            n = len(ptrs)
            c_ptrs = (ctypes.c_void_p * n)(*ptrs)
            c_starts = (ctypes.c_int64 * (n + 1))(*starts)
            _lib.call("rh3_attn_int8_scatter", pre.q8.data_ptr(), pre.qs.data_ptr(), pre.k8.data_ptr(),
                      pre.ks.data_ptr(), pre.vt.data_ptr(), pre.vscale.data_ptr(), pre.vmean.data_ptr(), pre.lq,
                      pre.q8.shape[1], pre.lk, pre.k8.shape[1], h, float(scale), c_ptrs, c_starts, n, o_ss, o_sh,
                      _lib.stream())
    return out


@dataclass
class TokPrepass:
    q8: torch.Tensor      # int8 [H, Lq_pad, 128], rotated, one scale per token
    qs: torch.Tensor      # fp32 [H, Lq_pad]
    k8: torch.Tensor      # int8 [H, Lk_pad, 128], rotated after the mean is removed
    ksb: torch.Tensor     # fp32 [H, Lk_pad/128, 2, 128]: per key tile 128 multipliers, then 128 biases
    vt: torch.Tensor      # int8 [H, 128, Lk_pad]
    vscale: torch.Tensor  # fp32 [H, 128]
    vmean: torch.Tensor   # fp32 [H, 128]
    kmean: torch.Tensor   # fp32 [H, 128]
    lq: int
    lk: int


def tok_prepass(q, k, v, tab=None, qw=None, kw=None, eps=1e-5, q_roped=None, k_roped=None, _tag="call"):
    """Operands of the token-scaled kernel (five launches); arguments as int8_prepass."""
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        _check_qkv(t, n)
    lq, h, _ = q.shape
    lk = k.shape[0]
    if k.shape != v.shape or k.shape[1] != h:
        raise RuntimeError("k and v must have the same shape and q's head count")
    if (qw is None) != (kw is None):
        raise RuntimeError("q and k norm weights come together")
    dev = q.device
    if qw is not None:
        for w in (qw, kw):
            if w.dtype != torch.bfloat16 or w.numel() != D:
                raise RuntimeError("norm weight must be bf16 [128]")
        qw, kw = qw.contiguous(), kw.contiguous()
        if k_roped is None:
            k_roped = torch.empty((lk, h, D), device=dev, dtype=torch.bfloat16)
        _check_qkv(k_roped, "k_roped")
        if q_roped is not None:
            _check_qkv(q_roped, "q_roped")
    if tab is not None:
        if qw is None or lq != lk or tab.dtype != torch.bfloat16 or tab.numel() != lq * 48 * 4:
            raise RuntimeError("a rope table (bf16 [S, 48, 2, 2]) needs the norm weights and Lq == Lk")
        tab = tab.contiguous()
    lqp, lkp = _pad256(lq), _pad128(lk)
    f32 = dict(device=dev, dtype=torch.float32)
    kmean, vmean, vscale = (torch.empty((h, D), **f32) for _ in range(3))
    nbytes = _lib.lib().rh3_attn_kv_stats_scratch_bytes(lk, h)
    scratch = torch.empty(nbytes, device=dev, dtype=torch.uint8)
    q8 = torch.empty((h, lqp, D), device=dev, dtype=torch.int8)
    k8 = torch.empty((h, lkp, D), device=dev, dtype=torch.int8)
    qs = torch.empty((h, lqp), **f32)
    ksb = torch.empty((h, lkp // 128, 2, 128), **f32)
    vt = torch.empty((h, D, lkp), device=dev, dtype=torch.int8)

    def view(t):
        return (None, 0, 0) if t is None else (t.data_ptr(), t.stride(0), t.stride(1))

    with _phase(f"attn_{_tag}_prepass", (q.shape[0] + 2 * k.shape[0]) * h * D * 3):
        _lib.call("rh3_attn_tok_prepass", q.data_ptr(), q.stride(0), q.stride(1), lq, lqp, k.data_ptr(), k.stride(0),
                  k.stride(1), v.data_ptr(), v.stride(0), v.stride(1), lk, lkp, h, _lib.ptr(qw), _lib.ptr(kw), float(eps),
                  _lib.ptr(tab), *view(q_roped if qw is not None else None), *view(k_roped if qw is not None else None),
                  scratch.data_ptr(), nbytes, q8.data_ptr(), qs.data_ptr(), k8.data_ptr(), ksb.data_ptr(), vt.data_ptr(),
                  vscale.data_ptr(), vmean.data_ptr(), kmean.data_ptr(), _lib.stream())
    return TokPrepass(q8, qs, k8, ksb, vt, vscale, vmean, kmean, lq, lk)


def attention_tok_pre(pre, scale=None, out=None, _tag="call"):
    """Token-scaled main kernel on the operands of tok_prepass -> out [Lq, H, 128] bf16 (strided `out` allowed)."""
    h = pre.q8.shape[0]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    if out is None:
        out = torch.empty((pre.lq, h, D), device=pre.q8.device, dtype=torch.bfloat16)
    _check_qkv(out, "out")
    if out.shape[0] != pre.lq or out.shape[1] != h:
        raise RuntimeError("out must be [Lq, H, 128]")
    with _phase(f"attn_{_tag}_main", 4 * pre.lq * pre.lk * D * h):
        _lib.call("rh3_attn_int8_tok", pre.q8.data_ptr(), pre.qs.data_ptr(), pre.k8.data_ptr(), pre.ksb.data_ptr(),
                  pre.vt.data_ptr(), pre.vscale.data_ptr(), pre.vmean.data_ptr(), pre.lq, pre.q8.shape[1], pre.lk,
                  pre.k8.shape[1], h, float(scale), out.data_ptr(), out.stride(0), out.stride(1), _lib.stream())
    return out


def attention(q, k, v, scale=None, config=0, smooth_k=True, smooth_v=True, rotate=False, out=None, _tag="call"):
    """q [Lq, H, 128], k, v [Lk, H, 128] bf16 (strided views allowed) -> [Lq, H, 128] bf16.
    `rotate=True` selects the token-scaled numerics (see the module text). `_tag` only names the timing phases of
    this call (timing.PHASES)."""
    if rotate:
        return attention_tok_pre(tok_prepass(q, k, v, _tag=_tag), scale, out, _tag=_tag)
    return attention_pre(int8_prepass(q, k, v, _tag=_tag), scale, out, _tag=_tag)


def attention_bhsd(q, k, v, scale=None, config=0, out=None):
    """[1, H, S, 128] layout of the reference's override; returns [1, H, S, 128]."""
    if q.ndim != 4 or q.shape[0] != 1:
        raise RuntimeError("attention_bhsd: expected [1, H, S, 128]")
    o = attention(q[0].transpose(0, 1), k[0].transpose(0, 1), v[0].transpose(0, 1), scale,
                  out=None if out is None else out[0].transpose(0, 1))
    return o.transpose(0, 1).unsqueeze(0) if out is None else out


def attention_rr(q, k, v, tab, qw, kw, eps, scale=None, config=0, out=None, q_roped=None, k_roped=None, _tag="call",
                 rotate=False):
    """attention() on raw q / k with the per-head RMSNorm (+ 3-D RoPE when `tab` is given) fused into the pre-pass.
    q and k are left untouched unless the caller passes them as `q_roped` / `k_roped` (views that receive the
    normalised rows; the fused block passes k itself, whose raw values nothing reads afterwards)."""
    if rotate:
        return attention_tok_pre(tok_prepass(q, k, v, tab, qw, kw, eps, q_roped, k_roped, _tag=_tag), scale, out, _tag=_tag)
    pre = int8_prepass(q, k, v, tab, qw, kw, eps, q_roped, k_roped, _tag=_tag)
    return attention_pre(pre, scale, out, _tag=_tag)
