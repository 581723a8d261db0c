"""fp16 int8-ConvRot linears of the VAE transformer decoder, over the CUDA kernels of this package.

Mirrors the operator layer of the reference's custom_nodes/rapid_h3/vae_fast.py and the extension it builds
(csrc/vae_ops.cu): `vae_out_quant`, `vae_gemm`, `vae_gemm_swiglu`, `_interleave_rows`, `gemm_config`, `_quantize`
(plain activations) and `_linear` (`vae_fast.py:55-63,71-85,118-169,259-263`). ComfyUI's `QuantizedTensor` and
comfy-kitchen are not required: a weight is passed as (int8 codes [N, K] of W . blockdiag(H256)^T, per-row scale
[N]), which is what the reference extracts from them (`vae_fast.py:131-142`). Also here: the quantizer's fused
prologues (`act` = "rms_norm" / "swiglu"), the feed-forward block on them (`_ff_forward`) and the whole-chunk tile
batching (`_tile_groups`, `tiled_decode_batched`). The D=64 attention pieces (`vae_qk_rope_quant` with its K-anchor
detector, and the attention kernel that consumes its operands) are not built. No fallback path: CPU tensors or other
dtypes raise.
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


_ACT_CODES = {"rms_norm": 1, "swiglu": 2}


def _input_act_width(act):
    """How many input columns make one quantized column: 2 for "swiglu" (gate | up), else 1."""
    return 2 if act == "swiglu" else 1


def _quantize(x2d, act="none", act_weight=None, eps=0.0):
    """ConvRot int8 quantizer of a linear's fp16 input -> (xq [M, K], xs [M, 1]). `act` fuses the prologue the
    decoder's linears ask for: "rms_norm" (with the pre-norm weight `act_weight` fp16 [K] or None, and `eps`) for the
    inputs of to_qkv and w1, "swiglu" (x = [gate | up], K = half the width) for the input of w2."""
    _check_f16(x2d)
    if x2d.ndim != 2 or x2d.stride(1) != 1:
        raise RuntimeError("x must be fp16 [M, K] with unit column stride")
    m = x2d.shape[0]
    k = x2d.shape[1] // _input_act_width(act)
    q = torch.empty((m, k), device=x2d.device, dtype=torch.int8)
    sc = torch.empty((m, 1), device=x2d.device, dtype=torch.float32)
    if act in ("none", None, 0):
        _lib.call("rh3_vae_quant_rows", x2d.data_ptr(), x2d.stride(0), m, k, q.data_ptr(), sc.data_ptr(), _lib.stream())
        return q, sc
    if act not in _ACT_CODES:
        raise ValueError(act)
    if act_weight is not None:
        _check_f16(act_weight)
        if act != "rms_norm" or act_weight.numel() != k:
            raise RuntimeError("act_weight is the rms_norm weight, fp16 [K]")
        act_weight = act_weight.contiguous()
    _lib.call("rh3_vae_quant_rows_act", x2d.data_ptr(), x2d.stride(0), m, k, _ACT_CODES[act], _lib.ptr(act_weight),
              float(eps), q.data_ptr(), sc.data_ptr(), _lib.stream())
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


def _linear(qdata, scale, bias, x, residual=None, residual_scale=None, xq_xs=None, act="none", act_weight=None, eps=0.0):
    """y = act(x) W^T + b for fp16 x [..., K] and a ConvRot int8 weight (codes, per-row scales); with `residual`,
    y * residual_scale + residual in the GEMM epilogue (the pre-norm block's addcmul). `act` is the quantizer's
    prologue (_quantize)."""
    lead = x.shape[:-1]
    n = qdata.shape[0]
    xq, xs = xq_xs if xq_xs is not None else _quantize(x.reshape(-1, x.shape[-1]).contiguous(), act, act_weight, eps)
    ws = scale.reshape(-1).float()
    ws = ws if ws.numel() == n else ws.expand(n).contiguous()
    bias16 = bias.to(torch.float16) if bias is not None else torch.zeros(n, dtype=torch.float16, device=x.device)
    rs = resid = None
    if residual is not None:
        rs = residual_scale.to(torch.float16).reshape(-1).contiguous()
        resid = residual.reshape(-1, n).contiguous()
    out = vae_gemm(xq, qdata.contiguous(), xs.reshape(-1), ws, bias16, rs, resid)
    return out.reshape(*lead, n)


class Int8Linear:
    """What the reference reads out of a ComfyUI int8-ConvRot linear (`vae_fast.py:131-142`): rotated int8 codes
    [N, K], one scale per output row (or one for the tensor) and an fp16 bias."""

    def __init__(self, qdata, scale, bias=None):
        self.qdata, self.scale, self.bias = qdata.contiguous(), scale, bias
        self._w1 = None

    def swiglu_rows(self):
        """Codes, scales and bias in the row order the SwiGLU epilogue reads (cached, as `_W1_CACHE`, :255-290)."""
        if self._w1 is None:
            n = self.qdata.shape[0]
            ws = self.scale.reshape(-1).float()
            ws = ws if ws.numel() == n else ws.expand(n)
            b16 = (self.bias.to(torch.float16) if self.bias is not None
                   else torch.zeros(n, dtype=torch.float16, device=self.qdata.device))
            self._w1 = (_interleave_rows(self.qdata, n).contiguous(), _interleave_rows(ws, n).contiguous(),
                        _interleave_rows(b16, n).contiguous())
        return self._w1


_SWIGLU = True


def install_swiglu(on=True):
    """SwiGLU in the w1 GEMM epilogue (the reference's level 3, `vae_fast.py:416-421`); off: w1 writes [gate | up]
    and the SwiGLU is the prologue of w2's quantizer."""
    global _SWIGLU
    _SWIGLU = bool(on)


def _ff_forward(w1, w2, x, pre_norm_weight, eps, residual, residual_scale):
    """The decoder's feed-forward block (`vae_fast.py:298-318`): w2(SwiGLU(w1(rms_norm(x)))) * residual_scale +
    residual, fp16 in and out; w1, w2 are Int8Linear. Three or four kernel launches per call, no fp16 round trip of
    the normalised input."""
    _check_f16(x, residual, residual_scale)
    lead, kdim = x.shape[:-1], x.shape[-1]
    x2 = x.reshape(-1, kdim).contiguous()
    if _SWIGLU:
        xq, xs = _quantize(x2, "rms_norm", pre_norm_weight, eps)
        wq, ws, b = w1.swiglu_rows()
        h = vae_gemm_swiglu(xq, wq, xs.reshape(-1), ws, b)
        return _linear(w2.qdata, w2.scale, w2.bias, h, residual, residual_scale).reshape(*lead, -1)
    h = _linear(w1.qdata, w1.scale, w1.bias, x2, act="rms_norm", act_weight=pre_norm_weight, eps=eps)
    return _linear(w2.qdata, w2.scale, w2.bias, h, residual, residual_scale, act="swiglu").reshape(*lead, -1)


def _tile_groups(n, batch):
    """How many tiles go into each decoder call when n tiles are decoded about `batch` at a time: group sizes as
    equal as possible, and never a single tile beside larger groups (the reference found that a decoder call on one
    tile does not reproduce the bits of that tile decoded with others, so a [batch, ..., rest] split made the
    picture depend on free memory; `vae_fast.py:321-333`)."""
    if n <= 1:
        return [n] if n else []
    groups = -(-n // max(1, batch))
    if n // groups < 2:
        groups = n // 2
    small, extra = divmod(n, groups)
    return [small + 1] * extra + [small] * (groups - extra)


def split_tiles(size, tile, overlap):
    """Tile starts, lengths and overlaps along one axis of `size` pixels: tiles of `tile` pixels that share `overlap`
    pixels with the next one; the last tile is shifted back so that it ends at the border."""
    if size <= tile:
        return [0], [size], []
    step = tile - overlap
    starts = list(range(0, size - tile, step)) + [size - tile]
    lens = [tile] * len(starts)
    overlaps = [starts[i] + lens[i] - starts[i + 1] for i in range(len(starts) - 1)]
    return starts, lens, overlaps


def blend(a, b, n, dim):
    """Cross-fade: the first n entries of `b` along `dim` become a linear mix with `a` (n entries), weight of b
    rising from 1/(n+1) to n/(n+1)."""
    if n <= 0:
        return b
    shape = [1] * b.dim()
    shape[dim] = n
    wide = torch.promote_types(b.dtype, torch.float32)   # half-precision pictures are mixed in fp32
    w = (torch.arange(1, n + 1, device=b.device, dtype=wide) / (n + 1)).reshape(shape)
    head = b.narrow(dim, 0, n)
    mixed = (a.to(wide) * (1 - w) + head.to(wide) * w).to(b.dtype)
    return torch.cat([mixed, b.narrow(dim, n, b.shape[dim] - n)], dim=dim)


def tiled_decode_batched(decode, z, ratio, tile, overlap, batch):
    """Decode a latent z [..., h, w] in spatial tiles, `batch` tiles per decoder call across tile rows (group sizes
    by _tile_groups), and stitch them with cross-faded seams: the scheme of the reference's `_tiled_decode_batched`
    (`vae_fast.py:336-400`) with this module's own split and blend (the reference takes both from ComfyUI's VAE
    class). `decode` maps a batch of latent tiles [n, ..., th, tw] to pixels [n, ..., th*ratio, tw*ratio]; `tile`
    and `overlap` are in pixels and multiples of `ratio`."""
    if tile % ratio or overlap % ratio or overlap >= tile:
        raise RuntimeError("tile and overlap must be multiples of the decoder's ratio, overlap < tile")
    height, width = z.shape[-2] * ratio, z.shape[-1] * ratio
    y_idx, y_len, y_ov = split_tiles(height, tile, overlap)
    x_idx, x_len, x_ov = split_tiles(width, tile, overlap)

    def all_tiles():
        slices = [z[..., i0 // ratio:(i0 + il) // ratio, j0 // ratio:(j0 + jl) // ratio]
                  for i0, il in zip(y_idx, y_len) for j0, jl in zip(x_idx, x_len)]
        k = 0
        for size in _tile_groups(len(slices), batch):
            out = decode(torch.cat(slices[k:k + size]))
            k += size
            yield from out.chunk(size)

    tiles = all_tiles()
    canvas = above = None
    for i in range(len(y_idx)):
        below = left = None
        for j in range(len(x_idx)):
            x0 = x_idx[j]
            t = next(tiles)
            if above is not None:
                t = blend(above[..., :, x0:x0 + x_len[j]], t, y_ov[i - 1], dim=-2)
            if left is not None:
                t = blend(left, t, x_ov[j - 1], dim=-1)
            h, w = t.shape[-2], t.shape[-1]
            if j + 1 < len(x_idx):
                w -= x_ov[j]
                left = t[..., :, w:].clone()
            if canvas is None:
                canvas = t.new_empty(*t.shape[:-2], height, width)
            if i + 1 < len(y_idx):
                h -= y_ov[i]
                if below is None:
                    below = t.new_empty(*t.shape[:-2], y_ov[i], width)
                below[..., :, x0:x0 + w] = t[..., h:, :w]
            canvas[..., y_idx[i]:y_idx[i] + h, x0:x0 + w].copy_(t[..., :h, :w])
        above = below
    return canvas
