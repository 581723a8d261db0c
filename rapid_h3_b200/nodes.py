"""Operator surface of the Rapid-H3 node pack for the DiT block, over the CUDA kernels of this package.

Mirrors custom_nodes/rapid_h3/__init__.py of the reference: `_QuantLinear` (:83-167), `_row_index`
(:189-200), `_fused_block` (:207-321), `RapidH3LinearQuant.patch` (:369-417) and
`RapidH3Int8Attention.patch` (:995-1047). ComfyUI is not required: `patch` takes any module tree whose
blocks expose the attributes the reference reads (see rapid_h3_b200.model) and returns a handle whose
`block_forward` list replaces the blocks' forwards. Calls the reference would silently route to the
stock path (non-bf16, CPU tensors, missing rope table) raise NotImplementedError here instead: there is
no fallback path.
"""
import re

import torch

from . import attn_int8, kernels
from .timing import phase as _phase
from . import gemm as cf
from . import quantizers as tq

NAME_RE = re.compile(r"^blocks\.(\d+)\.(attn|mlp|cross)\.(qkv_proj|out_proj|fc1|fc2|q_proj|kv_proj)$")

_IDX_CACHE = {}   # (segment tuple, S, device) -> int32 [S]; a handful of entries at most
_IDX_CACHE_MAX = 8


def _row_index(segments, s, device):
    """Which row of the modulation tables every token of the packed sequence reads: int32 [S].

    `segments` is the block's `mod_segments`, a list of (start, stop, row). `row` is either one table row for the
    whole span or an integer tensor with one row per token of the span (per-token conditioning). Spans given as
    plain integers are remembered by value, so the same segmentation costs one fill per process, however many
    list objects carry it; spans with tensors are rebuilt on every call because their content may change.
    Contract: custom_nodes/rapid_h3/__init__.py:189-200 of the reference."""
    per_token = any(torch.is_tensor(row) for _, _, row in segments)
    key = None
    if not per_token:
        key = (tuple((int(a), int(b), int(row)) for a, b, row in segments), int(s), str(device))
        hit = _IDX_CACHE.get(key)
        if hit is not None:
            return hit
    idx = torch.zeros(s, dtype=torch.int32, device=device)
    for a, b, row in segments:
        if b <= a:
            continue
        if torch.is_tensor(row):
            if row.numel() not in (1, b - a):
                raise RuntimeError(f"mod_segments: span [{a}, {b}) carries {row.numel()} rows")
            idx[a:b].copy_(row.reshape(-1).to(device=device, dtype=torch.int32))
        else:
            idx[a:b].fill_(int(row))
    if key is not None:
        if len(_IDX_CACHE) >= _IDX_CACHE_MAX:
            _IDX_CACHE.pop(next(iter(_IDX_CACHE)))
        _IDX_CACHE[key] = idx
    return idx


def _stored_as_rotated_int8(w):
    """True when `w` already is what the `int8_rot` recipe stores: ComfyUI's int8_convrot tensor, i.e. int8 codes
    `_qdata` [N, K] of the weight rotated in groups of 256 with one scale per output row in `_params`."""
    meta = getattr(w, "_params", None)
    codes = getattr(w, "_qdata", None)
    if meta is None or codes is None or codes.dtype != torch.int8:
        return False
    return (bool(getattr(meta, "convrot", False)) and getattr(meta, "convrot_groupsize", 0) == tq.ROT_GROUP
            and not getattr(meta, "transposed", False))


class _QuantLinear:
    """Replacement forward bound to one Linear: row quantizer + W8A8 GEMM, bias added afterwards in bf16
    (reference: __init__.py:132-167). The quantized weight is made on first use and kept until the weight it was
    made from changes: the cache key is the owning patcher's `patches_uuid` when the module came with one (the
    reference's key, __init__.py:119-130), the weight tensor's identity and in-place version, and the device."""

    def __init__(self, module, name, mode, measure_every=0, stats=None, patcher=None):
        self.module, self.name, self.mode = module, name, mode
        self.measure_every, self.stats = measure_every, stats if stats is not None else {}
        self.patcher = patcher
        self.qweight = None
        self.cache_key = None
        self.calls = 0

    def _make_qweight(self, w):
        """QWeight of `w` for this linear's mode. A checkpoint that is already stored as rotated int8 is taken over
        as it is when the mode is `int8_rot` (no bf16 copy is ever made); any other quantized tensor is expanded
        first and quantized again in this mode (contract: reference __init__.py:107-117)."""
        if self.mode == "int8_rot" and _stored_as_rotated_int8(w):
            scale = w._params.scale.to(torch.float32).reshape(1, -1)
            return kernels.QWeight(w._qdata.contiguous(), scale.contiguous())
        if hasattr(w, "_params") and hasattr(w, "dequantize"):
            w = w.dequantize()
        return kernels.quantize_weight(w.detach(), self.mode)

    def _weight_key(self, device):
        w = self.module.weight
        uuid = getattr(self.patcher, "patches_uuid", None)
        return (uuid, id(w), getattr(w, "_version", 0), tuple(w.shape), str(device))

    def qweight_for(self, x=None):
        w = self.module.weight
        if self.qweight is not None and w.numel() == 0:
            return self.qweight          # the bf16 copy was released on purpose: the int8 copy is all there is
        key = self._weight_key(w.device if x is None else x.device)
        if self.qweight is None or key != self.cache_key:
            self.qweight = self._make_qweight(w)
            self.cache_key = key
        return self.qweight

    def __call__(self, x):
        if x.device.type != "cuda" or x.dtype != torch.bfloat16:
            raise NotImplementedError("_QuantLinear: only CUDA bf16 activations are supported (no fallback path)")
        shape = x.shape
        qw = self.qweight_for(x)
        y = kernels.linear(x.reshape(-1, shape[-1]), qw, self.mode)
        if qw.layout == "swiglu8":  # the fused block keeps fc1 in its epilogue's row order: put the columns back
            y = y.index_select(-1, torch.argsort(cf.swiglu_perm(y.shape[-1], y.device)))
        if self.module.bias is not None:
            y = y + self.module.bias.to(y.dtype)
        y = y.reshape(*shape[:-1], y.shape[-1])
        self.calls += 1
        if self.measure_every and self.calls % self.measure_every == 0 and self.module.weight.numel():
            # error of this call against the unquantized linear (a measurement, not part of the path;
            # reference __init__.py:160-164)
            ref = torch.nn.functional.linear(x, self.module.weight.to(x.dtype), self.module.bias)
            err = ((y.float() - ref.float()).norm() / ref.float().norm().clamp_min(1e-12)).item()
            self.stats.setdefault(self.name, []).append(err)
        return y


class FusedBlock:
    """DiTBlock.forward with norm + modulation fused into the int8 quantizers, W8A8 GEMMs with fused
    epilogues, and the INT8 attention kernel (the graph of reference __init__.py:253-320, plus the
    cross-attention of the benchmark configuration):

        norm_mod_quant -> qkv GEMM -> q/k RMSNorm+RoPE -> [heads<->tokens exchange] -> attention
        -> row quantizer -> out_proj GEMM with gated residual (per modality segment)
        -> norm_quant -> q GEMM / kv GEMM on text -> q/k RMSNorm -> attention(Lq != Lk) -> quantizer
        -> out GEMM + residual
        -> norm_mod_quant -> fc1 GEMM with SwiGLU epilogue -> row quantizer -> fc2 GEMM with gated residual

    `sp` (rapid_h3_b200.sp.Ulysses or None) re-shards q/k/v from tokens to heads around self-attention.
    """

    def __init__(self, block, qkv_q, out_q, fc1_q, fc2_q, cq_q=None, ckv_q=None, co_q=None):
        self.block = block
        self.qkv_q, self.out_q, self.fc1_q, self.fc2_q = qkv_q, out_q, fc1_q, fc2_q
        self.cq_q, self.ckv_q, self.co_q = cq_q, ckv_q, co_q
        # `int8_rot`: every quantizer rotates its row with H256 and every weight is stored rotated
        self.rotate = qkv_q.mode == "int8_rot"
        self._const = {}

    # -- helpers -----------------------------------------------------------------------------
    @staticmethod
    def _norm_w(norm):
        w = getattr(norm, "weight", None)
        return None if w is None else w.detach().to(torch.bfloat16).contiguous()

    @staticmethod
    def _eps(norm):
        e = getattr(norm, "eps", None)
        return torch.finfo(torch.bfloat16).eps if e is None else e

    def _fc1_swiglu_weight(self):
        """(codes, scales) of fc1 with its output rows in the order the SwiGLU epilogue pairs them
        (gemm.swiglu_perm). The re-ordered copy takes the place of the plain one in fc1's cache, tagged
        `layout="swiglu8"`, so only one int8 copy of the largest weight of the block is resident."""
        qw = self.fc1_q.qweight_for()
        if qw.layout != "swiglu8":
            order = cf.swiglu_perm(qw.q.shape[0], qw.q.device)
            qw = kernels.QWeight(qw.q.index_select(0, order), qw.scale.index_select(1, order), layout="swiglu8")
            self.fc1_q.qweight = qw
        return qw.q, qw.scale

    @staticmethod
    def _eps_mismatch():
        raise NotImplementedError("the fused attention pre-pass needs q_norm and k_norm to share eps")

    def _zeros_tab(self, d, device):
        key = ("zeros", d, str(device))
        if key not in self._const:
            self._const[key] = (torch.zeros(1, d, device=device), torch.ones(d, device=device, dtype=torch.bfloat16))
        return self._const[key]

    @staticmethod
    def _gate_rows(gate_tab):
        """The gate table [R, d] as bf16 rows, converted once per forward (one row per modality)."""
        return gate_tab.to(torch.bfloat16).contiguous()

    @staticmethod
    def _gemm_gated(xq, xs, q, x, gates, segments):
        """x += gate * (xq @ W^T), one GEMM per modality segment, each with its own gate row of `gates` [R, d] bf16;
        a segment whose row is a per-token tensor is split into runs of equal rows."""
        qw = q.qweight_for()
        for a, b, row in segments:
            if b <= a:
                continue
            if torch.is_tensor(row) and row.numel() > 1:
                rows = row.reshape(-1).tolist()
                start = 0
                for i in range(1, len(rows) + 1):
                    if i == len(rows) or rows[i] != rows[start]:
                        cf.int8_gemm_gated_residual(xq[a + start:a + i], xs[a + start:a + i], qw.q, qw.scale,
                                                    gates[int(rows[start])], x[a + start:a + i])
                        start = i
            else:
                cf.int8_gemm_gated_residual(xq[a:b], xs[a:b], qw.q, qw.scale, gates[int(row)], x[a:b])
        return x

    # -- forward -----------------------------------------------------------------------------
    def forward(self, x, t_emb, mod_segments, rope_freqs, ctx=None, sp=None, trace=None):
        blk = self.block
        if rope_freqs is None or x.dtype != torch.bfloat16 or x.device.type != "cuda" or x.ndim != 2:
            raise NotImplementedError("FusedBlock: needs a 2-D CUDA bf16 packed sequence and a rope table")
        s, d = x.shape
        a = blk.attn
        hd = a.heads * a.head_dim
        f = blk.mlp.fc2.weight.shape[1] if blk.mlp.fc2.weight.numel() else self.fc2_q.qweight_for().q.shape[1]
        with _phase("adaln"):
            shift_msa, scale_msa, gate_msa, shift_mlp, scale_mlp, gate_mlp = blk.adaln_proj(t_emb)
            idx = _row_index(mod_segments, s, x.device)
            tab = rope_freqs.reshape(s, 48, 2, 2).contiguous()
            gates_msa, gates_mlp = self._gate_rows(gate_msa), self._gate_rows(gate_mlp)
        rot = self.rotate
        qbytes = lambda k: s * k * 3 + 4 * s  # noqa: E731  (row quantizer: 2 bytes in, 1 out per element, a scale per row)

        def rec(name, value):
            if trace is not None:
                trace[name] = value.clone() if torch.is_tensor(value) else value

        # ---- self-attention ----
        with _phase("quant_norm_mod", qbytes(d)):
            xq, xs = tq.norm_mod_rot_quant_rows_i8(x, self._norm_w(blk.norm1), self._eps(blk.norm1), idx, shift_msa, scale_msa, rotate=rot)
        rec("attn_in_q", xq), rec("attn_in_s", xs)
        qw = self.qkv_q.qweight_for()
        with _phase("gemm_qkv", 2 * s * 3 * hd * d):
            qkv = cf.int8_gemm(xq, xs, qw.q, qw.scale)
        rec("qkv", qkv)
        q, k, v = (t.view(s, a.heads, a.head_dim) for t in qkv.split(hd, dim=-1))
        if sp is not None and sp.fused:
            # both exchanges done by the kernels: rope + scatter to the head owners, attention epilogue scatters back
            if a.q_norm.eps != a.k_norm.eps:
                raise NotImplementedError("fused exchange: q and k norms must share eps")
            if ATTN_ROTATE:
                raise NotImplementedError("the token-scaled attention has no scattering epilogue: use the all-to-all exchange")
            with _phase("exchange_rope_scatter", s * hd * 2 * 3 * 2):
                qg, kg, vg = sp.rope_scatter(qkv, self._norm_w(a.q_norm), self._norm_w(a.k_norm), a.q_norm.eps, tab)
            o = sp.attention_scatter(qg, kg, vg)                    # [P, S_local, (H/P)*128] group-major
            with _phase("quant_attn_out", qbytes(hd)):
                oq, os_ = tq.quant_groups_i8(o, rotate=rot)
        else:
            if sp is None:
                # RMSNorm + RoPE of q and k run inside the attention pre-pass: q is quantized from registers, the
                # normalised k replaces the raw one in the qkv buffer (nothing reads the raw values afterwards);
                # when a trace is asked for, the normalised q is stored too
                raw = (q.clone(), k.clone()) if RR_CHECK else None
                o = attn_int8.attention_rr(q, k, v, tab, self._norm_w(a.q_norm), self._norm_w(a.k_norm), a.q_norm.eps
                                           if a.q_norm.eps == a.k_norm.eps else self._eps_mismatch(),
                                           q_roped=q if trace is not None else None, k_roped=k, _tag="self",
                                           rotate=ATTN_ROTATE)
                if raw is not None:
                    _rr_check(raw[0], raw[1], v, o, tab, self._norm_w(a.q_norm), self._norm_w(a.k_norm), a.q_norm.eps)
                rec("qkv_rr", qkv)
                rec("attn_out", o)                                     # [S, H, 128] token-major
                with _phase("quant_attn_out", qbytes(hd)):
                    oq, os_ = tq.rot_quant_rows_i8(o.view(s, hd), rotate=rot)
            else:
                with _phase("rms_rope", s * hd * 2 * 2 * 2):
                    attn_int8.rms_rope(q, self._norm_w(a.q_norm), a.q_norm.eps, tab, out=q)
                    attn_int8.rms_rope(k, self._norm_w(a.k_norm), a.k_norm.eps, tab, out=k)
                with _phase("exchange_all_to_all"):
                    qg, kg, vg = sp.tokens_to_heads(qkv, a.heads, a.head_dim)  # [S_total, H/P, 128] each
                og = attn_int8.attention(qg, kg, vg, _tag="self", rotate=ATTN_ROTATE)
                with _phase("exchange_all_to_all"):
                    o = sp.heads_to_tokens(og)                          # [P, S_local, (H/P)*128] group-major
                with _phase("quant_attn_out", qbytes(hd)):
                    oq, os_ = tq.quant_groups_i8(o, rotate=rot)
        del qkv, q, k, v
        with _phase("gemm_out_proj", 2 * s * d * hd):
            x = self._gemm_gated(oq, os_, self.out_q, x, gates_msa, mod_segments)
        rec("x_attn", x)

        # ---- cross-attention to text ----
        if self.cq_q is not None:
            c = blk.cross
            zeros, ones = self._zeros_tab(d, x.device)
            idx0 = self._const.setdefault(("idx0", s, str(x.device)), torch.zeros(s, dtype=torch.int32, device=x.device))
            with _phase("quant_norm_mod", qbytes(d)):
                xq, xs = tq.norm_mod_rot_quant_rows_i8(x, self._norm_w(blk.norm_c), self._eps(blk.norm_c), idx0, zeros, zeros, rotate=rot)
            rec("cross_in_q", xq), rec("cross_in_s", xs)
            qw = self.cq_q.qweight_for()
            with _phase("gemm_cross", 2 * s * hd * d):
                qc = cf.int8_gemm(xq, xs, qw.q, qw.scale).view(s, c.heads, c.head_dim)
            with _phase("cross_text_kv"):
                cq8, cs = tq.rot_quant_rows_i8(ctx, rotate=rot)
                qw = self.ckv_q.qweight_for()
                kv = cf.int8_gemm(cq8, cs, qw.q, qw.scale)
                kc, vc = (t.view(ctx.shape[0], c.heads, c.head_dim) for t in kv.split(hd, dim=-1))
            if c.q_norm.eps != c.k_norm.eps:
                self._eps_mismatch()
            oc = attn_int8.attention_rr(qc, kc, vc, None, self._norm_w(c.q_norm), self._norm_w(c.k_norm), c.q_norm.eps,
                                        q_roped=qc if trace is not None else None, k_roped=kc, _tag="cross",
                                        rotate=ATTN_ROTATE)
            rec("cross_q", qc), rec("cross_k", kc), rec("cross_v", vc)
            rec("cross_out", oc)
            with _phase("quant_attn_out", qbytes(hd)):
                oq, os_ = tq.rot_quant_rows_i8(oc.view(s, hd), rotate=rot)
            qw = self.co_q.qweight_for()
            with _phase("gemm_cross", 2 * s * d * hd):
                cf.int8_gemm_gated_residual(oq, os_, qw.q, qw.scale, ones, x)
            rec("x_cross", x)

        # ---- MLP ----
        with _phase("quant_norm_mod", qbytes(d)):
            xq, xs = tq.norm_mod_rot_quant_rows_i8(x, self._norm_w(blk.norm2), self._eps(blk.norm2), idx, shift_mlp, scale_mlp, rotate=rot)
        rec("mlp_in_q", xq), rec("mlp_in_s", xs)
        w1q, w1s = self._fc1_swiglu_weight()
        with _phase("gemm_fc1_swiglu", 2 * s * 2 * f * d):
            h = cf.int8_gemm_swiglu(xq, xs, w1q, w1s)
        rec("mlp_h", h)
        with _phase("quant_fc2_in", qbytes(f)):
            hq, hs = tq.rot_quant_rows_i8(h, rotate=rot)
        rec("fc2_in_q", hq), rec("fc2_in_s", hs)
        del h
        with _phase("gemm_fc2", 2 * s * d * f):
            out = self._gemm_gated(hq, hs, self.fc2_q, x, gates_mlp, mod_segments)
        rec("x_out", out)
        return out

    __call__ = forward


def prewarm_constants(blocks, s, mod_segments, device):
    """Create, on the current stream, every tensor the fused blocks cache per (token count, device): the row index
    of the segmentation and the constant modulation tables of the cross-attention norm. A caller that is about to
    run blocks on several streams calls this first."""
    _row_index(mod_segments, s, device)
    for fb in blocks:
        if isinstance(fb, FusedBlock) and fb.cq_q is not None:
            d = fb.block.norm_c.weight.shape[0]
            fb._zeros_tab(d, device)
            fb._const.setdefault(("idx0", s, str(device)), torch.zeros(s, dtype=torch.int32, device=device))


def _fused_mlp(mlp, fc2q):
    """MLP forward for blocks whose attention linears stay unquantized: fc1 through whatever forward it has, then
    SwiGLU fused into the quantizer of fc2's input and the W8A8 GEMM (reference __init__.py:170-186)."""

    def forward(x):
        if x.dtype != torch.bfloat16 or x.device.type != "cuda":
            raise NotImplementedError("_fused_mlp: only CUDA bf16 activations are supported (no fallback path)")
        hdn = mlp.fc1(x)
        shape = hdn.shape
        qw = fc2q.qweight_for(x)
        xq, sa = tq.swiglu_rot_quant_rows_i8(hdn.reshape(-1, shape[-1]).contiguous(), rotate=fc2q.mode == "int8_rot")
        y = cf.int8_gemm(xq, sa, qw.q, qw.scale)
        if fc2q.module.bias is not None:
            y = y + fc2q.module.bias.to(y.dtype)
        return y.reshape(*shape[:-1], y.shape[-1])
    return forward


def _fused_block(block, qkv_q, out_q, fc1_q, fc2_q, cq_q=None, ckv_q=None, co_q=None):
    """The reference's factory name: returns the fused forward bound to `block`."""
    return FusedBlock(block, qkv_q, out_q, fc1_q, fc2_q, cq_q, ckv_q, co_q)


class PatchedModel:
    """What `RapidH3LinearQuant.patch` returns in place of ComfyUI's patched MODEL clone."""

    def __init__(self, model, linears, block_forward, wrappers=(), stats=None):
        self.model, self.linears, self.block_forward = model, linears, block_forward
        self.wrappers, self.stats = list(wrappers), stats if stats is not None else {}

    def __call__(self, latent, audio, t_emb, rope_freqs, ctx):
        """Runs the model with the replacement forwards installed on the modules that are not covered by a fused
        block, and removes them afterwards (the reference's wrapper, __init__.py:396-413)."""
        saved = []
        for mod, fwd in self.wrappers:
            saved.append((mod, mod.__dict__.get("forward")))
            mod.forward = fwd
        try:
            return self.model(latent, audio, t_emb, rope_freqs, ctx, block_forward=self.block_forward)
        finally:
            for mod, prev in saved:
                if prev is None:
                    mod.__dict__.pop("forward", None)
                else:
                    mod.forward = prev


def _parse_blocks(spec):
    out = set()
    for part in filter(None, (p.strip() for p in spec.split(","))):
        if "-" in part:
            a, b = part.split("-")
            out.update(range(int(a), int(b) + 1))
        else:
            out.add(int(part))
    return out


class RapidH3LinearQuant:
    """Node adapter: quantize the DiT's linears and fuse the blocks (reference __init__.py:352-417)."""

    MODES = ["bf16", "fp8_rowwise", "int8_rowwise", "int8_fast", "int8_rot"]

    def patch(self, model, mode="int8_rowwise", targets="qkv_proj,out_proj,fc1,fc2,q_proj,kv_proj",
              keep_bf16_blocks="", measure_every=0, fuse_block=True):
        if mode == "bf16":
            return (PatchedModel(model, {}, None),)
        if mode not in self.MODES:
            kernels.quantize_weight(torch.zeros(1, 8), mode)  # raises ValueError / NotImplementedError by name
        want = {t.strip() for t in targets.split(",") if t.strip()}
        keep = _parse_blocks(keep_bf16_blocks)
        by_name, stats = {}, {}
        for name, mod in model.named_modules():
            hit = NAME_RE.match(name)
            if not hit or hit.group(3) not in want or int(hit.group(1)) in keep:
                continue
            by_name[name] = _QuantLinear(mod, name, mode, measure_every, stats)
        forwards, wrappers = [], []
        for i, blk in enumerate(model.blocks):
            n = f"blocks.{i}"
            parts = [by_name.get(f"{n}.{m}") for m in ("attn.qkv_proj", "attn.out_proj", "mlp.fc1", "mlp.fc2")]
            cross = [by_name.get(f"{n}.{m}") for m in ("cross.q_proj", "cross.kv_proj", "cross.out_proj")]
            int8 = mode in ("int8_rowwise", "int8_fast", "int8_rot")
            if all(parts) and fuse_block and int8 and not measure_every:
                if hasattr(blk, "cross") and not all(cross):
                    raise NotImplementedError("fused block needs the cross-attention linears quantized as well")
                forwards.append(_fused_block(blk, *parts, *(cross if hasattr(blk, "cross") else ())))
            else:
                # stock block forward; its quantized linears (if any) replace the modules' forwards during the call,
                # and an MLP with both linears quantized gets SwiGLU fused into fc2's quantizer
                forwards.append(blk)
                mine = [(nm, q) for nm, q in by_name.items() if nm.startswith(n + ".")]
                wrappers.extend((q.module, q) for _, q in mine)
                if parts[2] and parts[3] and int8 and not measure_every:
                    wrappers.append((blk.mlp, _fused_mlp(blk.mlp, parts[3])))
        return (PatchedModel(model, by_name, forwards, wrappers, stats),)


# When set to a file path, every fused self-attention call of a FusedBlock is verified against the unfused form on
# its own q / k / v (RMSNorm + RoPE as a separate pass on copies, then the plain pre-pass and attention): the
# output and every pre-pass operand must be bit-identical. One JSON line per call is appended to the file. This is
# the reference's config-2xx self-check (`_rr_check`, __init__.py:334-349); `RapidH3Int8Attention.patch(config >= 200)`
# switches it on with the path in $RAPIDH3_RRCHECK.
RR_CHECK = None

# Which attention numerics the fused blocks and the attention override use: False = the fast kernel (block-64 Q/K,
# e4m3 V and P), True = the reference's production numerics (per-token Q/K after the 128-point Hadamard rotation,
# int8 V, u8 P against the tile maximum; attn_int8.attention(..., rotate=True)). Set by
# RapidH3Int8Attention.patch(numerics=...).
ATTN_ROTATE = False


def _rr_check(q, k, v, out, tab, qw, kw, eps, block_index=None):
    """q, k: RAW [S, H, 128] views (copies made before the fused call), v, out as the fused call saw / produced them."""
    import json
    qc = attn_int8.rms_rope(q, qw, eps, tab)
    kc = attn_int8.rms_rope(k, kw, eps, tab)
    plain = attn_int8.int8_prepass(qc, kc, v)
    fused = attn_int8.int8_prepass(q, k, v, tab, qw, kw, eps)
    ref = attn_int8.attention_pre(plain)
    names = ("q8", "qs", "k8", "ks", "vt", "vscale", "vmean", "kmean")
    rec = {"block": block_index, "S": int(q.shape[0]), "out_equal": bool(torch.equal(ref, out)),
           "operands_equal": all(torch.equal(getattr(plain, n).view(torch.uint8), getattr(fused, n).view(torch.uint8))
                                 for n in names),
           "max_abs_diff": float((ref.float() - out.float()).abs().max())}
    with open(RR_CHECK, "a") as f:
        f.write(json.dumps(rec) + "\n")
    return rec


class RapidH3Int8Attention:
    """Node adapter: returns the attention override the reference installs in transformer_options
    (reference __init__.py:995-1047). The override takes the calls the reference's INT8 path takes (no mask,
    `skip_reshape`, q, k, v all [1, H, S, 128] bf16 with S >= 1024) and hands every other call on to the override
    that was installed before it, or to the framework's own attention function `func`, exactly as the reference
    does: those calls were never this node's. `exact_rows` names segment kinds of the packed layout
    (transformer_options["minimax_h3_layout"].segments = [(start, stop, kind)]) whose query rows are recomputed
    with bf16 scaled-dot-product attention after the INT8 kernel has run (the reference's patch-up, :1035-1037)."""

    NUMERICS = ["fast", "reference"]

    def patch(self, model, config=80, exact_rows="", previous=None, numerics="fast"):
        """`numerics`: "fast" = the block-64 / e4m3 kernel (the reference's FP8-P.V family, its configs 50-56);
        "reference" = the token-scaled kernel with the arithmetic of the reference's production configs
        (80 / 90 / 94 and their 1xx / 2xx forms). The choice also applies to the fused blocks' own attention calls."""
        global RR_CHECK, ATTN_ROTATE
        if numerics not in self.NUMERICS:
            raise ValueError(numerics)
        ATTN_ROTATE = rotate = numerics == "reference"
        import os
        import torch.nn.functional as F
        exact = {t.strip() for t in exact_rows.split(",") if t.strip()}
        rmsrope = config >= 100 and not exact
        if config >= 200:
            RR_CHECK = os.environ.get("RAPIDH3_RRCHECK", "rapidh3_rrcheck.jsonl")
        config = config % 100

        def exact_spans(options, s):
            layout = (options or {}).get("minimax_h3_layout")
            if layout is None or getattr(layout, "seq_len", None) != s:
                return []
            spans = []
            for a, b, kind in layout.segments:
                if kind in exact and b > a:
                    if spans and spans[-1][1] == a:
                        spans[-1][1] = b       # adjacent spans are recomputed in one call
                    else:
                        spans.append([a, b])
            return spans

        def override(func, q, k, v, heads=None, mask=None, skip_reshape=False, skip_output_reshape=False, scale=None,
                     **kwargs):
            ours = (mask is None and skip_reshape and q.dim() == 4 and q.shape[0] == 1 and q.shape == k.shape == v.shape
                    and q.shape[-1] == 128 and q.shape[2] >= 1024 and q.dtype == torch.bfloat16 and q.is_cuda)
            if not ours:
                rest = dict(heads=heads, mask=mask, skip_reshape=skip_reshape, skip_output_reshape=skip_output_reshape,
                            scale=scale, **kwargs)
                return previous(func, q, k, v, **rest) if previous else func(q, k, v, **rest)
            out = torch.empty_like(q)
            attn_int8.attention(q[0].transpose(0, 1), k[0].transpose(0, 1), v[0].transpose(0, 1), scale, config=config,
                                rotate=rotate, out=out[0].transpose(0, 1))
            for a, b in exact_spans(kwargs.get("transformer_options"), q.shape[2]):
                out[:, :, a:b] = F.scaled_dot_product_attention(q[:, :, a:b], k, v, scale=scale)
            return out if skip_output_reshape else out.transpose(1, 2).reshape(1, q.shape[2], -1)

        override.rapidh3_rmsrope = config if rmsrope else None
        override.rapidh3_rrcheck = RR_CHECK is not None
        return (model, override)


NODE_CLASS_MAPPINGS = {"RapidH3LinearQuant": RapidH3LinearQuant, "RapidH3Int8Attention": RapidH3Int8Attention}
