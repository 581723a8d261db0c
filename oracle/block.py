"""Oracle: one fused DiT block on CPU from the oracle primitives (TEST INFRASTRUCTURE ONLY).

Restates the graph of the reference's `_fused_block` (custom_nodes/rapid_h3/__init__.py:253-320):
norm+modulation quantizer -> qkv GEMM -> per-head RMSNorm + RoPE -> attention -> quantizer ->
out_proj GEMM with gated residual per modality segment -> norm+modulation quantizer -> fc1 GEMM with
SwiGLU epilogue -> quantizer -> fc2 GEMM with gated residual. The cross-attention to text tokens has no
counterpart in the reference (parity unpinned); it is built from the same quantized primitives.
`block` is a rapid_h3_b200.model.DiTBlock held on the CPU (only its parameters are read).
"""
import torch

from . import attention as oa
from . import attention_tok as ot
from . import linear as ol
from . import quant as oq


def _qlinear(x, weight):
    wq, ws = ol.quantize_weight(weight, "int8_rowwise")
    xq, xs = ol.quantize_rows(x, "int8_rowwise")
    return ol.int_mm(xq, wq), xs, ws


def fused_block(block, x, t_emb, mod_segments, rope_freqs, ctx=None, trace=None, mode="int8_rowwise", adaln=None,
                replay=None, attn="fast"):
    """`attn`: "fast" = the block-64 / e4m3 attention (oracle.attention), "token" = the token-scaled one
    (oracle.attention_tok), for self- and cross-attention alike.
    `adaln`: the six fp32 modulation tables, when the caller wants the block checked on given tables (the AdaLN
    projection is a plain bf16 matrix product of the host framework whose summation order differs between devices;
    it is an input of the quantized path, not part of it).
    `replay`: {"x_attn": ..., "x_cross": ...}: residual streams to start the cross-attention and the MLP stage from,
    instead of this function's own (a checker passes what the device produced, so that every stage is compared on
    identical inputs and a last-bit difference of one stage is not amplified through the next quantizer)."""
    s, d = x.shape
    attention = {"fast": oa.attention, "token": ot.attention}[attn]
    a = block.attn
    hd = a.heads * a.head_dim
    sh1, sc1, g1, sh2, sc2, g2 = block.adaln_proj(t_emb) if adaln is None else adaln
    idx = torch.empty(s, dtype=torch.int32)
    for lo, hi, row in mod_segments:
        idx[lo:hi] = int(row)
    tab = rope_freqs.reshape(s, 48, 2, 2)
    x = x.clone()
    rot = mode == "int8_rot"
    norm_mod_q = oq.norm_mod_rot_quant_rows_i8 if rot else oq.norm_mod_quant_rows_i8

    def rec(name, value):
        if trace is not None:
            trace[name] = value.clone()

    def gated(acc, xs, ws, gate_tab, x):
        for lo, hi, row in mod_segments:
            if hi > lo:
                x[lo:hi] = ol.gated_residual(acc[lo:hi], xs[lo:hi], ws, gate_tab[int(row)].to(torch.bfloat16), x[lo:hi])
        return x

    def q_weight(lin):
        return ol.quantize_weight(lin.weight.detach(), mode)

    # self-attention
    xq, xs = norm_mod_q(x, block.norm1.weight.detach(), block.norm1.eps, idx, sh1, sc1)
    rec("attn_in_q", xq), rec("attn_in_s", xs)
    wq, ws = q_weight(a.qkv_proj)
    qkv = ol.dequant(ol.int_mm(xq, wq), xs, ws)
    rec("qkv", qkv)
    q, k, v = (t.reshape(s, a.heads, a.head_dim) for t in qkv.split(hd, dim=-1))
    q = oa.rmsnorm_rope(q, a.q_norm.weight.detach(), a.q_norm.eps, tab)
    k = oa.rmsnorm_rope(k, a.k_norm.weight.detach(), a.k_norm.eps, tab)
    rec("qkv_rr", torch.cat([q.reshape(s, hd), k.reshape(s, hd), v.reshape(s, hd)], 1))
    o = attention(q, k, v)
    rec("attn_out", o)
    oq8, os_ = ol.quantize_rows(o.reshape(s, hd), mode)
    wq, ws = q_weight(a.out_proj)
    x = gated(ol.int_mm(oq8, wq), os_, ws, g1, x)
    rec("x_attn", x)
    if replay is not None and "x_attn" in replay:
        x = replay["x_attn"].clone()

    if hasattr(block, "cross"):
        c = block.cross
        zeros = torch.zeros(1, d)
        xq, xs = norm_mod_q(x, block.norm_c.weight.detach(), block.norm_c.eps,
                                           torch.zeros(s, dtype=torch.int32), zeros, zeros)
        rec("cross_in_q", xq), rec("cross_in_s", xs)
        wq, ws = q_weight(c.q_proj)
        qc = ol.dequant(ol.int_mm(xq, wq), xs, ws).reshape(s, c.heads, c.head_dim)
        cq8, cs = ol.quantize_rows(ctx, mode)
        wq, ws = q_weight(c.kv_proj)
        kv = ol.dequant(ol.int_mm(cq8, wq), cs, ws)
        kc, vc = (t.reshape(ctx.shape[0], c.heads, c.head_dim) for t in kv.split(hd, dim=-1))
        qc = oa.rmsnorm_rope(qc, c.q_norm.weight.detach(), c.q_norm.eps, None)
        kc = oa.rmsnorm_rope(kc, c.k_norm.weight.detach(), c.k_norm.eps, None)
        rec("cross_q", qc), rec("cross_k", kc), rec("cross_v", vc)
        oc = attention(qc, kc, vc)
        rec("cross_out", oc)
        oq8, os_ = ol.quantize_rows(oc.reshape(s, hd), mode)
        wq, ws = q_weight(c.out_proj)
        x = ol.gated_residual(ol.int_mm(oq8, wq), os_, ws, torch.ones(d, dtype=torch.bfloat16), x)
        rec("x_cross", x)
        if replay is not None and "x_cross" in replay:
            x = replay["x_cross"].clone()

    xq, xs = norm_mod_q(x, block.norm2.weight.detach(), block.norm2.eps, idx, sh2, sc2)
    rec("mlp_in_q", xq), rec("mlp_in_s", xs)
    wq, ws = q_weight(block.mlp.fc1)
    perm = ol.swiglu_perm(wq.shape[0])
    h = ol.swiglu_epilogue(ol.int_mm(xq, wq[perm]), xs, ws[:, perm])
    rec("mlp_h", h)
    if replay is not None and "mlp_h" in replay:
        h = replay["mlp_h"].clone()
    hq, hs = ol.quantize_rows(h, mode)
    rec("fc2_in_q", hq), rec("fc2_in_s", hs)
    wq, ws = q_weight(block.mlp.fc2)
    x = gated(ol.int_mm(hq, wq), hs, ws, g2, x)
    rec("x_out", x)
    return x
