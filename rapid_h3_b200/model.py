"""A minimal H3-shaped DiT (the stand-in for ComfyUI's `comfy.ldm.minimax.model`, which is not
available outside ComfyUI): the module surface the Rapid-H3 node pack reads from a DiT block
(`adaln_proj`, `norm1/norm2`, `attn.{qkv_proj,out_proj,q_norm,k_norm,heads,head_dim}`,
`mlp.{fc1,fc2}`; reference: custom_nodes/rapid_h3/__init__.py:207-321) plus the cross-attention to
text tokens that the benchmark configuration adds (`norm_c`, `cross.{q_proj,kv_proj,out_proj,
q_norm,k_norm}`).

`DiTBlock.forward` / `H3Transformer.forward` are the STOCK bf16 path (torch linears, fp32-softmax
attention). They exist as the unquantized yardstick of the step-divergence check and as the thing
the node adapters patch; the product path is rapid_h3_b200.nodes.FusedBlock.
"""
import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class H3Config:
    d_model: int = 4096
    heads: int = 32
    head_dim: int = 128
    mlp_hidden: int = 16384
    n_blocks: int = 48
    text_dim: int = 4096
    latent_ch: int = 16
    norm_eps: float = 1e-6
    qk_eps: float = 1e-5
    cross_attention: bool = True

    @staticmethod
    def tiny(**kw):
        base = dict(d_model=256, heads=2, mlp_hidden=512, n_blocks=2, text_dim=128, latent_ch=16)
        base.update(kw)
        return H3Config(**base)


class RMSNorm(nn.Module):
    def __init__(self, dim, eps):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=torch.bfloat16), requires_grad=False)
        self.eps = eps

    def forward(self, x):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight.float()).to(x.dtype)


def _linear(i, o, bias=False):
    lin = nn.Linear(i, o, bias=bias, dtype=torch.bfloat16)
    lin.requires_grad_(False)
    return lin


class AdaLN(nn.Module):
    """t_emb [R, d] -> six fp32 [R, d] tables (shift/scale/gate for attention and MLP), views of one [R, 6d]."""

    def __init__(self, d):
        super().__init__()
        self.proj = _linear(d, 6 * d, bias=True)

    def forward(self, t_emb):
        return self.proj(F.silu(t_emb)).float().chunk(6, dim=-1)


def apply_rope(x, tab):
    """x [S, H, 128] fp32, tab [S, 48, 2, 2]: split-half partial rotation of the first 96 channels."""
    t = tab.float().view(x.shape[0], 1, 48, 2, 2)
    a, b = x[..., :48], x[..., 48:96]
    return torch.cat([a * t[..., 0, 0] + b * t[..., 0, 1], a * t[..., 1, 0] + b * t[..., 1, 1], x[..., 96:]], -1)


def sdpa_fp32(q, k, v, scale=None):
    """q [Lq, H, 128], k, v [Lk, H, 128] -> [Lq, H, 128]; softmax in fp32, rows processed in chunks."""
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    qh, kh, vh = (t.transpose(0, 1).float() for t in (q, k, v))
    out = torch.empty_like(qh)
    for r in range(0, qh.shape[1], 2048):
        s = torch.matmul(qh[:, r:r + 2048], kh.transpose(1, 2)) * scale
        out[:, r:r + 2048] = torch.matmul(torch.softmax(s, -1), vh)
    return out.transpose(0, 1).to(q.dtype)


class SelfAttention(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        d = cfg.d_model
        self.heads, self.head_dim = cfg.heads, cfg.head_dim
        self.qkv_proj, self.out_proj = _linear(d, 3 * d), _linear(d, d)
        self.q_norm, self.k_norm = RMSNorm(cfg.head_dim, cfg.qk_eps), RMSNorm(cfg.head_dim, cfg.qk_eps)

    def forward(self, h, rope):
        s = h.shape[0]
        q, k, v = (t.view(s, self.heads, self.head_dim) for t in self.qkv_proj(h).chunk(3, -1))
        q = apply_rope(self.q_norm(q).float(), rope).to(h.dtype)
        k = apply_rope(self.k_norm(k).float(), rope).to(h.dtype)
        return self.out_proj(sdpa_fp32(q, k, v).reshape(s, -1))


class CrossAttention(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        d = cfg.d_model
        self.heads, self.head_dim = cfg.heads, cfg.head_dim
        self.q_proj, self.kv_proj, self.out_proj = _linear(d, d), _linear(cfg.text_dim, 2 * d), _linear(d, d)
        self.q_norm, self.k_norm = RMSNorm(cfg.head_dim, cfg.qk_eps), RMSNorm(cfg.head_dim, cfg.qk_eps)

    def forward(self, h, ctx):
        s, t = h.shape[0], ctx.shape[0]
        q = self.q_norm(self.q_proj(h).view(s, self.heads, self.head_dim))
        k, v = (u.view(t, self.heads, self.head_dim) for u in self.kv_proj(ctx).chunk(2, -1))
        return self.out_proj(sdpa_fp32(q, self.k_norm(k), v).reshape(s, -1))


class MLP(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.fc1, self.fc2 = _linear(cfg.d_model, 2 * cfg.mlp_hidden), _linear(cfg.mlp_hidden, cfg.d_model)

    def forward(self, h):
        g, u = self.fc1(h).chunk(2, -1)
        return self.fc2(F.silu(g) * u)


def row_index(segments, s, device):
    """Per-token modulation-row index (int32 [S]) from [(start, stop, row)]."""
    idx = torch.empty(s, dtype=torch.int32, device=device)
    for a, b, row in segments:
        idx[a:b] = int(row)
    return idx


class DiTBlock(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.cfg = cfg
        d = cfg.d_model
        self.adaln_proj = AdaLN(d)
        self.norm1, self.norm2 = RMSNorm(d, cfg.norm_eps), RMSNorm(d, cfg.norm_eps)
        self.attn, self.mlp = SelfAttention(cfg), MLP(cfg)
        if cfg.cross_attention:
            self.norm_c, self.cross = RMSNorm(d, cfg.norm_eps), CrossAttention(cfg)

    def forward(self, x, t_emb, mod_segments, rope_freqs, ctx=None):
        """x [S, d] bf16 packed sequence; t_emb [R, d]; mod_segments [(start, stop, row)];
        rope_freqs bf16 [.., S, .., 48, 2, 2]; ctx [T, text_dim] text tokens."""
        sh1, sc1, g1, sh2, sc2, g2 = self.adaln_proj(t_emb)
        idx = row_index(mod_segments, x.shape[0], x.device).long()
        rope = rope_freqs.reshape(x.shape[0], 48, 2, 2)

        def mod(norm, shift, scale):
            return (norm(x).float() * (1 + scale[idx]) + shift[idx]).to(x.dtype)

        x = torch.addcmul(x, self.attn(mod(self.norm1, sh1, sc1), rope), g1[idx].to(x.dtype))
        if self.cfg.cross_attention:
            x = x + self.cross(self.norm_c(x), ctx)
        return torch.addcmul(x, self.mlp(mod(self.norm2, sh2, sc2)), g2[idx].to(x.dtype))


class H3Transformer(nn.Module):
    """Token embedding of the latent grid, n_blocks DiT blocks, final norm + projection back to latent
    channels. The latent grid [C, T, H, W] is taken as the token grid (one token per latent site)."""

    def __init__(self, cfg):
        super().__init__()
        self.cfg = cfg
        self.embed = _linear(cfg.latent_ch, cfg.d_model, bias=True)
        self.audio_embed = _linear(cfg.latent_ch, cfg.d_model, bias=True)
        self.blocks = nn.ModuleList([DiTBlock(cfg) for _ in range(cfg.n_blocks)])
        self.final_norm = RMSNorm(cfg.d_model, cfg.norm_eps)
        self.unembed = _linear(cfg.d_model, cfg.latent_ch, bias=True)
        self.audio_unembed = _linear(cfg.d_model, cfg.latent_ch, bias=True)

    def tokens(self, latent, audio):
        """latent [C, T, H, W], audio [A, C] -> packed [T*H*W + A, d] bf16."""
        v = self.embed(latent.flatten(1).t().to(torch.bfloat16))
        if audio is None or audio.shape[0] == 0:
            return v
        return torch.cat([v, self.audio_embed(audio.to(torch.bfloat16))], 0)

    def untokens(self, x, latent_shape):
        n_video = latent_shape[1] * latent_shape[2] * latent_shape[3]
        h = self.final_norm(x)
        video = self.unembed(h[:n_video]).t().reshape(latent_shape)
        audio = self.audio_unembed(h[n_video:])
        return video, audio

    def forward(self, latent, audio, t_emb, rope_freqs, ctx, block_forward=None):
        x = self.tokens(latent, audio)
        n_video = x.shape[0] - (0 if audio is None else audio.shape[0])
        segs = [(0, n_video, 0)] + ([(n_video, x.shape[0], 1)] if x.shape[0] > n_video else [])
        for i, blk in enumerate(self.blocks):
            fwd = blk if block_forward is None else block_forward[i]
            x = fwd(x, t_emb, segs, rope_freqs, ctx)
        return self.untokens(x, latent.shape)


def init_weights(module, seed, device=None):
    """Random init of the benchmark configurations: Linear weights ~ N(0, 0.02), biases ~ N(0, 0.01),
    d-wide norm weights 1 + 0.1 N(0,1), per-head q/k norm weights 1 + 0.3 N(0,1). Generated on CPU so the
    oracle sees the same values; AdaLN projections are scaled so the modulation tables are ~ N(0, 0.1)."""
    g = torch.Generator().manual_seed(seed)
    for name, p in module.named_parameters():
        if name.endswith("norm.weight") and p.numel() == 128:
            v = 1 + 0.3 * torch.randn(p.shape, generator=g)
        elif "norm" in name:
            v = 1 + 0.1 * torch.randn(p.shape, generator=g)
        elif name.endswith("bias"):
            v = 0.01 * torch.randn(p.shape, generator=g)
        elif "adaln_proj" in name:
            v = torch.randn(p.shape, generator=g) * (0.1 / math.sqrt(p.shape[1]) / 0.6)
        else:
            v = 0.02 * torch.randn(p.shape, generator=g)
        p.data.copy_(v.to(p.dtype))
    return module if device is None else module.to(device)


def init_weights_on_device(module, generator, skip_prefix=None):
    """Same distributions as init_weights, generated on the parameters' own device (for the full-size model)."""
    dev = generator.device
    for name, p in module.named_parameters():
        if skip_prefix and name.startswith(skip_prefix):
            continue
        if name.endswith("norm.weight") and p.numel() == 128:
            v = 1 + 0.3 * torch.randn(p.shape, generator=generator, device=dev)
        elif "norm" in name:
            v = 1 + 0.1 * torch.randn(p.shape, generator=generator, device=dev)
        elif name.endswith("bias"):
            v = 0.01 * torch.randn(p.shape, generator=generator, device=dev)
        elif "adaln_proj" in name:
            v = torch.randn(p.shape, generator=generator, device=dev) * (0.1 / math.sqrt(p.shape[1]) / 0.6)
        else:
            v = 0.02 * torch.randn(p.shape, generator=generator, device=dev)
        p.data.copy_(v.to(p.dtype))
    return module
