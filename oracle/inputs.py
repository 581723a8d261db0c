"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations
(TEST INFRASTRUCTURE ONLY). Generators run on CPU so the oracle and the kernels see identical bits.
Distributions follow the reference's own generators: bench/int8_bench.py:39-41 (outlier channels),
bench/rmsrope_fuse.py:22-54 (rope table, qkv buffer, norm weights), bench/attn_cake.py:20-35.
"""
import math

import torch


def gen(seed):
    return torch.Generator().manual_seed(seed)


def linear_case(m=4096, k=4096, n=4096, seed=0, outlier_frac=0.01, outlier_scale=20.0):
    """X ~ N(0,1) with 1% of channels x20, W ~ N(0,0.02), bias ~ N(0,0.01); all bf16."""
    g = gen(seed)
    x = torch.randn(m, k, generator=g)
    n_out = int(outlier_frac * k)
    if n_out:
        ch = torch.randperm(k, generator=g)[:n_out]
        x[:, ch] *= outlier_scale
    w = torch.randn(n, k, generator=g) * 0.02
    b = torch.randn(n, generator=g) * 0.01
    return x.to(torch.bfloat16), w.to(torch.bfloat16), b.to(torch.bfloat16)


def rope_positions_grid(t, h, w, n_audio=0):
    """(t, h, w) position of every token of a T x H x W latent grid, then n_audio audio tokens
    that advance along t only."""
    tt, hh, ww = torch.meshgrid(torch.arange(t), torch.arange(h), torch.arange(w), indexing="ij")
    pos = torch.stack([tt.reshape(-1), hh.reshape(-1), ww.reshape(-1)], 1).double()
    if n_audio:
        a = torch.zeros(n_audio, 3, dtype=torch.float64)
        a[:, 0] = torch.arange(n_audio, dtype=torch.float64) * (t / max(n_audio, 1))
        pos = torch.cat([pos, a], 0)
    return pos


def rope_table(pos):
    """bf16 [S, 48, 2, 2] rotation table = (cos, -sin, sin, cos) for rot_dim 96: 3 axes x 16
    frequencies, first half of every axis then repeated (split-half layout)."""
    pos = pos.to(torch.float32)
    inv = 1.0 / (10000.0 ** (torch.arange(16, dtype=torch.float32) / 16))
    half = torch.cat((pos.unsqueeze(-1) * inv.view(1, 1, -1)).unbind(1), -1)  # [S, 48]
    c, s = torch.cos(half), torch.sin(half)
    return torch.stack([c, -s, s, c], -1).reshape(pos.shape[0], 48, 2, 2).to(torch.bfloat16)


def random_positions(s, seed=0):
    g = gen(seed)
    t = torch.randint(0, 40, (s,), generator=g).double() * (5.0 / 3.0)
    hh = torch.rand(s, generator=g, dtype=torch.float64) * 32
    ww = torch.rand(s, generator=g, dtype=torch.float64) * 32
    return torch.stack([t, hh, ww], 1)


def norm_weights(seed=1, d=128):
    g = gen(seed)
    return tuple((1 + 0.3 * torch.randn(d, generator=g)).to(torch.bfloat16) for _ in range(2))


def attention_case(l, h, seed=0, d=128, k_offset_std=2.0):
    """Q, K, V bf16 [L, H, D] ~ N(0,1); K gets a per-(head, channel) offset ~ N(0, k_offset_std)."""
    g = gen(seed)
    q = torch.randn(l, h, d, generator=g)
    k = torch.randn(l, h, d, generator=g) + k_offset_std * torch.randn(1, h, d, generator=g)
    v = torch.randn(l, h, d, generator=g)
    return q.to(torch.bfloat16), k.to(torch.bfloat16), v.to(torch.bfloat16)


def attention_outlier_case(l, h, seed=0, d=128, device="cpu"):
    """The value distribution of the reference's synthetic attention benchmark (bench/attn_cake.py:20-35): N(0,1) q
    and k times 1.6, four outlier channels per head scaled by 3 that also carry a per-head K offset ~ 6 N(0,1), V with a
    per-channel scale in [1, 2) and a heavy tail 0.05 N(0,1)^3. bf16 [L, H, D]."""
    g = torch.Generator(device=device).manual_seed(seed)
    q = torch.randn(l, h, d, generator=g, device=device)
    k = torch.randn(l, h, d, generator=g, device=device)
    idx = torch.randint(0, d, (h, 4), generator=g, device=device)
    kbias = torch.zeros(1, h, d, device=device)
    kbias.scatter_(2, idx.view(1, h, 4), 6.0 * torch.randn(1, h, 4, generator=g, device=device))
    boost = torch.ones(1, h, d, device=device)
    boost.scatter_(2, idx.view(1, h, 4), 3.0)
    q = q * boost * 1.6
    k = k * boost * 1.6 + kbias
    v = torch.randn(l, h, d, generator=g, device=device) * (1 + torch.rand(1, h, d, generator=g, device=device))
    v = v + 0.05 * torch.randn(l, h, d, generator=g, device=device).pow(3)
    return q.to(torch.bfloat16), k.to(torch.bfloat16), v.to(torch.bfloat16)


def softmax_scale(d=128):
    return 1.0 / math.sqrt(d)
