"""The CPU oracle of the token-scaled attention against first principles (no GPU): the rotation, the operand
layout, and the distance of the quantized result from exact attention."""
import math

import torch

from oracle import attention as oa
from oracle import attention_tok as ot
from oracle import inputs


def test_hadamard128_is_symmetric_orthogonal_times_sqrt128():
    h = ot.hadamard128(torch.eye(128))
    assert torch.equal(h.abs(), torch.ones(128, 128)) and torch.equal(h, h.t())
    assert torch.equal(h @ h, 128.0 * torch.eye(128))
    g = inputs.gen(1)
    q, k = torch.randn(7, 128, generator=g).to(torch.bfloat16), torch.randn(9, 128, generator=g).to(torch.bfloat16)
    exact = q.double() @ k.double().t()
    rot = ot.hadamard128(q).double() @ ot.hadamard128(k).double().t() / 128.0
    assert torch.allclose(rot, exact, rtol=0, atol=1e-4)      # Q.K^T is unchanged up to the factor 128


def test_operands_layout_and_padding():
    q, _, _ = inputs.attention_case(300, 2, seed=3)
    _, k, v = inputs.attention_case(200, 2, seed=4)
    pre = ot.prepass(q, k, v)
    assert pre["q8"].shape == (2, 512, 128) and pre["k8"].shape == (2, 256, 128) and pre["vt"].shape == (2, 128, 256)
    assert pre["qs"].shape == (2, 512) and pre["ksb"].shape == (2, 2, 2, 128)
    assert not pre["q8"][:, 300:].any() and not pre["k8"][:, 200:].any() and not pre["vt"][:, :, 200:].any()
    bias = pre["ksb"][:, :, 1].reshape(2, 256)
    assert (bias[:, :200] == 0).all() and torch.isinf(bias[:, 200:]).all() and (bias[:, 200:] < 0).all()
    assert (pre["ksb"][:, :, 0].reshape(2, 256)[:, 200:] == 0).all()
    # every token row uses the full code range: its largest code is 127 in magnitude
    assert (pre["q8"][:, :300].abs().amax(-1) == 127).all() and (pre["k8"][:, :200].abs().amax(-1) == 127).all()
    assert pre["vt"].abs().max() <= 127 and (pre["vt"][:, :, :200].abs().amax(-1) == 127).all()


def test_token_scaled_attention_is_closer_to_exact_attention_than_the_e4m3_variant():
    q, _, _ = inputs.attention_case(256, 2, seed=5)
    _, k, v = inputs.attention_case(700, 2, seed=6)
    full = oa.attention_fp32(q, k, v)
    err_tok = ((ot.attention(q, k, v).float() - full).norm() / full.norm()).item()
    err_fast = ((oa.attention(q, k, v).float() - full).norm() / full.norm()).item()
    assert err_tok < 0.02 and err_tok < 0.5 * err_fast


def test_one_dominant_key_in_the_first_tile_does_not_erase_the_later_tiles():
    """8-bit P against the RUNNING maximum would round every weight of the later tiles to zero here; against each
    tile's own maximum they survive (the reason for the per-tile fold, custom_nodes/rapid_h3/csrc/README.md)."""
    g = inputs.gen(12)
    q = torch.randn(64, 1, 128, generator=g).to(torch.bfloat16)
    k = 0.05 * torch.randn(1024, 1, 128, generator=g)
    k[3] = 0.6 * q[:, 0].float().mean(0, keepdim=True) + 0.3 * torch.randn(1, 128, generator=g)
    k = k.to(torch.bfloat16)
    v = torch.randn(1024, 1, 128, generator=g).to(torch.bfloat16)
    full = oa.attention_fp32(q, k, v)
    out = ot.attention(q, k, v)
    assert ((out.float() - full).norm() / full.norm()).item() < 0.02
    w = torch.softmax((q[:, 0].float() @ k[:, 0].float().t()) / math.sqrt(128), -1)
    assert w[:, 128:].sum(1).mean() > 0.3      # the later tiles do carry weight in this case
