"""Generates tests/golden/linear_ref.pt by importing the reference's own PyTorch emulation
(custom_nodes/rapid_h3/kernels.py of jeet0733/Rapid-H3) on CPU. Run where the reference tree is
mounted:

    python tests/golden/make_golden.py /path/to/Rapid-H3

linear_ref.pt holds small seeded inputs and the reference's outputs for quantize_rows,
quantize_weight and linear in the int8_rowwise and fp8_rowwise(_torch) modes, plus the un-rotated
pieces of the fused-quantizer fp32 expression of bench/rot_test.py:42-51.

rot_ref.pt holds what the reference's own H256 ConvRot code gives on CPU: the matrix
`triton_fp8.regular_hadamard(256)`, `triton_fp8.convrot(x)` of seeded activations, the yardstick
quantizer of bench/rot_test.py:16-19 on them, and `kernels.quantize_weight(w, "int8_rot")`.

tensor_ref.pt holds `kernels.quantize_weight(w, "fp8_tensor")` and `kernels.linear(x, qw, "fp8_tensor")`
(kernels.py:63-65, :125-128) of one seeded case.

attn_ref.pt holds the operand fake-quantizers of bench/attn_emulate.py (`q8(x, 1, 64)`, `f8(x, 0)`,
:10-23) applied to seeded q / k - kmean / v - vmean, and the output of its `attn(..., pmode="run_fp8")`
(:33-65) on those operands. The K / V channel means are an input of those functions; they are taken
from the oracle's fixed-order statistics and stored with the fixture, so that both sides quantize the
same numbers.
"""
import os
import sys

import torch


def main(ref_root):
    sys.path.insert(0, os.path.join(ref_root, "custom_nodes", "rapid_h3"))
    import kernels as ref  # the reference module

    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, os.path.dirname(os.path.dirname(here)))
    from oracle import inputs

    out = {}
    for name, (m, k, n, seed) in {"a": (96, 256, 128, 0), "b": (50, 512, 136, 3)}.items():
        x, w, b = inputs.linear_case(m, k, n, seed=seed, outlier_frac=0.02)
        if name == "b":
            x[5] = 0  # an all-zero row exercises the 1e-12 scale clamp
        case = {"x": x, "w": w, "b": b}
        for mode, emu_mode in (("int8_rowwise", "int8_rowwise"), ("fp8_rowwise", "fp8_rowwise_torch")):
            xq, xs = ref.quantize_rows(x, mode)
            qw = ref.quantize_weight(w, mode)
            y = ref.linear(x, qw, emu_mode)
            case[mode] = {"xq": xq.view(torch.uint8) if xq.dtype != torch.int8 else xq, "xs": xs,
                          "wq": qw.q.view(torch.uint8) if qw.q.dtype != torch.int8 else qw.q, "ws": qw.scale,
                          "y": y}
        out[name] = case
    path = os.path.join(here, "linear_ref.pt")
    torch.save(out, path)
    print(path, os.path.getsize(path), "bytes")
    rot_fixture(ref, here)
    attn_fixture(ref_root, here)
    tensor_fixture(ref, here)


def rot_fixture(ref, here):
    """H256 ConvRot through the reference's own functions (triton_fp8.py:70-90, kernels.py:58-60)."""
    tq = ref._tq
    g = torch.Generator().manual_seed(11)
    x = torch.randn(24, 768, generator=g)
    x[:, :6] *= 20                                   # outlier channels, as bench/rot_test.py:31
    x = x.to(torch.bfloat16)
    w = (0.02 * torch.randn(40, 512, generator=g)).to(torch.bfloat16)
    r = tq.convrot(x.float())
    s = (r.abs().amax(dim=1, keepdim=True) / 127).clamp_min(1e-12)     # bench/rot_test.py:16-19
    qw = ref.quantize_weight(w, "int8_rot")
    out = {"h256": tq.regular_hadamard(256, "cpu", torch.float32), "x": x, "x_rot": r,
           "x_q": (r / s).round().clamp(-127, 127).to(torch.int8), "x_s": s,
           "w": w, "w_q": qw.q, "w_s": qw.scale}
    path = os.path.join(here, "rot_ref.pt")
    torch.save(out, path)
    print(path, os.path.getsize(path), "bytes")


def tensor_fixture(ref, here):
    """The per-tensor FP8 mode through the reference's own branches (kernels.py:63-65 and :125-128)."""
    from oracle import inputs
    x, w, _ = inputs.linear_case(72, 384, 136, seed=5, outlier_frac=0.02)
    qw = ref.quantize_weight(w, "fp8_tensor")
    out = {"x": x, "w": w, "wq": qw.q.view(torch.uint8), "ws": qw.scale, "y": ref.linear(x, qw, "fp8_tensor")}
    path = os.path.join(here, "tensor_ref.pt")
    torch.save(out, path)
    print(path, os.path.getsize(path), "bytes")


def attn_fixture(ref_root, here):
    """Block-64 Q/K and e4m3-V operands and the `run_fp8` attention of bench/attn_emulate.py."""
    sys.path.insert(0, os.path.join(ref_root, "bench"))
    import attn_emulate as emu
    from oracle import attention as oa

    g = torch.Generator().manual_seed(5)
    l, h = 200, 2                                    # 200 = three full 64-token blocks and a ragged one
    q = torch.randn(l, h, 128, generator=g).to(torch.bfloat16)
    k = (torch.randn(l, h, 128, generator=g) + 2 * torch.randn(1, h, 128, generator=g)).to(torch.bfloat16)
    v = (torch.randn(l, h, 128, generator=g) + 0.5 * torch.randn(1, h, 128, generator=g)).to(torch.bfloat16)
    kmean, vmean, _ = oa.kv_stats(k, v)
    out = {"q": q, "k": k, "v": v, "kmean": kmean, "vmean": vmean, "heads": []}
    for hh in range(h):
        qq = emu.q8(q[:, hh].float(), 1, 64)
        kq = emu.q8(k[:, hh].float() - kmean[hh][None], 1, 64)
        vq = emu.f8(v[:, hh].float() - vmean[hh][None], 0)
        o = emu.attn(qq, kq, vq + vmean[hh][None], pmode="run_fp8")
        o_exact_p = emu.attn(qq, kq, vq + vmean[hh][None])
        out["heads"].append({"q_fq": qq, "k_fq": kq, "v_fq": vq, "out_run_fp8": o, "out_exact_p": o_exact_p})
    path = os.path.join(here, "attn_ref.pt")
    torch.save(out, path)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/Rapid-H3")
    main(sys.argv[1])
