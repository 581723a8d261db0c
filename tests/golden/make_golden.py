"""Generates tests/golden/linear_ref.pt by importing the reference's own PyTorch emulation
(custom_nodes/rapid_h3/kernels.py of jeet0733/Rapid-H3) on CPU. Run where the reference tree is
mounted:

    python tests/golden/make_golden.py /path/to/Rapid-H3

The fixture holds small seeded inputs and the reference's outputs for quantize_rows,
quantize_weight and linear in the int8_rowwise and fp8_rowwise(_torch) modes, plus the un-rotated
pieces of the fused-quantizer fp32 expression of bench/rot_test.py:42-51.
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


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/Rapid-H3")
    main(sys.argv[1])
