"""rapid_h3_b200: the quantized DiT step of the Rapid-H3 node pack, rebuilt for B200 (sm_100a).

Python host code over a C-ABI CUDA library (librapidh3_b200.so). Importing the package does not
load the library; the first operator call does, and raises if it is missing.
"""
from . import _lib, attn_int8, gemm, kernels, model, nodes, quantizers, sp, step, te_quant, timing, vae, vae_fast  # noqa: F401

__all__ = ["_lib", "attn_int8", "gemm", "kernels", "model", "nodes", "quantizers", "sp", "step"]
