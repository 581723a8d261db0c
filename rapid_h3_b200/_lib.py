"""ctypes binding of librapidh3_b200.so (the C ABI declared in include/rapidh3_b200.h).

The library is the only compute path: if it is missing or a call fails this module raises; there
is no PyTorch or CPU fallback behind any operator of the package.
"""
import ctypes
import os
import re

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "librapidh3_b200.so")
HEADER_PATH = os.path.join(os.path.dirname(HERE), "include", "rapidh3_b200.h")

_P, _I64, _I, _F = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float

# argument types per entry point, in header order (every pointer / stream is a void*)
SIGNATURES = {
    "rh3_version": [],
    "rh3_sm_count": [],
    "rh3_check_status": [_P, _P],
    "rh3_selftest_wait_expiry": [_I64, _P, _P],
    "rh3_gemm_use_pairs": [_I],
    "rh3_selftest_mma_rate": [_I, _I64, _I, _I, _P, _P],
    "rh3_selftest_mma_feed": [_P, _I64, _I64, _I, _P, _P],
    "rh3_quant_rows_i8": [_P, _I64, _I64, _I64, _P, _I64, _P, _P],
    "rh3_quant_rows_fp8": [_P, _I64, _I64, _I64, _P, _I64, _P, _P],
    "rh3_quant_tensor_fp8": [_P, _I64, _I64, _I64, _P, _I64, _P, _P, _P],
    "rh3_swiglu_quant_rows_i8": [_P, _I64, _I64, _I64, _P, _I64, _P, _P],
    "rh3_quant_heads_i8": [_P, _I64, _I64, _I64, _P, _I64, _P, _P],
    "rh3_quant_groups_i8": [_P, _I64, _I64, _I64, _I64, _P, _I64, _P, _P],
    "rh3_norm_mod_quant_rows_i8": [_P, _I64, _P, _F, _P, _P, _P, _I64, _I64, _I64, _P, _I64, _P, _P],
    "rh3_rot_quant_rows_i8": [_P, _I64, _I64, _I64, _P, _I64, _P, _P],
    "rh3_swiglu_rot_quant_rows_i8": [_P, _I64, _I64, _I64, _P, _I64, _P, _P],
    "rh3_rot_quant_groups_i8": [_P, _I64, _I64, _I64, _I64, _P, _I64, _P, _P],
    "rh3_norm_mod_rot_quant_rows_i8": [_P, _I64, _P, _F, _P, _P, _P, _I64, _I64, _I64, _P, _I64, _P, _P],
    "rh3_rot_residual_quant_rows_i8": [_P, _I64, _P, _I64, _P, _P, _I64, _I64, _P, _P, _P],
    "rh3_rope_scatter_heads": [_P, _I64, _I64, _I64, _I64, _I64, _P, _P, _F, _P, _P, _P],
    "rh3_attn_int8_scatter": [_P, _P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _F, _P, _P, _I64, _I64, _I64, _P],
    "rh3_vae_out_quant": [_P, _I64, _I64, _I64, _I64, _P, _P, _P],
    "rh3_vae_quant_rows": [_P, _I64, _I64, _I64, _P, _P, _P],
    "rh3_vae_quant_rows_act": [_P, _I64, _I64, _I64, _I, _P, _F, _P, _P, _P],
    "rh3_vae_gemm": [_P, _I64, _P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _P, _I64, _P],
    "rh3_vae_gemm_swiglu": [_P, _I64, _P, _P, _P, _P, _I64, _I64, _I64, _P, _I64, _P],
    "rh3_gemm_w8a8": [_P, _I64, _P, _P, _P, _P, _I64, _I64, _I64, _I, _P, _I64, _P, _P],
    "rh3_gemm_w8a8_gated_residual": [_P, _I64, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I, _P],
    "rh3_gemm_w8a8_swiglu": [_P, _I64, _P, _P, _P, _I64, _I64, _I64, _I, _P, _I64, _P],
    "rh3_rmsnorm_rope3d": [_P, _I64, _I64, _P, _I64, _I64, _I64, _I64, _P, _F, _P, _P],
    "rh3_attn_kv_stats_scratch_bytes": [_I64, _I64],
    "rh3_attn_kv_stats": [_P, _I64, _I64, _P, _I64, _I64, _I64, _I64, _P, _I64, _P, _P, _P, _P],
    "rh3_attn_kv_stats_noalloc": [_P, _I64, _I64, _P, _I64, _I64, _I64, _I64, _P, _P, _P, _P],
    "rh3_attn_prepass": [_P, _I64, _I64, _I64, _I64, _P, _I64, _I64, _P, _I64, _I64, _I64, _I64, _I64, _P, _P, _F, _P, _P,
                         _I64, _I64, _P, _I64, _I64, _P, _I64, _P, _P, _P, _P, _P, _P, _P, _P, _P],
    "rh3_attn_tok_prepass": [_P, _I64, _I64, _I64, _I64, _P, _I64, _I64, _P, _I64, _I64, _I64, _I64, _I64, _P, _P, _F, _P, _P,
                         _I64, _I64, _P, _I64, _I64, _P, _I64, _P, _P, _P, _P, _P, _P, _P, _P, _P],
    "rh3_attn_int8_tok": [_P, _P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _F, _P, _I64, _I64, _P],
    "rh3_attn_quant_qk": [_P, _I64, _I64, _I64, _I64, _I64, _P, _P, _P, _P],
    "rh3_attn_quant_v": [_P, _I64, _I64, _I64, _I64, _I64, _P, _P, _P, _P],
    "rh3_attn_int8": [_P, _P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _F, _P, _I64, _I64, _P],
    "rh3_attn_int8_dump_scores": [_P, _P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _F, _P, _I64, _I64, _I64, _I64,
                                  _I64, _P, _P],
    "rh3_depth_to_space8": [_P, _P, _I64, _I64, _I64, _I64, _P],
    "rh3_conv3d_causal": [_P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _P],
    "rh3_conv3d_gn_part_rows": [_I64, _I64, _I64, _I64],
    "rh3_gn_reduce": [_P, _I64, _I64, _P, _P],
    "rh3_gn_silu_apply": [_P, _P, _P, _P, _I64, _I64, _I64, _P, _P],
    "rh3_upsample_causal2x": [_P, _P, _I64, _I64, _I64, _I64, _I64, _P],
}
# entry points that return a value instead of a status
RETURNS_I64 = ("rh3_attn_kv_stats_scratch_bytes", "rh3_conv3d_gn_part_rows")

KIND_I8, KIND_F8 = 0, 1

_lib = None

# kernels launched per entry point (for launch accounting in benchmarks)
LAUNCHES = {"rh3_attn_kv_stats": 2, "rh3_attn_kv_stats_noalloc": 2, "rh3_attn_prepass": 3, "rh3_attn_tok_prepass": 5, "rh3_quant_tensor_fp8": 2, "rh3_version": 0, "rh3_gemm_use_pairs": 0, "rh3_sm_count": 0, "rh3_check_status": 0,
            "rh3_attn_kv_stats_scratch_bytes": 0, "rh3_conv3d_gn_part_rows": 0}
launch_count = 0


def declared_symbols():
    """Names of the functions include/rapidh3_b200.h declares."""
    text = open(HEADER_PATH).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rh3_[a-z0-9_]+)\s*\(", text)))


def lib():
    """The loaded shared library (loads it on first use; raises if it has not been built)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m rapid_h3_b200._build` (needs nvcc). "
                "rapid_h3_b200 has no fallback path.")
        handle = ctypes.CDLL(LIB_PATH)
        handle.rh3_last_error_string.restype = ctypes.c_char_p
        handle.rh3_last_error_string.argtypes = []
        for name, args in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = ctypes.c_int64 if name in RETURNS_I64 else ctypes.c_int
            fn.argtypes = args
        _lib = handle
    return _lib


def last_error():
    return lib().rh3_last_error_string().decode()


def ptr(t):
    """Device pointer of a tensor (None -> NULL)."""
    return None if t is None else t.data_ptr()


def stream():
    return torch.cuda.current_stream().cuda_stream


def call(name, *args):
    """Invoke an entry point; a non-zero return raises RuntimeError with the library's message."""
    global launch_count
    rc = getattr(lib(), name)(*args)
    launch_count += LAUNCHES.get(name, 1)
    if rc != 0:
        raise RuntimeError(f"{name} failed ({rc}): {last_error()}")


def check_status():
    """Synchronise the current stream and raise if a bounded device-side wait gave up."""
    st = ctypes.c_int(0)
    call("rh3_check_status", stream(), ctypes.addressof(st))
    if st.value != 0:
        raise RuntimeError(f"device status {st.value}: {last_error()}")


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("rapid_h3_b200 operators need CUDA tensors; there is no CPU path")
