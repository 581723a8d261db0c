"""The C-ABI shared library builds, loads and exports every symbol include/rapidh3_b200.h declares.
No compute call is made here (there is no GPU on the CPU test box)."""
import ctypes

from rapid_h3_b200 import _build, _lib


def test_library_builds_and_exports_declared_symbols():
    path = _build.build()
    handle = ctypes.CDLL(path)
    declared = _lib.declared_symbols()
    assert len(declared) >= 10
    for name in declared:
        assert hasattr(handle, name), f"{name} declared in the header but not exported"


def test_signature_table_covers_the_header():
    declared = set(_lib.declared_symbols()) - {"rh3_last_error_string"}
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)


def test_argument_errors_are_reported_without_a_gpu():
    lib = _lib.lib()
    assert lib.rh3_version() >= 100
    # K not a multiple of 8 is rejected before anything touches the device
    rc = lib.rh3_quant_rows_i8(None, 8, 4, 7, None, 8, None, None)
    assert rc < 0 and b"multiple of 8" in lib.rh3_last_error_string()
    rc = lib.rh3_gemm_w8a8(None, 16, None, None, None, None, 4, 8, 16, 7, None, 8, None, None)
    assert rc < 0 and b"kind" in lib.rh3_last_error_string()


def test_argument_errors_of_the_later_entry_points():
    """Shape rules that the host side relies on are enforced by the library itself, before any CUDA call."""
    lib = _lib.lib()
    err = lib.rh3_last_error_string
    # rotated widths are whole groups of 256 channels
    assert lib.rh3_rot_quant_rows_i8(None, 384, 0, 384, None, 384, None, None) < 0 and b"256" in err()
    assert lib.rh3_swiglu_rot_quant_rows_i8(None, 1024, 0, 128, None, 128, None, None) < 0 and b"256" in err()
    # fp16 VAE quantizer: D must divide 256 and H*D be a multiple of 256
    assert lib.rh3_vae_out_quant(None, 1, 4, 8, 48, None, None, None) < 0
    assert lib.rh3_vae_quant_rows(None, 512, 4, 384, None, None, None) < 0 and b"256" in err()
    # fp16 SwiGLU GEMM: N in whole groups of 16 columns (M = 0: the null-pointer check is skipped)
    assert lib.rh3_vae_gemm_swiglu(None, 256, None, None, None, None, 0, 24, 256, None, 16, None) < 0 and b"16" in err()
    # scatter attention: 1..8 destinations
    assert lib.rh3_attn_int8_scatter(None, None, None, None, None, None, None, 256, 256, 128, 128, 1, 0.1, None, None,
                                     0, 128, 128, None) < 0 and b"n_dst" in err()
    assert lib.rh3_rope_scatter_heads(None, 1536, 4, 4, 3, 0, None, None, 1e-6, None, None, None) < 0  # 4 heads over 3 ranks
    assert lib.rh3_rot_residual_quant_rows_i8(None, 100, None, 100, None, None, 2, 100, None, None, None) < 0
    # the no-allocation statistics entry refuses what its built-in scratch cannot hold
    assert lib.rh3_attn_kv_stats_noalloc(None, 128, 128, None, 128, 128, 1 << 22, 64, None, None, None, None) < 0
