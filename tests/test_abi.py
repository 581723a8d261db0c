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
